"""Parity of the decode-attention kernels with the oracle, through the C ABI, on a B200.

Tolerance: 2e-3 relative (max|o - o_ref| / max|o_ref|) against the order-faithful oracle; the
kernels split the context across warps and partitions, so their summation order differs from the
reference's.  Addressing differentials (paged == gathered-contiguous, batched == one at a time)
are bit-for-bit between our own variants, as the reference's are between its own."""
import numpy as np
import pytest
import torch

import oracle as orc
from accel_b200 import tensor as T
from util import ATTN_TOL, assert_close, attn_scale, normal, paged_fixture

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a):
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).to(DEV)
    return torch.from_numpy(a).to(DEV)


def bits(a):
    return a.view(np.uint16) if a.dtype == np.float16 else a


def test_reference_fixtures_on_the_device():
    # internal/kernels/paged_test.go:28-110: four page tables, one answer; and the device's answer
    # is the oracle's within tolerance
    qH, kvH, D, B, L = 4, 2, 8, 4, 10
    q = np.sin(np.arange(qH * D) * 0.31).astype(np.float32).reshape(qH, D)
    i = np.arange(L * kvH * D)
    lk = np.cos(i * 0.17).astype(np.float32).reshape(L, kvH, D)
    lv = ((i % 9) - 4).astype(np.float32).reshape(L, kvH, D)
    lengths = np.array([L], np.uint32)
    want = orc.attention_decode(q, lk, lv, lengths, qH, kvH, D, attn_scale(D)).reshape(qH, D)
    cont = T.attention(dev(q), dev(lk), dev(lv),
                       T.AttentionOptions(lengths=dev(lengths), scale=attn_scale(D))).cpu().numpy()
    assert_close(cont, want, ATTN_TOL, "contiguous")
    for pages in ([0, 1, 2], [5, 4, 3], [7, 2, 5], [9, 0, 4]):
        pk = np.zeros((12 * B, kvH, D), np.float32)
        pv = np.zeros_like(pk)
        for j in range(L):
            phys = pages[j // B] * B + j % B
            pk[phys], pv[phys] = lk[j], lv[j]
        got = T.attention(dev(q), dev(pk), dev(pv),
                          T.AttentionOptions(lengths=dev(lengths), pages=dev(np.array(pages, np.uint32)),
                                             block=B, scale=attn_scale(D))).cpu().numpy()
        assert np.array_equal(got, cont), pages      # paging changes addressing, not arithmetic


def test_batched_equals_one_at_a_time_and_the_oracle():
    # internal/kernels/batched_test.go:29-104
    batch, qH, kvH, D, B, MP, blocks = 3, 2, 1, 8, 4, 3, 12
    lengths = np.array([9, 3, 6], np.uint32)
    pages = np.array([[0, 3, 6], [1, 0, 0], [4, 7, 0]], np.uint32)
    i = np.arange(blocks * B * kvH * D)
    pk = np.sin(i * 0.13).astype(np.float32).reshape(-1, kvH, D)
    pv = np.cos(i * 0.21).astype(np.float32).reshape(-1, kvH, D)
    q = np.sin(np.arange(batch * qH * D) * 0.37).astype(np.float32).reshape(batch, 1, qH, D)
    sc = attn_scale(D)
    got = T.attention(dev(q), dev(pk), dev(pv),
                      T.AttentionOptions(lengths=dev(lengths), pages=dev(pages), block=B, scale=sc)).cpu().numpy()
    want = orc.attention_decode_batched(q, pk, pv, pages, lengths, batch, qH, kvH, D, B, MP, sc)
    assert_close(got, want.reshape(batch, qH, D), ATTN_TOL, "batched")
    for s in range(batch):
        alone = T.attention(dev(q[s, 0]), dev(pk), dev(pv),
                            T.AttentionOptions(lengths=dev(lengths[s:s + 1]), pages=dev(pages[s]),
                                               block=B, scale=sc)).cpu().numpy()
        assert np.array_equal(got[s], alone)


def test_a_length_past_the_page_table_is_truncated():
    # internal/kernels/batched_test.go:171-234
    batch, qH, kvH, D, B, MP, pool = 2, 2, 1, 8, 4, 2, 8
    reach = MP * B
    q = np.sin(np.arange(batch * qH * D) * 0.4).astype(np.float32).reshape(batch, 1, qH, D)
    i = np.arange(pool * B * kvH * D)
    pk = np.cos(i * 0.13).astype(np.float32).reshape(-1, kvH, D)
    pv = (i // (B * kvH * D)).astype(np.float32).reshape(-1, kvH, D)
    pages = np.array([[0, 1], [4, 5]], np.uint32)
    run = lambda lens: T.attention(dev(q), dev(pk), dev(pv), T.AttentionOptions(
        lengths=dev(np.array(lens, np.uint32)), pages=dev(pages), block=B, scale=attn_scale(D))).cpu().numpy()
    over, exact = run([reach + 5, reach]), run([reach, reach])
    assert np.array_equal(over, exact) and not np.any(np.isnan(over))
    want = orc.attention_decode_batched(q, pk, pv, pages, [reach + 5, reach], batch, qH, kvH, D, B, MP, attn_scale(D))
    assert_close(over, want.reshape(batch, qH, D), ATTN_TOL, "truncated")


@pytest.mark.parametrize("f16", [False, True])
@pytest.mark.parametrize("qH,kvH,D,block", [(32, 8, 128, 16), (32, 32, 128, 16), (8, 4, 64, 8),
                                            (6, 2, 40, 4), (16, 2, 128, 32), (4, 4, 8, 1), (8, 4, 128, 16),
                                            (6, 2, 128, 8)])
def test_batched_matches_the_oracle(qH, kvH, D, block, f16):
    batch = 5
    rng = np.random.default_rng(qH * 1000 + D)
    lengths = np.array([1, 255, 256, 257, int(rng.integers(300, 700))], np.uint32)
    k, v, pages, mp = paged_fixture(3, batch, kvH, D, block, lengths, f16=f16)
    q = normal(4, (batch, 1, qH, D))
    sc = attn_scale(D)
    want = orc.attention_decode_batched(q, bits(k), bits(v), pages, lengths, batch, qH, kvH, D,
                                        block, mp, sc).reshape(batch, qH, D)
    got = T.attention(dev(q), dev(k), dev(v), T.AttentionOptions(
        lengths=dev(lengths), pages=dev(pages), block=block, scale=sc)).cpu().numpy()
    assert_close(got, want, ATTN_TOL, f"batched qH={qH} kvH={kvH} D={D} f16={f16}")
    # single-sequence paged kernel on each row, f32 and f16 (paged.go:47,362)
    for s in (1, 4):
        alone = T.attention(dev(q[s, 0]), dev(k), dev(v), T.AttentionOptions(
            lengths=dev(lengths[s:s + 1]), pages=dev(pages[s]), block=block, scale=sc)).cpu().numpy()
        w1 = orc.attention_decode_paged(q[s, 0], bits(k), bits(v), pages[s], lengths[s:s + 1], qH,
                                        kvH, D, block, sc).reshape(qH, D)
        assert_close(alone, w1, ATTN_TOL, "paged single")


def test_config3_shape_against_the_oracle():
    # 32 sequences, 32 query / 8 KV heads, D=128, block 16, context uniform in [512, 4096]
    batch, qH, kvH, D, block = 32, 32, 8, 128, 16
    rng = np.random.default_rng(3)
    lengths = rng.integers(512, 4097, batch).astype(np.uint32)
    k, v, pages, mp = paged_fixture(3, batch, kvH, D, block, lengths, max_pages=256)
    q = normal(4, (batch, 1, qH, D))
    sc = attn_scale(D)
    got = T.attention(dev(q), dev(k), dev(v), T.AttentionOptions(
        lengths=dev(lengths), pages=dev(pages), block=block, scale=sc)).cpu().numpy()
    want = orc.attention_decode_batched(q, k, v, pages, lengths, batch, qH, kvH, D, block, mp,
                                        sc).reshape(batch, qH, D)
    assert_close(got, want, ATTN_TOL, "config 3")
    # size-independent property: every output row lies inside the convex hull of V per dimension
    # (softmax weights are a convex combination), checked for the longest sequence
    s = int(np.argmax(lengths))
    rows = np.array([pages[s, j // block] * block + j % block for j in range(lengths[s])])
    for h in (0, qH - 1):
        vv = v[rows, h // (qH // kvH)]
        assert np.all(got[s, h] <= vv.max(0) + 1e-5) and np.all(got[s, h] >= vv.min(0) - 1e-5)


@pytest.mark.parametrize("qH,kvH", [(4, 4), (8, 2)])
def test_a_nan_score_poisons_its_head_and_no_other(qH, kvH):
    """kmath.Max propagates a NaN (kmath/kmath.go:96-104), so in the reference a NaN score makes the
    running maximum, and with it every weight of that (sequence, query head), NaN.  These kernels
    keep the maximum with fmaxf (which drops a NaN) but the NaN score still enters the sum of
    weights and the output, so the outcome is the same: the oracle (which follows kmath.Max) and the
    device give NaN on exactly the same heads and agree elsewhere."""
    batch, D, block = 3, 32, 8
    lengths = np.array([300, 40, 9], np.uint32)
    k, v, pages, mp = paged_fixture(7, batch, kvH, D, block, lengths)
    q = normal(8, (batch, 1, qH, D))
    # one K element of sequence 1, position 17, KV head 0: NaN for the query heads that read that head
    row = pages[1, 17 // block] * block + 17 % block
    k[row, 0, 3] = np.nan
    sc = attn_scale(D)
    got = T.attention(dev(q), dev(k), dev(v), T.AttentionOptions(
        lengths=dev(lengths), pages=dev(pages), block=block, scale=sc)).cpu().numpy()
    want = orc.attention_decode_batched(q, k, v, pages, lengths, batch, qH, kvH, D, block, mp,
                                        sc).reshape(batch, qH, D)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    group = qH // kvH
    assert np.all(np.isnan(got[1, :group])) and not np.any(np.isnan(got[1, group:]))
    assert not np.any(np.isnan(got[0])) and not np.any(np.isnan(got[2]))
    ok = ~np.isnan(want)
    assert_close(got[ok], want[ok], ATTN_TOL, "the heads beside the poisoned one")


def test_zero_length_is_nan_as_in_the_reference():
    # internal/kernels/batched.go:104,347-349: l = 0, out = 0/0
    batch, qH, kvH, D, block = 2, 4, 2, 16, 4
    lengths = np.array([0, 5], np.uint32)
    k, v, pages, mp = paged_fixture(1, batch, kvH, D, block, [4, 5])
    q = normal(2, (batch, 1, qH, D))
    got = T.attention(dev(q), dev(k), dev(v), T.AttentionOptions(
        lengths=dev(lengths), pages=dev(pages), block=block, scale=1.0)).cpu().numpy()
    want = orc.attention_decode_batched(q, k, v, pages, lengths, batch, qH, kvH, D, block, mp, 1.0)
    assert np.all(np.isnan(got[0])) and np.all(np.isnan(want.reshape(batch, qH, D)[0]))
    assert_close(got[1], want.reshape(batch, qH, D)[1], ATTN_TOL, "row beside an empty one")


@pytest.mark.parametrize("f16", [False, True])
@pytest.mark.parametrize("qH,kvH,D", [(8, 2, 64), (8, 2, 128), (4, 2, 128)])
def test_ragged_matches_the_oracle(qH, kvH, D, f16):
    # internal/kernels/ragged.go:61-241: a prefill chunk, three decodes, an empty row, padding
    # (head dimension 128 with grouped heads runs on the tensor cores)
    block, MP = 8, 80
    extents = np.array([37, 1, 0, 1, 1], np.uint32)
    lengths = np.array([300, 77, 9, 1, 600], np.uint32)
    batch = extents.size
    k, v, pages, mp = paged_fixture(5, batch, kvH, D, block, lengths, max_pages=MP, f16=f16)
    tokens = int(extents.sum()) + 2                      # two padding tokens
    q = normal(6, (tokens, qH, D))
    sc = attn_scale(D)
    off = orc.segment_offsets(extents)
    want = orc.attention_ragged(q, bits(k), bits(v), pages, lengths, off, tokens, batch, qH, kvH,
                                D, block, mp, sc).reshape(tokens, qH, D)
    got = T.attention(dev(q), dev(k), dev(v), T.AttentionOptions(
        lengths=dev(lengths), pages=dev(pages), block=block, scale=sc,
        query_extents=dev(extents))).cpu().numpy()
    assert np.all(got[-2:] == 0) and np.all(want[-2:] == 0)
    assert_close(got, want, ATTN_TOL, f"ragged f16={f16}")
    # a sequence shorter than its count: tokens with no position write zero
    lengths2 = lengths.copy()
    lengths2[0] = 30
    got2 = T.attention(dev(q), dev(k), dev(v), T.AttentionOptions(
        lengths=dev(lengths2), pages=dev(pages), block=block, scale=sc,
        query_extents=dev(extents))).cpu().numpy()
    want2 = orc.attention_ragged(q, bits(k), bits(v), pages, lengths2, off, tokens, batch, qH, kvH,
                                 D, block, mp, sc).reshape(tokens, qH, D)
    assert np.all(got2[:7] == 0)
    assert_close(got2, want2, ATTN_TOL, "ragged, short sequence")


def test_ragged_with_unit_extents_equals_the_batched_kernel_bit_for_bit():
    batch, qH, kvH, D, block = 6, 8, 2, 128, 16
    lengths = np.array([5, 130, 256, 700, 1, 999], np.uint32)
    k, v, pages, mp = paged_fixture(8, batch, kvH, D, block, lengths)
    q = normal(9, (batch, qH, D))
    sc = attn_scale(D)
    opts = dict(lengths=dev(lengths), pages=dev(pages), block=block, scale=sc)
    b = T.attention(dev(q.reshape(batch, 1, qH, D)), dev(k), dev(v), T.AttentionOptions(**opts)).cpu().numpy()
    r = T.attention(dev(q), dev(k), dev(v), T.AttentionOptions(
        query_extents=dev(np.ones(batch, np.uint32)), **opts)).cpu().numpy()
    assert np.array_equal(b, r)


def test_refusals():
    qH, kvH, D = 4, 2, 8
    q = torch.zeros(qH, D, device=DEV)
    k = torch.zeros(16, kvH, D, device=DEV)
    L = torch.ones(1, dtype=torch.int32, device=DEV)
    with pytest.raises(T.Refused, match="f32 query"):
        T.attention(q.half(), k, k, T.AttentionOptions(lengths=L))
    with pytest.raises(T.Refused, match="same dtype"):
        T.attention(q, k, k.half(), T.AttentionOptions(lengths=L))
    with pytest.raises(T.Refused, match="Lengths is required"):
        T.attention(q, k, k, T.AttentionOptions())
    with pytest.raises(T.Refused, match="multiple of the second"):
        T.attention(torch.zeros(3, D, device=DEV), k, k, T.AttentionOptions(lengths=L))
    with pytest.raises(T.Refused, match="wide"):
        T.attention(torch.zeros(qH, 16, device=DEV), k, k, T.AttentionOptions(lengths=L))
    with pytest.raises(T.Refused, match="Block is 0"):
        T.attention(q, k, k, T.AttentionOptions(lengths=L, pages=torch.zeros(4, dtype=torch.int32, device=DEV)))
    with pytest.raises(T.Refused, match="needs Pages"):
        T.attention(torch.zeros(2, 1, qH, D, device=DEV), k, k,
                    T.AttentionOptions(lengths=torch.ones(2, dtype=torch.int32, device=DEV)))
    with pytest.raises(T.Refused, match="one length per sequence"):
        T.attention(torch.zeros(2, 1, qH, D, device=DEV), k, k, T.AttentionOptions(
            lengths=L, pages=torch.zeros(2, 4, dtype=torch.int32, device=DEV), block=4))
    with pytest.raises(T.Refused, match="one token per sequence"):
        T.attention(torch.zeros(2, 3, qH, D, device=DEV), k, k, T.AttentionOptions(
            lengths=torch.ones(2, dtype=torch.int32, device=DEV),
            pages=torch.zeros(2, 4, dtype=torch.int32, device=DEV), block=4))


@pytest.mark.parametrize("f16", [False, True])
@pytest.mark.parametrize("qH,kvH,D,block,lengths", [
    (32, 32, 128, 16, [1, 300, 2048, 700]),        # several partitions: the combine kernel writes out
    (32, 8, 128, 16, [5, 900, 64, 1500]),          # grouped heads
    (8, 4, 64, 8, [3, 17, 40, 9]),                 # one partition: the partition kernels write out
    (6, 2, 40, 4, [1, 30, 0, 12]),                 # a head dimension that leaves lanes idle; a zero length (NaN)
])
def test_batched_with_the_rows_maxima(qH, kvH, D, block, lengths, f16):
    """AttentionDecodeBatched(F16)Max: out is bit-identical to the plain kernel's, and outmax
    [Batch][QHeads][4] holds, per head, maxima whose largest is the largest |out| of the head (NaN
    counts as the largest), for the int4 product that reads out next."""
    from accel_b200 import runtime as rt
    import struct
    lengths = np.array(lengths, np.uint32)
    batch = len(lengths)
    k, v, pages, mp = paged_fixture(7, batch, kvH, D, block, np.maximum(lengths, 1), f16=f16)
    q = normal(8, (batch, 1, qH, D))
    u = struct.pack("<IIIIIIfI", batch, qH, kvH, D, block, mp, attn_scale(D), 0)
    b = [dev(q), dev(k), dev(v), dev(pages.reshape(-1)), dev(lengths)]
    o0 = torch.full((batch, qH, D), float("nan"), device=DEV)
    o1 = torch.full((batch, qH, D), float("nan"), device=DEV)
    mx = torch.full((batch, qH, 4), float("nan"), device=DEV)
    name = "AttentionDecodeBatchedF16" if f16 else "AttentionDecodeBatched"
    rt.launch(name, b + [o0], u)
    rt.launch(name + "Max", b + [o1, mx], u)
    torch.cuda.synchronize()
    assert torch.equal(o0.view(torch.int32), o1.view(torch.int32))
    # compare magnitudes by their bit patterns: a NaN is the largest
    want = o1.abs().view(torch.int32).amax(dim=2)
    got = mx.abs().view(torch.int32).amax(dim=2)
    assert torch.equal(got, want)
