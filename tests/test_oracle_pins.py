"""Pins the CPU oracle against every known-answer fixture the reference's own tests hold for the
path.  The reference commits no numeric output vectors; its tests are deterministic fixtures with
exact assertions (codes, words, reconstructed constants, page lists) and bit-for-bit differentials
between kernels, and each is replayed here.  File:line citations are to the accel module."""
import math

import numpy as np
import pytest

import oracle as orc

G = 128


# ----------------------------------------------------------------------------- f16 conversion
def test_f16_conversion_matches_ieee_except_the_flushed_interval():
    # internal/kernel/narrow.go:67-105: RNE, overflow to inf, canonical NaN, signed zero, and
    # every value below 2^-24 flushed to zero (IEEE would round (2^-25, 2^-24) up).
    xs = np.array([0.0, -0.0, 1.0, -2.5, 65504.0, 65520.0, 1e9, 1.9997, 6.1e-5, 5.96e-8,
                   3.1e-8, 2.9e-8, 1e-10, 0.1, 0.3333333, np.inf, -np.inf], np.float32)
    got = orc.to_f16_bits(xs)
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16).copy()
    tiny = (np.abs(xs) < 2.0 ** -24) & (xs != 0)
    want[tiny] = (np.signbit(xs[tiny]).astype(np.uint16) << 15)
    assert np.array_equal(got, want)
    assert orc.to_f16_bits([np.nan])[0] == 0x7e00
    # every finite f16 widens and narrows back to itself
    allh = np.arange(0, 0x7c00, dtype=np.uint16)
    assert np.array_equal(orc.to_f16_bits(orc.from_f16_bits(allh)), allh)
    assert np.array_equal(orc.from_f16_bits(allh), allh.view(np.float16).astype(np.float32))


def test_f16_conversion_random_sweep(rng):
    x = (rng.standard_normal(200000) * np.exp(rng.uniform(-12, 12, 200000))).astype(np.float32)
    got = orc.to_f16_bits(x)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16).copy()
    tiny = np.abs(x) < 2.0 ** -24
    want[tiny] = (np.signbit(x[tiny]).astype(np.uint16) << 15)
    assert np.array_equal(got, want)


# ----------------------------------------------------------------------------- quantizer KATs
@pytest.mark.parametrize("c", [0.0, 1.0, -2.5, 0.125])
def test_constant_group_reconstructs_exactly(c):
    # quant/int4_test.go:22-36
    w = np.full(G, c, np.float32)
    p, s, z = orc.int4_quantize(w)
    assert orc.from_f16_bits(s)[0] == 0
    assert np.all(orc.int4_dequantize(p, s, z, G) == np.float32(c))


def test_packs_low_nibble_first():
    # quant/int4_test.go:261-286
    w = np.full(G, 0.5, np.float32)
    w[0], w[1] = 0, 10
    p, _, _ = orc.int4_quantize(w)
    assert orc.int4_nibble(p, 0) == 0
    assert orc.int4_nibble(p, 1) == 15
    assert int(p[0]) & 0xFF == 0xF0


def test_packing_round_trips_at_an_odd_length():
    # quant/int4_test.go:225-253
    w = (np.arange(G + 1) % 16).astype(np.float32) / 4
    p, s, z = orc.int4_quantize(w)
    assert p.size == (w.size + 7) // 8 == 17
    back = orc.int4_dequantize(p, s, z, w.size)
    assert back.size == w.size and back[-1] == w[-1]
    assert int(p[-1]) >> 4 == 0          # the last word's high nibbles stay zero


@pytest.mark.parametrize("lo,hi", [(-1, 1), (0.9, 1.0), (-3, -2.75), (-0.25, 4), (1000, 1001),
                                   (-2000, -1999)])
def test_reconstruction_is_inside_the_derived_bound(lo, hi, rng):
    # quant/int4_test.go:46-90 with a generator of our own (the reference's PCG stream is not
    # reproduced; the assertion is an inequality that holds for any weights in the span)
    w = rng.uniform(lo, hi, 3 * G + 17).astype(np.float32)
    p, s, z = orc.int4_quantize(w)
    back = orc.int4_dequantize(p, s, z, w.size)
    one = np.ones(1, np.float32)
    for i in range(w.size):
        g = i // G
        bound = orc.int4_error_bound(one, s[g:g + 1], z[g:g + 1])
        assert abs(float(back[i]) - float(w[i])) <= bound * (1 + 1e-12), (i, back[i], w[i], bound)


def test_quantizer_against_a_direct_numpy_statement(rng):
    # quant/int4.go:71-138 written a second time, independently, with numpy's own f16
    w = (rng.standard_normal(8 * G) * 0.02).astype(np.float32)
    p, s, z = orc.int4_quantize(w)
    for g in range(8):
        grp = w[g * G:(g + 1) * G]
        lo, hi = grp.min(), grp.max()
        s16 = np.float32(np.float16((hi - lo) / np.float32(15)))
        z16 = np.float32(np.float16(-lo / s16))
        q = np.clip(np.rint(grp.astype(np.float64) / np.float64(s16) + np.float64(z16)), 0, 15)
        codes = [orc.int4_nibble(p, g * G + i) for i in range(G)]
        assert np.array_equal(np.array(codes), q.astype(np.int64))
        assert orc.from_f16_bits(s[g:g + 1])[0] == s16 and orc.from_f16_bits(z[g:g + 1])[0] == z16


# ----------------------------------------------------------------------------- int4 kernels
def test_kernel_agrees_about_which_nibble_is_which():
    # internal/kernels/int4_test.go:189-228: 40, not 4
    K, N = 8, 1
    w = np.ones(K * N, np.float32)
    w[0], w[1] = 0, 4
    a = np.zeros(K, np.float32)
    a[0], a[1] = 1, 10
    p, s, z = orc.int4_quantize(w)
    out = orc.quant_matvec_int4(a, p, s, z, N, K)
    assert abs(out[0] - 40.0) <= 1 and abs(out[0] - 4.0) > abs(out[0] - 40.0)


def test_kernels_read_a_constant_group_as_the_quantizer_wrote_it(rng):
    # internal/kernels/int4_test.go:99-182
    K, N, M = 2 * G, 2, 3
    w = np.empty(K * N, np.float32)
    w[:G] = 0.75
    w[G:] = rng.uniform(-1, 1, K * N - G).astype(np.float32)
    p, s, z = orc.int4_quantize(w)
    assert orc.from_f16_bits(s)[0] == 0 and orc.from_f16_bits(z)[0] == 0.75
    back = orc.int4_dequantize(p, s, z, w.size)
    a = np.ones((M, K), np.float32)
    want, mag = orc.matmul_definition_f64(a, back, M, N, K)
    row = orc.quant_matvec_int4(a[0], p, s, z, N, K)
    tiled = orc.quant_matmul_int4(a, p, s, z, M, N, K)
    nu = (K - 1) * 2.0 ** -24
    gamma = nu / (1 - nu)
    assert np.all(np.abs(row - want[0]) <= gamma * mag[0])
    assert np.all(np.abs(tiled - want) <= gamma * mag)


@pytest.mark.parametrize("M,K,N", [(1, 64, 128), (3, 50, 37), (9, 130, 19), (8, 16, 16)])
def test_matmul_matches_definition_at_odd_shapes(M, K, N, rng):
    # internal/kernels/int4_test.go:291-306: shapes that are not multiples of the tiles, where
    # groups straddle rows and the last word is partial
    w = (rng.standard_normal(K * N)).astype(np.float32)
    a = rng.standard_normal((M, K)).astype(np.float32)
    p, s, z = orc.int4_quantize(w)
    back = orc.int4_dequantize(p, s, z, w.size)
    want, mag = orc.matmul_definition_f64(a, back, M, N, K)
    tiled = orc.quant_matmul_int4(a, p, s, z, M, N, K)
    nu = (K - 1) * 2.0 ** -24
    assert np.all(np.abs(tiled - want) <= nu / (1 - nu) * mag + 1e-30)
    for m in range(M):
        row = orc.quant_matvec_int4(a[m], p, s, z, N, K)
        assert np.all(np.abs(row - want[m]) <= nu / (1 - nu) * mag[m] + 1e-30)


# ----------------------------------------------------------------------------- attention
def _scale(d):
    return float(np.float32(1) / np.float32(math.sqrt(d)))


def test_paged_decode_matches_contiguous_bit_for_bit():
    # internal/kernels/paged_test.go:28-110
    qH, kvH, D, B, L = 4, 2, 8, 4, 10
    q = np.sin(np.arange(qH * D) * 0.31).astype(np.float32)
    i = np.arange(L * kvH * D)
    lk = np.cos(i * 0.17).astype(np.float32)
    lv = ((i % 9) - 4).astype(np.float32)
    contiguous = orc.attention_decode(q, lk, lv, [L], qH, kvH, D, _scale(D))
    assert not np.any(np.isnan(contiguous))
    for pages in ([0, 1, 2], [5, 4, 3], [7, 2, 5], [9, 0, 4]):
        pk = np.zeros(12 * B * kvH * D, np.float32)
        pv = np.zeros_like(pk)
        w = kvH * D
        for j in range(L):
            phys = pages[j // B] * B + j % B
            pk[phys * w:(phys + 1) * w] = lk[j * w:(j + 1) * w]
            pv[phys * w:(phys + 1) * w] = lv[j * w:(j + 1) * w]
        paged = orc.attention_decode_paged(q, pk, pv, pages, [L], qH, kvH, D, B, _scale(D))
        assert np.array_equal(paged, contiguous), pages


def test_two_sequences_share_a_pool_without_seeing_each_other():
    # internal/kernels/paged_test.go:118-185
    qH, kvH, D, B, blocks = 2, 1, 8, 4, 8
    pk = np.zeros(blocks * B * kvH * D, np.float32)
    pv = np.zeros_like(pk)
    seqs = [([0, 2], 6, 1.0), ([1, 3], 5, -1.0)]
    for pages, n, fill in seqs:
        for j in range(n):
            phys = pages[j // B] * B + j % B
            pk[phys * D:(phys + 1) * D] = fill * (j + 1)
            pv[phys * D:(phys + 1) * D] = fill * (j + 1)
    q = np.full(qH * D, 0.1, np.float32)
    for pages, n, fill in seqs:
        out = orc.attention_decode_paged(q, pk, pv, pages, [n], qH, kvH, D, B, _scale(D))
        assert np.all(out * fill > 0)


def test_batched_decode_matches_one_at_a_time_bit_for_bit():
    # internal/kernels/batched_test.go:29-104
    batch, qH, kvH, D, B, MP, blocks = 3, 2, 1, 8, 4, 3, 12
    lengths = [9, 3, 6]
    pages = [0, 3, 6, 1, 0, 0, 4, 7, 0]
    i = np.arange(blocks * B * kvH * D)
    pk = np.sin(i * 0.13).astype(np.float32)
    pv = np.cos(i * 0.21).astype(np.float32)
    q = np.sin(np.arange(batch * qH * D) * 0.37).astype(np.float32)
    got = orc.attention_decode_batched(q, pk, pv, pages, lengths, batch, qH, kvH, D, B, MP,
                                       _scale(D))
    for s in range(batch):
        alone = orc.attention_decode_paged(q[s * qH * D:(s + 1) * qH * D], pk, pv,
                                           pages[s * MP:(s + 1) * MP], lengths[s:s + 1], qH, kvH,
                                           D, B, _scale(D))
        assert np.array_equal(got[s * qH * D:(s + 1) * qH * D], alone)


def test_batch_of_one_is_the_unbatched_kernel():
    # internal/kernels/batched_test.go:108-155
    qH, kvH, D, B, MP, blocks = 2, 1, 8, 4, 2, 6
    i = np.arange(blocks * B * kvH * D)
    pk = ((i % 11) - 5).astype(np.float32)
    pv = ((i % 7) - 3).astype(np.float32)
    q = np.sin(np.arange(qH * D) * 0.4).astype(np.float32)
    one = orc.attention_decode_batched(q, pk, pv, [3, 1], [5], 1, qH, kvH, D, B, MP, _scale(D))
    un = orc.attention_decode_paged(q, pk, pv, [3, 1], [5], qH, kvH, D, B, _scale(D))
    assert np.array_equal(one, un)


def test_a_batched_length_past_its_page_table_is_truncated():
    # internal/kernels/batched_test.go:171-234
    batch, qH, kvH, D, B, MP, pool = 2, 2, 1, 8, 4, 2, 8
    reach = MP * B
    q = np.sin(np.arange(batch * qH * D) * 0.4).astype(np.float32)
    i = np.arange(pool * B * kvH * D)
    pk = np.cos(i * 0.13).astype(np.float32)
    pv = (i // (B * kvH * D)).astype(np.float32)
    pages = [0, 1, 4, 5]
    sc = float(np.float32(1 / math.sqrt(D)))
    over = orc.attention_decode_batched(q, pk, pv, pages, [reach + 5, reach], batch, qH, kvH, D,
                                        B, MP, sc)
    exact = orc.attention_decode_batched(q, pk, pv, pages, [reach, reach], batch, qH, kvH, D, B,
                                         MP, sc)
    assert np.array_equal(over, exact)
    assert not np.any(np.isnan(over)) and not (over[0] == 0 and over[1] == 0)


def test_decode_agrees_with_the_f64_definition_over_several_blocks(rng):
    # internal/kernels/attention_test.go:29-110 and paged_test.go:190-267: a cache longer than one
    # 128-position block, against the composed definition
    qH, kvH, D, B = 4, 2, 16, 4
    L = 300
    npages = (L + B - 1) // B
    pages = rng.permutation(npages + 5)[:npages].astype(np.uint32)
    cap = (npages + 5) * B
    pk = rng.standard_normal(cap * kvH * D).astype(np.float32)
    pv = rng.standard_normal(cap * kvH * D).astype(np.float32)
    q = rng.standard_normal(qH * D).astype(np.float32)
    got = orc.attention_decode_paged(q, pk, pv, pages, [L], qH, kvH, D, B, _scale(D))
    rows = np.array([pages[j // B] * B + j % B for j in range(L)], np.uint32)
    want = orc.attention_definition_f64(q, pk, pv, rows, qH, kvH, D, _scale(D))
    assert np.max(np.abs(got - want)) < 2e-6 * max(1.0, np.max(np.abs(want)))
    # and the f16-cache kernel reads the same values widened
    hk, hv = orc.to_f16_bits(pk), orc.to_f16_bits(pv)
    got16 = orc.attention_decode_paged(q, hk, hv, pages, [L], qH, kvH, D, B, _scale(D))
    wide = orc.attention_decode_paged(q, orc.from_f16_bits(hk), orc.from_f16_bits(hv), pages, [L],
                                      qH, kvH, D, B, _scale(D))
    assert np.array_equal(got16, wide)


def test_ragged_with_unit_extents_is_a_batched_decode(rng):
    # internal/kernels/ragged.go:61-241: extents of one make each token a decode step; the
    # summation order differs from the batched kernel, so the comparison carries a tolerance
    batch, qH, kvH, D, B, MP = 3, 4, 2, 8, 4, 5
    lengths = np.array([17, 1, 9], np.uint32)
    pages = rng.permutation(batch * MP).astype(np.uint32)
    cap = batch * MP * B
    pk = rng.standard_normal(cap * kvH * D).astype(np.float32)
    pv = rng.standard_normal(cap * kvH * D).astype(np.float32)
    q = rng.standard_normal(batch * qH * D).astype(np.float32)
    off = np.arange(batch + 1, dtype=np.uint32)
    r = orc.attention_ragged(q, pk, pv, pages, lengths, off, batch, batch, qH, kvH, D, B, MP,
                             _scale(D))
    b = orc.attention_decode_batched(q, pk, pv, pages, lengths, batch, qH, kvH, D, B, MP,
                                     _scale(D))
    assert np.allclose(r, b, rtol=0, atol=1e-5)
    # a padding token past the last segment writes zeros (ragged.go:101-117)
    q2 = np.concatenate([q, q[:qH * D]])
    r2 = orc.attention_ragged(q2, pk, pv, pages, lengths, off, batch + 1, batch, qH, kvH, D, B,
                              MP, _scale(D))
    assert np.array_equal(r2[:r.size], r) and np.all(r2[r.size:] == 0)


def test_ragged_causal_limit(rng):
    # specs/046 via ragged.go:119-151: token i of n sits at L-n+i and sees positions <= that
    qH, kvH, D, B, MP = 2, 1, 8, 4, 4
    L, n = 11, 3
    pages = np.array([2, 0, 3, 1], np.uint32)
    pk = rng.standard_normal(16 * D).astype(np.float32)
    pv = rng.standard_normal(16 * D).astype(np.float32)
    q = rng.standard_normal(n * qH * D).astype(np.float32)
    r = orc.attention_ragged(q, pk, pv, pages, [L], [0, n], n, 1, qH, kvH, D, B, MP, _scale(D))
    for i in range(n):
        vis = L - n + i + 1
        rows = np.array([pages[j // B] * B + j % B for j in range(vis)], np.uint32)
        want = orc.attention_definition_f64(q[i * qH * D:(i + 1) * qH * D], pk, pv, rows, qH, kvH,
                                            D, _scale(D))
        assert np.allclose(r[i * qH * D:(i + 1) * qH * D], want, atol=1e-5)
    # a sequence shorter than its count: the tokens with no position write zero
    r = orc.attention_ragged(q, pk, pv, pages, [2], [0, n], n, 1, qH, kvH, D, B, MP, _scale(D))
    assert np.all(r[:qH * D] == 0) and not np.any(r[qH * D:2 * qH * D] == 0)


# ----------------------------------------------------------------------------- grouped
def _grouped_fixture(E, K, N, counts):
    # internal/kernels/grouped_test.go:17-41
    off = orc.segment_offsets(counts)
    tokens = int(off[-1])
    x = np.sin(np.arange(tokens * K) * 0.23).astype(np.float32)
    base = np.cos(np.arange(K * N) * 0.17).astype(np.float32)
    w = np.concatenate([base * np.float32(e + 1) for e in range(E)]).astype(np.float32)
    return x, w, off, tokens


@pytest.mark.parametrize("E,K,N,counts", [(3, 64, 5, [2, 1, 3]), (4, 64, 3, [2, 0, 2, 0]),
                                          (2, 64, 2, [1, 1])])
def test_grouped_product_matches_each_expert_alone(E, K, N, counts):
    # internal/kernels/grouped_test.go:65-122
    x, w, off, tokens = _grouped_fixture(E, K, N, counts)
    assert list(off) == list(np.concatenate([[0], np.cumsum(counts)]))
    mv = orc.grouped_matvec(x, w, off, tokens, E, K, N)
    mm = orc.grouped_matmul(x, w, off, tokens, E, K, N)
    for e in range(E):
        for tok in range(off[e], off[e + 1]):
            want = x[tok * K:(tok + 1) * K].astype(np.float64) @ \
                w[e * K * N:(e + 1) * K * N].reshape(K, N).astype(np.float64)
            assert np.all(np.abs(mv[tok] - want) <= 1e-4)
            assert np.all(np.abs(mm[tok] - want) <= 1e-4)


def test_grouped_padding_token_and_clamp():
    # internal/kernels/grouped_test.go:188,304: a row past the last segment is zero in the row
    # kernel and untouched in the tiled one; counts that sum past the rows are clamped
    E, K, N = 2, 64, 4
    x, w, off, tokens = _grouped_fixture(E, K, N, [2, 1])
    xpad = np.concatenate([x, np.ones(K, np.float32)])
    mv = orc.grouped_matvec(xpad, w, off, tokens + 1, E, K, N)
    assert np.all(mv[tokens] == 0)
    out = np.full((tokens + 1, N), 7.0, np.float32)
    orc.grouped_matmul(xpad, w, off, tokens + 1, E, K, N, out=out)
    assert np.all(out[tokens] == 7.0)
    big = np.array([0, 2, 9], np.uint32)      # claims nine rows; three exist
    out = np.full((tokens, N), 7.0, np.float32)
    orc.grouped_matmul(x, w, big, tokens, E, K, N, out=out)
    assert not np.any(out == 7.0)


# ----------------------------------------------------------------------------- block pool
def test_block_pool():
    # tensor/blockpool_test.go:16-91
    p = orc.BlockPool(4, 8)
    assert p.block_size() == 8 and p.available() == 4
    a = p.grow(None, 9)
    assert a == [1, 0] and p.available() == 2 and p.positions(a) == 16
    before = list(a)
    a = p.grow(a, 17)
    assert len(a) == 3 and a[:2] == before and a[2] == 2
    same = p.grow(a, 20)
    assert len(same) == 3 and p.available() == 1
    with pytest.raises(ValueError, match="does not evict"):
        p.grow(a, 100)
    p.free(a)
    assert p.available() == 4
    with pytest.raises(ValueError):
        p.free(a)
    with pytest.raises(ValueError):
        orc.BlockPool(0, 8)
    with pytest.raises(ValueError):
        orc.BlockPool(4, 0)
    with pytest.raises(ValueError):
        p.grow(None, -1)


# ----------------------------------------------------------------------------- support operators
def test_support_operators_against_numpy(rng):
    x = rng.standard_normal((5, 300)).astype(np.float32)
    w = rng.standard_normal(300).astype(np.float32)
    got = orc.rmsnorm(x, w, 1e-5)
    want = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean(1, keepdims=True) + 1e-5) * w
    assert np.allclose(got, want, rtol=2e-6, atol=1e-6)

    pos = np.array([0, 1, 7, 2048, 100000], np.uint32)
    r = orc.rope(x[:, :64].copy(), pos, 64, 10000.0)
    k = np.arange(32)
    theta = pos[:, None].astype(np.float64) * np.exp(-2.0 * k / 64 * np.log(10000.0))
    xe, xo = x[:, 0:64:2].astype(np.float64), x[:, 1:64:2].astype(np.float64)
    assert np.allclose(r[:, 0::2], xe * np.cos(theta) - xo * np.sin(theta), atol=2e-2)
    assert np.allclose(r[:3, 0::2], (xe * np.cos(theta) - xo * np.sin(theta))[:3], atol=1e-5)
    assert np.allclose(r[:3, 1::2], (xe * np.sin(theta) + xo * np.cos(theta))[:3], atol=1e-5)

    a, b = x[0], x[1]
    assert np.allclose(orc.swiglu(a, b), a / (1 + np.exp(-a.astype(np.float64))) * b, rtol=1e-6, atol=1e-7)
    assert np.array_equal(orc.elem_add(a, b), a + b)

    logits = rng.standard_normal((4, 1000)).astype(np.float32)
    logits[1, 10] = logits[1, 500] = 50.0          # a tie goes to the lowest index
    logits[2, :] = -5.0
    am = orc.sample_argmax(logits)
    assert am[0] == logits[0].argmax() and am[1] == 10 and am[2] == 0 and am[3] == logits[3].argmax()

    table = rng.standard_normal((10, 6)).astype(np.float32)
    g = orc.gather_rows(table, [3, 99, 0], 6)
    assert np.array_equal(g[0], table[3]) and np.all(g[1] == 0) and np.array_equal(g[2], table[0])
    state = np.zeros((10, 6), np.float32)
    orc.scatter_rows(table[:3].copy(), [9, 10, 2], state)
    assert np.array_equal(state[9], table[0]) and np.array_equal(state[2], table[2])
    assert np.count_nonzero(state) == 12          # the row with id 10 was dropped


# ----------------------------------------------------------------------------- prefill attention
def test_prefill_equals_incremental_decode():
    # internal/kernels/prefill_test.go:185-250: cos/sin fixtures, n = 6 tokens prefilled at once
    # against one decode step per token over a growing cache, within 1e-5 (1 + |x|)
    qH, kvH, D, n = 4, 2, 8, 6
    scale = _scale(D)
    i = np.arange(n * kvH * D)
    k = np.cos(i * 0.23).astype(np.float32)
    v = (np.sin(i * 0.19).astype(np.float32) * np.float32(2)).astype(np.float32)
    q = np.sin(np.arange(n * qH * D) * 0.41).astype(np.float32)
    kc, vc = k.reshape(n, kvH, D), v.reshape(n, kvH, D)
    pre = orc.attention_prefill(q, kc, vc, np.array([n], np.uint32), qH, kvH, D, n, 0, scale)
    for step in range(n):
        one = orc.attention_decode(q[step * qH * D:(step + 1) * qH * D], kc[:step + 1], vc[:step + 1],
                                   np.array([step + 1], np.uint32), qH, kvH, D, scale)
        got = pre[step * qH * D:(step + 1) * qH * D]
        assert np.all(np.abs(got - one) <= 1e-5 * (1 + np.abs(one))), step


def test_paged_prefill_matches_the_contiguous_one_bit_for_bit(rng):
    # internal/kernels/prefill_test.go:1120-1190: a page table is an addressing, so the two answers
    # are the same answer (qHeads 4, kvHeads 2, headDim 16, block 8, 300 tokens from position 0)
    qH, kvH, D, block, q_seq, base = 4, 2, 16, 8, 300, 0
    kv_len = base + q_seq
    n_pages = (kv_len + block - 1) // block
    pool = 4 * n_pages
    q = rng.standard_normal(q_seq * qH * D).astype(np.float32)
    pk = rng.standard_normal((pool * block, kvH, D)).astype(np.float32)
    pv = rng.standard_normal((pool * block, kvH, D)).astype(np.float32)
    pages = rng.permutation(pool)[:n_pages].astype(np.uint32)
    lengths = np.array([kv_len], np.uint32)
    scale = _scale(D)
    paged = orc.attention_prefill_paged(q, pk, pv, pages, lengths, qH, kvH, D, q_seq, base, block, scale)
    rows = np.array([pages[j // block] * block + j % block for j in range(kv_len)])
    contiguous = orc.attention_prefill(q, pk[rows], pv[rows], lengths, qH, kvH, D, q_seq, base, scale)
    assert np.array_equal(paged, contiguous)
    # and against the definition in binary64, row by row of the causal mask
    for s_ in (0, 1, 127, 128, 299):
        want = orc.attention_definition_f64(q[s_ * qH * D:(s_ + 1) * qH * D], pk, pv, rows[:base + s_ + 1],
                                            qH, kvH, D, scale)
        assert np.max(np.abs(paged[s_ * qH * D:(s_ + 1) * qH * D] - want)) <= 1e-5


# ----------------------------------------------------------------------------- sampling policy
def _kept(out):
    return [i for i, v in enumerate(np.ravel(out)) if v != 0]


def test_categorical_walks_the_distribution():
    # internal/kernels/sample_test.go:105-150
    probs = np.array([0.1, 0.2, 0.3, 0.4], np.float32)
    for draw, want in [(0, 0), (0.05, 0), (0.1, 1), (0.15, 1), (0.3, 2), (0.45, 2), (0.6, 3), (0.99, 3),
                       (0.999999, 3), (-0.5, 0), (1.5, 3), (1.0, 3)]:
        assert orc.sample_rows(probs, [draw])[0] == want, draw
    short = np.array([0.25, 0.25, 0.25, 0.2499], np.float32)
    assert orc.sample_rows(short, [0.9999])[0] == 3


def test_top_k_keeps_exactly_k_and_the_largest():
    # internal/kernels/topk_test.go:67-105, ties to the lowest indices
    for w, k, want in [([0.1, 0.5, 0.2, 0.4, 0.3], 2, [1, 3]), ([0.1, 0.5, 0.2], 1, [1]),
                       ([0.3, 0.1, 0.2], 3, [0, 1, 2]), ([5, 5, 5, 5, 1], 2, [0, 1]),
                       ([2, 2, 2, 2], 3, [0, 1, 2]), ([0, 3, 0, 1, 0], 2, [1, 3])]:
        out = orc.topk_mask(np.array(w, np.float32), k)
        assert _kept(out) == want, (w, k)
        assert all(out[i] == np.float32(w[i]) for i in want)


def test_top_p_keeps_the_nucleus_and_is_relative_to_its_input():
    # internal/kernels/topk_test.go:152-225
    w = np.array([0.1, 0.2, 0.3, 0.4], np.float32)
    for p, want in [(0.3, [3]), (0.4, [3]), (0.5, [2, 3]), (0.7, [2, 3]), (0.9, [1, 2, 3]), (1.0, [0, 1, 2, 3])]:
        assert _kept(orc.topp_mask(w, p)) == want, p
    assert _kept(orc.topp_mask(w * np.float32(37), 0.5)) == _kept(orc.topp_mask(w, 0.5))
    ramp = np.arange(1, 65, dtype=np.float32)
    after_k = orc.topk_mask(ramp, 8)
    after_p = _kept(orc.topp_mask(after_k, 0.5))
    assert 0 < len(after_p) <= 8 and set(after_p) <= set(_kept(after_k))


def test_truncation_respects_its_bound_and_matches_a_sort(rng):
    # internal/kernels/topk_test.go:110-150, 229-260: at most TopMaxRounds = 128 entries are kept
    w = rng.random(400).astype(np.float32)
    assert len(_kept(orc.topk_mask(w, 300))) == 128
    for k in (1, 7, 50):
        want = sorted(sorted(range(400), key=lambda i: (-w[i], i))[:k])
        assert _kept(orc.topk_mask(w, k)) == want
    # per-row parameters: k = 0 passes the row through; so does k >= vocab, but the bound of 128
    # rounds is applied FIRST (rowsample.go:51-57), so with 400 entries k = 400 keeps 128 of them
    rows = np.stack([w, w, w])
    out = orc.topk_mask(rows, np.array([0, 5, 400], np.uint32))
    assert np.array_equal(out[0], w) and len(_kept(out[1])) == 5 and len(_kept(out[2])) == 128
    small = orc.topk_mask(np.stack([w[:100]]), np.array([100], np.uint32))
    assert np.array_equal(small[0], w[:100])
    outp = orc.topp_mask(rows, np.array([0.0, 0.5, 1.0], np.float32))
    assert np.array_equal(outp[0], w) and 0 < len(_kept(outp[1])) < 400 and np.array_equal(outp[2], w)


def test_penalties():
    # internal/kernels/penalty_test.go:40-135
    logits = np.array([0.1, -0.3, 2.7, -1.9, 0.30000001, 1e-30, -1e-30, 3.3], np.float32)
    got, _ = orc.penalty_rows(logits, [2, 5, 0, 0], 2, 1.3, 0.5, 0.25)
    for i in range(8):
        if i not in (2, 5):
            assert got[0, i] == logits[i]
    got, _ = orc.penalty_rows(np.array([2.0, -2.0], np.float32), [0, 1], 2, 2.0, 0.0, 0.0)
    assert got[0, 0] < 2.0 and got[0, 1] == np.float32(-4)
    got, _ = orc.penalty_rows(np.zeros(3, np.float32), [0, 1, 1, 2, 2, 2, 0, 0], 6, 0.0, 1.0, 0.5)
    assert np.array_equal(got[0], np.array([-1.5, -2, -2.5], np.float32))
    got, _ = orc.penalty_rows(np.zeros(4, np.float32), [1, 2, 3, 0, 0, 0, 0, 0], 3, 0.0, 1.0, 0.0)
    assert np.array_equal(got[0], np.array([0, -1, -1, -1], np.float32))
    got, counts = orc.penalty_rows(np.zeros(4, np.float32), [9, 4, 1, 4], 4, 0.0, 1.0, 0.0)
    assert got[0, 3] == 0 and np.array_equal(counts[0], np.array([0, 1, 0, 0], np.uint32))


def test_softmax_is_a_distribution_and_matches_binary64(rng):
    x = (rng.standard_normal((3, 1000)) * 5).astype(np.float32)
    x[1] += 100                                       # a logit of 100 is ordinary
    y = orc.softmax(x)
    e = np.exp(x.astype(np.float64) - x.max(axis=1, keepdims=True))
    assert np.max(np.abs(y - e / e.sum(axis=1, keepdims=True))) < 1e-6
    assert np.all(np.abs(y.sum(axis=1) - 1) < 1e-5)


# ---------------------------------------------------------------- int8 weights
def test_int8_dequantize_is_quant_times_scale():
    # quant/quant_test.go:227-238
    got = orc.int8_dequantize(np.array([1, -2, 127, -127], np.int8), orc.to_f16_bits(np.array([0.5], np.float32)))
    assert np.array_equal(got, np.array([0.5, -1, 63.5, -63.5], np.float32))


def _int8_cases():
    smooth = np.array([math.sin(i * 0.31) * 3 for i in range(200)], np.float32)
    outlier = np.full(128, 0.01, np.float32)
    outlier[::32] = 100
    half_zero = np.zeros(64, np.float32)
    half_zero[32:] = np.arange(32, 64)
    return {"smooth": smooth, "one outlier per block": outlier, "ragged": np.array([1, -2, 3, -4, 5], np.float32),
            "zeros": np.zeros(64, np.float32), "a block of zeros beside values": half_zero,
            "negatives": -np.arange(1, 41, dtype=np.float32)}


@pytest.mark.parametrize("name", sorted(_int8_cases()))
def test_int8_every_weight_is_within_half_a_step(name):
    # quant/quant_test.go:22-100
    w = _int8_cases()[name]
    q, s = orc.int8_quantize(w)
    assert q.size == w.size and s.size == (w.size + 31) // 32
    back = orc.int8_dequantize(q, s)
    step = orc.from_f16_bits(s)[np.arange(w.size) // 32].astype(np.float64)
    assert np.all(np.abs(back.astype(np.float64) - w) <= step / 2 * (1 + 1e-3))
    assert q.min() >= -127 and q.max() <= 127


def test_int8_clamp_and_underflow():
    # quant/quant_test.go:110-133: values a few ulps under the peak must not wrap to -128
    peak = np.float32(1.0)
    w = (np.full(32, peak.view(np.uint32), np.uint32) - np.arange(32, dtype=np.uint32)).view(np.float32)
    q, s = orc.int8_quantize(w)
    assert q.min() >= 0 and np.all(orc.int8_dequantize(q, s) >= 0)
    # quant/quant_test.go:203-224: a scale that underflows f16 gives zero quants and zeros back
    q, s = orc.int8_quantize(np.full(32, 1e-12, np.float32))
    assert orc.from_f16_bits(s)[0] == 0 and not q.any() and not orc.int8_dequantize(q, s).any()


@pytest.mark.parametrize("m,n,k", [(1, 8, 32), (1, 5, 64), (4, 8, 32), (3, 7, 96), (1, 16, 256)])
def test_int8_products_are_exact_where_the_arithmetic_is(m, n, k):
    """internal/kernels/f32variants_test.go:770-850: activations in quarters, quants i % 201 - 100,
    scales 1/4 + (i % 3) / 8.  Every product and partial sum is a small dyadic rational, exact in
    f32 in any order, so both kernels must return the integer arithmetic's answer bit for bit."""
    a = np.array([((i % 13) - 6) / 4 for i in range(m * k)], np.float32)
    bq = np.array([i % 201 - 100 for i in range(k * n)], np.int8)
    sv = np.array([0.25 + (i % 3) / 8 for i in range((k * n + 31) // 32)], np.float32)
    bs = orc.to_f16_bits(sv)
    want = np.zeros((m, n), np.float64)
    for r in range(m):
        for c in range(n):
            idx = np.arange(k) * n + c
            want[r, c] = np.sum(a[r * k:(r + 1) * k].astype(np.float64) * bq[idx] * sv[idx // 32].astype(np.float64))
    got = orc.quant_matmul_tiled_f32(a, bq, bs, m, n, k)
    assert np.array_equal(got.astype(np.float64), want)
    if m == 1:
        assert np.array_equal(orc.quant_matvec_f32(a, bq, bs, n, k).astype(np.float64), want[0])


@pytest.mark.parametrize("m,n,k", [(1, 8, 64), (4, 16, 128), (3, 5, 33), (2, 7, 96)])
def test_int8_products_meet_the_reference_budget(m, n, k):
    # internal/kernels/quant_test.go:45-117: half a scale step per term plus gamma(K-1) of accumulation
    a = np.array([math.sin(i * 0.23) * 2 for i in range(m * k)], np.float32)
    w = np.array([math.cos(i * 0.31) * 1.5 for i in range(k * n)], np.float32)
    bq, bs = orc.int8_quantize(w)
    sc = orc.from_f16_bits(bs).astype(np.float64)
    outs = [orc.quant_matmul_tiled_f32(a, bq, bs, m, n, k)]
    if m == 1:
        outs.append(orc.quant_matvec_f32(a, bq, bs, n, k)[None, :])
    nu = (k - 1) / (1 << 24)
    for out in outs:
        for r in range(m):
            for c in range(n):
                idx = np.arange(k) * n + c
                x = a[r * k:(r + 1) * k].astype(np.float64)
                exact = np.sum(x * w[idx])
                budget = np.sum(np.abs(x) * sc[idx // 32] / 2) + nu / (1 - nu) * np.sum(np.abs(x * w[idx]))
                assert abs(out[r, c] - exact) <= budget
