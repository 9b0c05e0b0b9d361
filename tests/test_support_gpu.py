"""The support operators of a decode step against the oracle, through the C ABI, on a B200.
Copies, gathers, scatters, casts and argmax are bit-exact; RMSNorm, RoPE and SwiGLU are within
1e-5 relative (f32, a different reduction order and the device's exp)."""
import numpy as np
import pytest
import torch

import oracle as orc
from accel_b200 import tensor as T
from util import assert_close, normal

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a):
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).to(DEV)
    return torch.from_numpy(a).to(DEV)


def test_rmsnorm():
    for rows, width in [(16, 4096), (3, 300), (1, 11008), (5, 8)]:
        x, w = normal(1, (rows, width)), normal(2, (width,))
        got = T.rms_norm(dev(x), dev(w), 1e-5).cpu().numpy()
        assert_close(got, orc.rmsnorm(x, w, 1e-5), 1e-5, f"RMSNorm {rows}x{width}")


def test_rope_interleaved_pairs_one_position_per_row():
    rows, width = 16 * 32, 128
    x = normal(3, (rows, width))
    pos = np.random.default_rng(4).integers(0, 4096, rows).astype(np.uint32)
    pos[:4] = [0, 1, 2048, 100000]
    got = T.rope(dev(x), dev(pos), width, 10000.0).cpu().numpy()
    want = orc.rope(x, pos, width, 10000.0)
    assert_close(got, want, 1e-5, "RoPE")
    # partial rotary dimension leaves the tail of each row untouched
    got = T.rope(dev(x), dev(pos), 64, 10000.0).cpu().numpy()
    assert np.array_equal(got[:, 64:], x[:, 64:])
    assert_close(got, orc.rope(x, pos, 64, 10000.0), 1e-5, "RoPE, rotary 64")


def test_swiglu_and_add():
    a, b = normal(5, (16, 11008)), normal(6, (16, 11008))
    a[0, :4] = [0.0, -100.0, 100.0, -0.0]
    assert_close(T.swiglu(dev(a), dev(b)).cpu().numpy(), orc.swiglu(a, b), 1e-5, "SwiGLU")
    assert np.array_equal(T.add(dev(a), dev(b)).cpu().numpy(), orc.elem_add(a, b))


def test_gather_and_scatter_rows():
    table = normal(7, (1000, 96))
    ids = np.array([3, 999, 1000, 0, 4000000000, 17], np.uint32)
    got = T.gather_rows(dev(table), dev(ids)).cpu().numpy()
    assert np.array_equal(got, orc.gather_rows(table, ids, 96))
    assert np.array_equal(T.gather_rows(dev(table.astype(np.float16)), dev(ids)).cpu().numpy(),
                          orc.gather_rows(table.astype(np.float16).astype(np.float32), ids, 96))
    for dt in (np.float32, np.float16):
        state = np.zeros((64, 32, 8), dt)
        rows = normal(8, (5, 32, 8)).astype(dt)
        ids = np.array([63, 64, 0, 7, 4000000000], np.uint32)     # two are out of range: dropped
        want = orc.scatter_rows(rows.view(np.uint16) if dt == np.float16 else rows, ids,
                                (state.view(np.uint16) if dt == np.float16 else state).copy(), 64)
        st = dev(state)
        T.scatter_rows(st, dev(rows), dev(ids))
        got = st.cpu().numpy()
        assert np.array_equal(got.view(np.uint16) if dt == np.float16 else got, want)


def test_argmax_ties_go_to_the_lowest_index():
    logits = normal(9, (16, 32000))
    logits[1, 10] = logits[1, 31999] = 50.0
    logits[2, :] = -5.0
    logits[3, 31999] = 60.0
    got = T.argmax(dev(logits)).cpu().numpy().view(np.uint32)
    assert np.array_equal(got, orc.sample_argmax(logits))
    assert got[1] == 10 and got[2] == 0 and got[3] == 31999


@pytest.mark.parametrize("parts", [2, 4, 8])
def test_argmax_over_a_vocabulary_split_by_columns_equals_sample_argmax(parts):
    """The tensor-parallel lm_head's exchange on one GPU: every shard's (largest logit, index)
    pairs summed slot by slot (what the all-reduce over ranks does, the other slots being zero),
    merged, against SampleArgmax over the unsplit logits, ties and all."""
    import struct
    from accel_b200 import runtime as rt
    rows, vocab = 16, 32000
    logits = normal(31, (rows, vocab))
    logits[3, 100] = logits[3, 31000] = 9.0              # a tie across shards: the lowest index wins
    logits[4, :] = -1.0                                  # all equal: index 0
    logits[5, 17] = np.nan                               # a NaN is never the largest
    logits[5, 18] = 8.0
    x = torch.from_numpy(logits).to(DEV)
    want = torch.empty(rows, dtype=torch.int32, device=DEV)
    rt.launch("SampleArgmax", [x, want], rt.sample_dims(vocab, rows))
    width = vocab // parts
    total = torch.zeros(rows, parts, 2, device=DEV)
    for r in range(parts):
        shard = x[:, r * width:(r + 1) * width].contiguous()
        pairs = torch.full((rows, parts, 2), float("nan"), device=DEV)
        rt.launch("ArgmaxShard", [shard, pairs], struct.pack("<IIIIIIII", width, rows, parts, r, r * width, 0, 0, 0))
        total += pairs
    got = torch.empty(rows, dtype=torch.int32, device=DEV)
    rt.launch("ArgmaxMerge", [total, got], struct.pack("<IIII", rows, parts, 0, 0))
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    assert got[3].item() == 100 and got[4].item() == 0 and got[5].item() == 18


def test_casts_round_as_the_reference_does():
    rng = np.random.default_rng(10)
    x = (rng.standard_normal(100000) * np.exp(rng.uniform(-20, 12, 100000))).astype(np.float32)
    x[:8] = [0.0, -0.0, 3.1e-8, 2.9e-8, 65520.0, np.inf, -np.inf, 1.9997]
    h = T.cast(dev(x), torch.float16)
    assert np.array_equal(h.cpu().numpy().view(np.uint16), orc.to_f16_bits(x))
    back = T.cast(h, torch.float32).cpu().numpy()
    assert np.array_equal(back, orc.from_f16_bits(orc.to_f16_bits(x)))
