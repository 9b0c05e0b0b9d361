"""Parity of the grouped (per-expert) products with the oracle, through the C ABI, on a B200.
Tolerance: 1e-3 relative, f32 accumulate; the int4 form is checked against the composition
dequantize-per-expert -> grouped product, which is its definition (no reference kernel exists)."""
import numpy as np
import pytest
import torch

import oracle as orc
from accel_b200 import runtime
from accel_b200 import tensor as T
from util import GEMM_TOL, assert_close, normal

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a):
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).to(DEV)
    return torch.from_numpy(a).to(DEV)


def fixture(E, K, N, counts):
    # internal/kernels/grouped_test.go:17-41
    off = orc.segment_offsets(np.array(counts, np.uint32))
    tokens = int(off[-1])
    x = np.sin(np.arange(tokens * K) * 0.23).astype(np.float32).reshape(tokens, K)
    base = np.cos(np.arange(K * N) * 0.17).astype(np.float32)
    w = np.stack([base * np.float32(e + 1) for e in range(E)]).reshape(E, K, N)
    return x, w, off, tokens


@pytest.mark.parametrize("E,K,N,counts", [(3, 64, 5, [2, 1, 3]), (4, 64, 3, [2, 0, 2, 0]),
                                          (2, 64, 2, [1, 1]), (3, 64, 256, [130, 0, 7]),
                                          (5, 48, 132, [9, 300, 0, 1, 128])])
def test_reference_fixtures(E, K, N, counts):
    x, w, off, tokens = fixture(E, K, N, counts)
    c = dev(np.array(counts, np.uint32))
    assert np.array_equal(T.segment_offsets(c).cpu().numpy().view(np.uint32), off)
    want = orc.grouped_matmul(x, w, off, tokens, E, K, N)
    mm = T.grouped_matmul(dev(x), dev(w), c).cpu().numpy()
    mv = T.grouped_matvec(dev(x), dev(w), c).cpu().numpy()
    assert_close(mm, want, GEMM_TOL, "GroupedMatMul")
    assert_close(mv, orc.grouped_matvec(x, w, off, tokens, E, K, N), GEMM_TOL, "GroupedMatVec")


def test_padding_rows_and_clamp():
    # grouped.go:72-77 (zeros), groupedtiled.go:87-91,96-133 (untouched; clamp to Tokens)
    E, K, N = 2, 64, 8
    x, w, off, tokens = fixture(E, K, N, [2, 1])
    xpad = np.concatenate([x, np.ones((2, K), np.float32)])
    c = dev(np.array([2, 1], np.uint32))
    mv = T.grouped_matvec(dev(xpad), dev(w), c).cpu().numpy()
    assert np.all(mv[tokens:] == 0)
    out = torch.full((tokens + 2, N), 7.0, device=DEV)
    T.grouped_matmul(dev(xpad), dev(w), c, out=out)
    assert torch.all(out[tokens:] == 7.0) and not torch.any(out[:tokens] == 7.0)
    big = dev(np.array([2, 9], np.uint32))            # claims eleven rows; three exist
    out = torch.full((tokens, N), 7.0, device=DEV)
    T.grouped_matmul(dev(x), dev(w), big, out=out)
    want = orc.grouped_matmul(x, w, np.array([0, 2, 11], np.uint32), tokens, E, K, N)
    assert_close(out.cpu().numpy(), want, GEMM_TOL, "clamped")


def test_moe_shape_reduced_against_the_oracle():
    # eight experts, seeded multinomial counts, d=4096 contracting into a 1024-column slice of the
    # expert FFN: the full 14336 columns are the same kernel over more column tiles
    E, K, N, rows = 8, 4096, 1024, 512
    rng = np.random.default_rng(5)
    counts = rng.multinomial(rows, np.ones(E) / E).astype(np.uint32)
    x = normal(6, (rows, K))
    w = normal(7, (E, K, N), 0.02)
    off = orc.segment_offsets(counts)
    want = orc.grouped_matmul(x, w, off, rows, E, K, N)
    got = T.grouped_matmul(dev(x), dev(w), dev(counts)).cpu().numpy()
    assert_close(got, want, GEMM_TOL, "MoE slice")


@pytest.mark.parametrize("K,kernel", [(256, "tensor-core kernel"), (80, "register-tiled kernel")])
def test_int4_grouped_is_the_composition(K, kernel):
    E, N, rows = 4, 384, 200
    counts = np.array([70, 0, 129, 1], np.uint32)        # an empty expert, a two-tile expert, one row
    x = normal(9, (rows, K))
    w = normal(10, (E, K, N), 0.02)
    w[2, 5, 128:256] = 0.125                              # a constant group: scale 0, weight = zero point
    planes = [orc.int4_quantize(w[e]) for e in range(E)]
    back = np.stack([orc.int4_dequantize(*planes[e], K * N).reshape(K, N) for e in range(E)])
    q = T.Int4(dev(np.concatenate([p[0] for p in planes])),
               torch.from_numpy(np.concatenate([p[1] for p in planes]).view(np.float16)).to(DEV),
               torch.from_numpy(np.concatenate([p[2] for p in planes]).view(np.float16)).to(DEV),
               E * K * N)
    off = orc.segment_offsets(counts)
    want = orc.grouped_matmul(x, back, off, rows, E, K, N)
    got = T.grouped_matmul_int4(dev(x), q, E, dev(counts)).cpu().numpy()
    assert kernel in runtime.last_selection()
    assert_close(got, want, GEMM_TOL, "int4 grouped")
    # tiny activations keep the accuracy of ordinary ones (rows are scaled by exact powers of two)
    tiny = (x * np.float32(1e-4)).astype(np.float32)
    got = T.grouped_matmul_int4(dev(tiny), q, E, dev(counts)).cpu().numpy()
    assert_close(got, orc.grouped_matmul(tiny, back, off, rows, E, K, N), GEMM_TOL, "int4 grouped, activations x 1e-4")


@pytest.mark.parametrize("E,K,N,counts", [(4, 256, 384, [70, 0, 129, 1]), (8, 4096, 1024, None), (3, 100, 128, [128, 128, 5]),
                                          (2, 512, 256, [0, 0])])
def test_int4_grouped_on_the_prepacked_stream(E, K, N, counts):
    """GroupedMatMulInt4Packed (the tcgen05 tile kernel, every expert's segment in row blocks of its
    own) against the reference GroupedMatMul over each expert's dequantized weights: segments that
    are empty, one row, exact multiples of 128 and ragged."""
    from accel_b200 import quant
    rows = 512 if counts is None else int(np.sum(counts))
    if counts is None:
        counts = np.random.default_rng(5).multinomial(rows, np.ones(E) / E)
    counts = np.asarray(counts, np.uint32)
    x = normal(9, (max(rows, 1), K))[:rows]
    w = normal(10, (E, K, N), 0.02)
    w[E - 1, 5, :128] = 0.125                             # a constant group: scale 0, weight = zero point
    planes = [orc.int4_quantize(w[e]) for e in range(E)]
    back = np.stack([orc.int4_dequantize(*planes[e], K * N).reshape(K, N) for e in range(E)])
    f16 = lambda a: torch.from_numpy(a.view(np.float16)).to(DEV)
    packed = torch.cat([quant.int4_prepack(dev(p[0]), f16(p[1]), f16(p[2]), K, N) for p in planes])
    off = orc.segment_offsets(counts)
    out = torch.full((rows, N), float("nan"), device=DEV)
    runtime.launch("GroupedMatMulInt4Packed", [dev(x), packed, dev(off), out], runtime.grouped_tiled_dims(E, rows, K, N))
    torch.cuda.synchronize()
    quant.int4_stream_check()
    if rows:
        assert "grouped int4 tile kernel on tcgen05" in runtime.last_selection()
        assert_close(out.cpu().numpy(), orc.grouped_matmul(x, back, off, rows, E, K, N), GEMM_TOL, "int4 grouped, packed")


def test_refusals():
    x = torch.zeros(4, 8, device=DEV)
    w = torch.zeros(2, 8, 3, device=DEV)
    c = torch.zeros(2, dtype=torch.int32, device=DEV)
    with pytest.raises(T.Refused, match="counts is nil"):
        T.grouped_matmul(x, w, None)
    with pytest.raises(T.Refused, match="reads f32"):
        T.grouped_matmul(x.half(), w, c)
    with pytest.raises(T.Refused, match=r"\[tokens, K\]"):
        T.grouped_matmul(x[0], w, c)
    with pytest.raises(T.Refused, match="one matrix per expert"):
        T.grouped_matmul(x, w[0], c)
    with pytest.raises(T.Refused, match="same width"):
        T.grouped_matmul(torch.zeros(4, 9, device=DEV), w, c)
    with pytest.raises(T.Refused, match="one token count per expert"):
        T.grouped_matvec(x, w, torch.zeros(3, dtype=torch.int32, device=DEV))
