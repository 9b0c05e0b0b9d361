"""The batch int4 kernel over prepacked weights (tcgen05, weights dequantised into tensor memory,
activation tiles by bulk copies) against the oracle, on a B200.  From 49 activation rows the packed
entry points select it; the decode kernel's tests (test_int4_stream_gpu.py) cover fewer rows."""
import struct

import numpy as np
import pytest
import torch

import oracle as orc
from accel_b200 import quant, runtime
from util import GEMM_TOL, assert_close, normal

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def packed_of(p, s, z, K, N):
    dev = lambda a, dt: torch.from_numpy(a.view(dt)).to(DEV)
    return quant.int4_prepack(dev(p, np.int32), dev(s, np.float16), dev(z, np.float16), K, N)


def product(a, packed, M, K, N):
    out = torch.full((M, N), float("nan"), device=DEV)
    x = torch.from_numpy(a).to(DEV)
    runtime.launch("QuantMatMulInt4Packed", [x, packed, out], runtime.gemm_dims(M, N, K))
    torch.cuda.synchronize()
    quant.int4_stream_check()
    assert "tile kernel on tcgen05" in runtime.last_selection(), runtime.last_selection()
    return out.cpu().numpy()


def with_constant_groups(seed, K, N, std=0.02):
    w = normal(seed, (K, N), std)
    w.reshape(-1)[3 * N:3 * N + 128] = 0.25          # constant groups: scale 0, value in the zero point
    w.reshape(-1)[K * N - 128:] = -0.125
    return w


@pytest.mark.parametrize("M,K,N", [(49, 4096, 1024), (64, 4096, 4096), (128, 1024, 384), (130, 512, 256),
                                   (70, 4100, 512), (300, 100, 256), (64, 4096, 11008), (257, 2048, 1536)])
def test_matches_the_oracle(M, K, N):
    w = with_constant_groups(2, K, N)
    p, s, z = orc.int4_quantize(w)
    a = normal(1, (M, K))
    got = product(a, packed_of(p, s, z, K, N), M, K, N)
    assert_close(got, orc.quant_matmul_int4(a, p, s, z, M, N, K), GEMM_TOL, f"int4 tiles M={M} K={K} N={N}")


@pytest.mark.parametrize("M", [128, 512])
def test_full_size_against_a_binary64_product(M):
    """K=4096, N=11008 at the larger batch sizes of the reference's tiled kernel
    (internal/kernels/int4tiled.go:66-137): the definition in binary64 over the dequantized weights,
    and a sample of rows against the order-faithful oracle."""
    K, N = 4096, 11008
    w = with_constant_groups(2, K, N)
    p, s, z = orc.int4_quantize(w)
    back = orc.int4_dequantize(p, s, z, K * N).reshape(K, N)
    a = normal(1, (M, K))
    want = (torch.from_numpy(a).to(DEV).double() @ torch.from_numpy(back).to(DEV).double()).cpu().numpy()
    got = product(a, packed_of(p, s, z, K, N), M, K, N)
    assert_close(got, want, GEMM_TOL, f"full size M={M}")
    rows = [0, M // 2, M - 1]
    assert_close(got[rows], orc.quant_matmul_int4(a[rows], p, s, z, len(rows), N, K), GEMM_TOL, "oracle rows")


@pytest.mark.parametrize("factor", [1e-4, 1e4, 1e-20, 1e20])
def test_activation_magnitude_does_not_matter(factor):
    M, K, N = 80, 2048, 512
    p, s, z = orc.int4_quantize(normal(4, (K, N), 0.02))
    a = normal(5, (M, K)) * np.float32(factor)
    a[1] *= np.float32(1e-3)                          # rows of very different magnitude in one call
    got = product(a, packed_of(p, s, z, K, N), M, K, N)
    want = orc.quant_matmul_int4(a, p, s, z, M, N, K)
    for m in range(M):
        assert_close(got[m], want[m], GEMM_TOL, f"row {m} at activations x {factor:g}")


@pytest.mark.parametrize("std", [1e-5, 30.0])
def test_weight_magnitude_does_not_matter(std):
    M, K, N = 80, 2048, 512
    p, s, z = orc.int4_quantize(normal(6, (K, N), std))
    a = normal(7, (M, K))
    got = product(a, packed_of(p, s, z, K, N), M, K, N)
    assert_close(got, orc.quant_matmul_int4(a, p, s, z, M, N, K), GEMM_TOL, f"weights of std {std:g}")


def test_per_element_bound():
    """|y - y_f64| <= (gamma(K) + 2 * 2^-11) * sum_k |a_k| |w_k| for EVERY output: gamma(K) is the
    reference's bound for its own f32 accumulation (internal/kernels/int4_test.go:99-182); this
    kernel rounds both operands to f16, 2^-11 each."""
    M, K, N = 128, 4096, 4096
    w = normal(8, (K, N), 0.02)
    p, s, z = orc.int4_quantize(w)
    a = normal(9, (M, K))
    back = orc.int4_dequantize(p, s, z, w.size)
    want, mag = orc.matmul_definition_f64(a, back, M, N, K)
    got = product(a, packed_of(p, s, z, K, N), M, K, N)
    nu = (K - 1) * 2.0 ** -24
    bound = (nu / (1 - nu) + 2.0 ** -10) * mag
    assert np.all(np.abs(got - want) <= bound), float(np.max(np.abs(got - want) / mag))


def test_the_three_output_form_equals_the_plain_product_bit_for_bit():
    M, K, N1, N2, N3 = 200, 1024, 512, 256, 256
    N = N1 + N2 + N3
    p, s, z = orc.int4_quantize(normal(12, (K, N), 0.02))
    packed = packed_of(p, s, z, K, N)
    a = torch.from_numpy(normal(13, (M, K))).to(DEV)
    whole = torch.empty(M, N, device=DEV)
    runtime.launch("QuantMatMulInt4Packed", [a, packed, whole], runtime.gemm_dims(M, N, K))
    o = [torch.full((M, n), float("nan"), device=DEV) for n in (N1, N2, N3)]
    runtime.launch("QuantMatMulInt4PackedSplit3", [a, packed, *o], struct.pack("<IIIIIIII", M, N, K, N1, N2, 0, 0, 0))
    torch.cuda.synchronize()
    quant.int4_stream_check()
    assert torch.equal(torch.cat(o, dim=1), whole)


@pytest.mark.parametrize("M,K,F", [(64, 4096, 11008), (150, 512, 256)])
def test_the_swiglu_epilogue_equals_the_product_followed_by_swiglu(M, K, F):
    wg, wu = normal(14, (K, F), 0.02), normal(15, (K, F), 0.02)
    qg, qu = orc.int4_quantize(wg), orc.int4_quantize(wu)
    G = F // 128
    inter = lambda x, y, per: np.stack([x.reshape(K, G, per), y.reshape(K, G, per)], axis=2).reshape(-1)
    packed = packed_of(inter(qg[0], qu[0], 16), inter(qg[1], qu[1], 1), inter(qg[2], qu[2], 1), K, 2 * F)
    a = torch.from_numpy(normal(16, (M, K))).to(DEV)
    out = torch.full((M, F), float("nan"), device=DEV)
    runtime.launch("QuantMatMulInt4PackedSwiGLU", [a, packed, out], runtime.gemm_dims(M, 2 * F, K))
    both = torch.empty(M, 2 * F, device=DEV)
    runtime.launch("QuantMatMulInt4Packed", [a, packed, both], runtime.gemm_dims(M, 2 * F, K))
    parts = both.view(M, G, 2, 128)
    gate, up = parts[:, :, 0, :].contiguous().view(M, F), parts[:, :, 1, :].contiguous().view(M, F)
    want = torch.empty(M, F, device=DEV)
    runtime.launch("SwiGLU", [gate, up, want])
    torch.cuda.synchronize()
    quant.int4_stream_check()
    assert_close(out.cpu().numpy(), want.cpu().numpy(), 1e-5, "SwiGLU epilogue against the chain")


def test_more_rows_than_one_pass_converts():
    """Activations are converted 4096 rows at a time; a call with more rows runs several passes."""
    M, K, N = 4096 + 130, 256, 256
    p, s, z = orc.int4_quantize(normal(20, (K, N), 0.02))
    a = normal(21, (M, K))
    got = product(a, packed_of(p, s, z, K, N), M, K, N)
    rows = [0, 4095, 4096, M - 1]
    assert_close(got[rows], orc.quant_matmul_int4(a[rows], p, s, z, len(rows), N, K), GEMM_TOL, "pass boundaries")
    back = orc.int4_dequantize(p, s, z, K * N).reshape(K, N)
    assert_close(got, a.astype(np.float64) @ back.astype(np.float64), GEMM_TOL, "all rows")
