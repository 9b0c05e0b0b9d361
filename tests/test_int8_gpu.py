"""The int8 linear path (quant.Int8Quantize weights, f32 activations) against the oracle's
restatement of QuantMatVecF32 and QuantMatMulTiledF32, on a B200."""
import math

import numpy as np
import pytest
import torch

import oracle as orc
from accel_b200 import quant, runtime
from accel_b200 import tensor as T
from util import GEMM_TOL, assert_close, normal

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def weight(bq, bs, K, N):
    return T.Quantized(torch.from_numpy(bq.reshape(K, N)).to(DEV),
                       torch.from_numpy(bs.view(np.float16)).to(DEV))


def product(a, bq, bs, M, K, N):
    out = T.quant_matmul(torch.from_numpy(a.reshape(M, K)).to(DEV), weight(bq, bs, K, N))
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("m,n,k", [(1, 8, 32), (1, 5, 64), (4, 8, 32), (3, 7, 96), (1, 16, 256),
                                   (1, 64, 96), (5, 256, 128), (9, 320, 64)])
def test_exact_where_the_arithmetic_is(m, n, k):
    """internal/kernels/f32variants_test.go:770-850: activations in quarters, quants i % 201 - 100,
    scales 1/4 + (i % 3) / 8: every product and partial sum is a small dyadic rational, so any order
    of f32 sums gives the same bits, and the device must equal the oracle exactly (both kernels,
    the generic one for N off the block and the streaming one)."""
    a = np.array([((i % 13) - 6) / 4 for i in range(m * k)], np.float32)
    bq = np.array([i % 201 - 100 for i in range(k * n)], np.int8)
    bs = orc.to_f16_bits(np.array([0.25 + (i % 3) / 8 for i in range((k * n + 31) // 32)], np.float32))
    got = product(a, bq, bs, m, k, n)
    want = orc.quant_matmul_tiled_f32(a, bq, bs, m, n, k)
    assert np.array_equal(got, want), runtime.last_selection()
    if m == 1:
        assert np.array_equal(got[0], orc.quant_matvec_f32(a, bq, bs, n, k))


@pytest.mark.parametrize("M,K,N", [(1, 4096, 4096), (1, 4096, 11008), (16, 4096, 4096), (8, 11008, 4096),
                                   (3, 1000, 384), (20, 512, 96), (1, 33, 160), (5, 100, 7)])
def test_matches_the_oracle(M, K, N):
    w = normal(3, (K, N), 0.02)
    w.reshape(-1)[64:96] = 0                          # a block of zeros: scale 0, quants 0
    bq, bs = orc.int8_quantize(w)
    a = normal(4, (M, K))
    got = product(a, bq, bs, M, K, N)
    if M == 1:
        want = orc.quant_matvec_f32(a[0], bq, bs, N, K)[None, :]
    else:
        want = orc.quant_matmul_tiled_f32(a, bq, bs, M, N, K)
    assert_close(got, want, GEMM_TOL, f"int8 M={M} K={K} N={N}")
    if N % 32 == 0:
        assert "streaming kernel" in runtime.last_selection()


def test_per_element_budget():
    """The reference's own budget (internal/kernels/quant_test.go:45-117) on every output of a
    decode-shaped product: half a scale step per term against the ORIGINAL weights, plus the f32
    accumulation bound gamma(K - 1)."""
    M, K, N = 4, 2048, 512
    a = np.array([math.sin(i * 0.23) * 2 for i in range(M * K)], np.float32).reshape(M, K)
    w = np.array([math.cos(i * 0.31) * 1.5 for i in range(K * N)], np.float32)
    bq, bs = orc.int8_quantize(w)
    got = product(a, bq, bs, M, K, N).astype(np.float64)
    W = w.reshape(K, N).astype(np.float64)
    S = orc.from_f16_bits(bs).astype(np.float64)[(np.arange(K * N) // 32)].reshape(K, N)
    A = a.astype(np.float64)
    exact = A @ W
    nu = (K - 1) / (1 << 24)
    budget = np.abs(A) @ (S / 2) + nu / (1 - nu) * (np.abs(A) @ np.abs(W))
    assert np.all(np.abs(got - exact) <= budget)


def test_host_quantizer_is_bit_identical_to_the_oracle(rng):
    for n in (5, 64, 200, 4096 * 3 + 7):
        w = (rng.standard_normal(n) * 0.3).astype(np.float32)
        q, s = quant.int8_quantize(w)
        oq, os_ = orc.int8_quantize(w)
        assert np.array_equal(q, oq) and np.array_equal(s, os_)
        assert np.array_equal(quant.int8_dequantize(q, s), orc.int8_dequantize(oq, os_))


def test_refusals():
    x = torch.zeros(2, 64, device=DEV)
    good = T.Quantized(torch.zeros(64, 32, dtype=torch.int8, device=DEV), torch.zeros(64, dtype=torch.float16, device=DEV))
    with pytest.raises(T.Refused, match="blocks of 32"):
        T.quant_matmul(x, T.Quantized(good.quants, good.scales[:10]))
    with pytest.raises(T.Refused, match="must be i8"):
        T.quant_matmul(x, T.Quantized(good.quants.int(), good.scales))
    with pytest.raises(T.Refused, match="contracted axes"):
        T.quant_matmul(torch.zeros(2, 48, device=DEV), good)
    with pytest.raises(T.Refused, match="f32-activation"):
        T.quant_matmul(x.half(), good)
