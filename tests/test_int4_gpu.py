"""Parity of the int4 linear kernels with the oracle, through the C ABI, on a B200.

Tolerance: 1e-3 relative with f32 accumulation, measured as max|y - y_ref| / max|y_ref| against
the order-faithful oracle and, at full size, against a binary64 product over the dequantized
weights.  Packing is bit-exact."""
import numpy as np
import pytest
import torch

import oracle as orc
from accel_b200 import _lib, quant, runtime
from accel_b200 import tensor as T
from util import GEMM_TOL, assert_close, normal

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def to_int4(packed, scales, zeros, n):
    return T.Int4(torch.from_numpy(packed.view(np.int32)).to(DEV),
                  torch.from_numpy(scales.view(np.float16)).to(DEV),
                  torch.from_numpy(zeros.view(np.float16)).to(DEV), n)


def quantized(seed, K, N, std=0.02):
    w = normal(seed, (K, N), std)          # flat [K, N]: w[k*N+n] = W[n][k]
    p, s, z = orc.int4_quantize(w)
    return w, p, s, z


def test_reference_known_answers_on_the_device():
    # internal/kernels/int4_test.go:189-228 (40, not 4) and :99-182 (constant group = 96)
    w = np.ones(8, np.float32)
    w[0], w[1] = 0, 4
    a = np.zeros(8, np.float32)
    a[0], a[1] = 1, 10
    p, s, z = orc.int4_quantize(w)
    out = T.int4_matvec(torch.from_numpy(a).to(DEV), to_int4(p, s, z, 8)).cpu().numpy()
    assert abs(out[0] - 40.0) <= 1

    K, N, M = 256, 2, 3
    rng = np.random.default_rng(5)
    w = np.empty(K * N, np.float32)
    w[:128] = 0.75
    w[128:] = rng.uniform(-1, 1, K * N - 128)
    p, s, z = orc.int4_quantize(w)
    a = np.ones((M, K), np.float32)
    want = orc.quant_matmul_int4(a, p, s, z, M, N, K)
    got = T.int4_matmul(torch.from_numpy(a).to(DEV), to_int4(p, s, z, K * N)).cpu().numpy()
    assert_close(got, want, 1e-5, "constant group")
    row = T.int4_matvec(torch.from_numpy(a[0]).to(DEV), to_int4(p, s, z, K * N)).cpu().numpy()
    assert_close(row, want[0], 1e-5, "constant group, row kernel")


@pytest.mark.parametrize("M,K,N", [(1, 4096, 4096), (1, 4096, 11008), (8, 4096, 11008),
                                   (32, 4096, 11008), (2, 11008, 4096), (3, 512, 384),
                                   (5, 100, 128), (1, 33, 256), (7, 4096, 128)])
def test_matches_the_oracle(M, K, N):
    w, p, s, z = quantized(2, K, N)
    a = normal(1, (M, K))
    want = orc.quant_matmul_int4(a, p, s, z, M, N, K) if M > 1 else \
        orc.quant_matvec_int4(a[0], p, s, z, N, K)[None, :]
    q = to_int4(p, s, z, K * N)
    if M == 1:
        got = T.int4_matvec(torch.from_numpy(a[0]).to(DEV), q).cpu().numpy()[None, :]
        assert "streaming row kernel" in runtime.last_selection()
    else:
        got = T.int4_matmul(torch.from_numpy(a).to(DEV), q).cpu().numpy()
        # the tensor-core kernels walk K in steps of 16 rows; other depths stay on the CUDA cores
        assert ("tensor-core kernel" if K % 16 == 0 else "row kernel") in runtime.last_selection()
    assert_close(got, want, GEMM_TOL, f"int4 M={M} K={K} N={N}")


@pytest.mark.parametrize("M,K,N", [(3, 50, 37), (9, 130, 19), (1, 8, 1), (4, 64, 200)])
def test_shapes_whose_groups_straddle_rows(M, K, N):
    # N is not a multiple of 128: groups run across row ends and the last word is partial
    w, p, s, z = quantized(7, K, N, std=1.0)
    a = normal(8, (M, K))
    want = orc.quant_matmul_int4(a, p, s, z, M, N, K)
    got = T.int4_matmul(torch.from_numpy(a).to(DEV), to_int4(p, s, z, K * N)).cpu().numpy()
    assert "generic" in runtime.last_selection()
    assert_close(got, want, GEMM_TOL, f"odd shape {M}x{K}x{N}")


def test_scales_and_zeros_are_read_per_group_along_n():
    # every group gets its own range, so a kernel that took groups along K, or the neighbour's
    # scale, is wrong by a factor rather than a rounding
    K, N = 64, 512
    rng = np.random.default_rng(9)
    w = np.empty((K, N), np.float32)
    for k in range(K):
        for g in range(N // 128):
            lo = rng.uniform(-4, 4)
            w[k, g * 128:(g + 1) * 128] = rng.uniform(lo, lo + rng.uniform(0.01, 3), 128)
    w[3, 128:256] = -1.5           # constant groups carry their value in the zero point
    w[40, 0:128] = 0.0
    p, s, z = orc.int4_quantize(w)
    a = normal(10, (4, K))
    want = orc.quant_matmul_int4(a, p, s, z, 4, N, K)
    got = T.int4_matmul(torch.from_numpy(a).to(DEV), to_int4(p, s, z, K * N)).cpu().numpy()
    assert_close(got, want, GEMM_TOL, "per-group metadata")


@pytest.mark.parametrize("M", [128, 512])
def test_full_size_against_a_binary64_product(M):
    # K=4096, N=11008 at the larger batch sizes: the oracle's scalar loop is minutes here, so the
    # reference is the definition in binary64 over the dequantized weights (torch, on the device)
    K, N = 4096, 11008
    w, p, s, z = quantized(2, K, N)
    back = orc.int4_dequantize(p, s, z, K * N).reshape(K, N)
    a = normal(1, (M, K))
    want = (torch.from_numpy(a).to(DEV).double() @ torch.from_numpy(back).to(DEV).double()).cpu().numpy()
    got = T.int4_matmul(torch.from_numpy(a).to(DEV), to_int4(p, s, z, K * N)).cpu().numpy()
    assert "tile kernel" in runtime.last_selection()    # large batches take 128-row tensor-core tiles
    assert_close(got, want, GEMM_TOL, f"full size M={M}")
    # and a sample of rows against the order-faithful oracle
    rows = [0, M // 2, M - 1]
    wo = orc.quant_matmul_int4(a[rows], p, s, z, len(rows), N, K)
    assert_close(got[rows], wo, GEMM_TOL, "oracle rows")


@pytest.mark.parametrize("M,K,N", [(1, 4096, 4096), (16, 4096, 11008)])
def test_per_element_bound_on_the_reference_layout(M, K, N):
    """The bound the reference states for its own kernels, applied to EVERY output of the kernels
    that read quant.Int4Quantize's planes (not only relative to the largest output):
    |y - y_f64| <= (gamma(K) + 2^-11) * sum_k |a_k| |w_k|, gamma(K) for the f32 accumulation
    (internal/kernels/int4_test.go:99-182), 2^-11 for the one operand rounded to f16."""
    w, p, s, z = quantized(8, K, N)
    a = normal(9, (M, K))
    back = orc.int4_dequantize(p, s, z, w.size)
    want, mag = orc.matmul_definition_f64(a, back, M, N, K)
    x = torch.from_numpy(a).to(DEV)
    if M == 1:
        got = T.int4_matvec(x[0], to_int4(p, s, z, K * N)).cpu().numpy()[None, :]
    else:
        got = T.int4_matmul(x, to_int4(p, s, z, K * N)).cpu().numpy()
    nu = (K - 1) * 2.0 ** -24
    bound = (nu / (1 - nu) + 2.0 ** -11) * mag
    assert np.all(np.abs(got - want) <= bound), float(np.max(np.abs(got - want) / mag))


@pytest.mark.parametrize("factor", [1e-4, 1e4, 1e-20, 1e20])
@pytest.mark.parametrize("M,K,N,kernel", [(1, 4096, 1024, "streaming row kernel"), (16, 4096, 1024, "cluster"),
                                          (4, 4096, 32000, "column groups x"), (80, 1024, 512, "tile kernel")])
def test_activation_magnitude_does_not_matter_on_the_reference_layout(M, K, N, kernel, factor):
    """The kernels over quant.Int4Quantize's planes round a * s to f16; each scales its activation
    rows by an exact power of two first (undone in f32), so tiny and huge activations keep the
    accuracy of ordinary ones, as the reference's f32 arithmetic does: the row kernel, the 16-row
    cluster kernel, the two-kernel form for wide matrices and the tile kernel."""
    w, p, s, z = quantized(4, K, N)
    a = normal(5, (M, K)) * np.float32(factor)
    if M > 1:
        a[1] *= np.float32(1e-3)                          # rows of very different magnitude in one call
    x = torch.from_numpy(a).to(DEV)
    if M == 1:
        got = T.int4_matvec(x[0], to_int4(p, s, z, K * N)).cpu().numpy()[None, :]
        want = orc.quant_matvec_int4(a[0], p, s, z, N, K)[None, :]
    else:
        got = T.int4_matmul(x, to_int4(p, s, z, K * N)).cpu().numpy()
        want = orc.quant_matmul_int4(a, p, s, z, M, N, K)
    assert kernel in runtime.last_selection(), runtime.last_selection()
    for m in range(M):
        assert_close(got[m], want[m], GEMM_TOL, f"row {m} at activations x {factor:g}")


def test_device_quantizer_is_bit_identical(rng):
    n = 128 * 4000 + 77
    w = (rng.standard_normal(n) * 0.02).astype(np.float32)
    w[128:256] = 0.75
    w[256:384] = w[256] + (rng.standard_normal(128) * 1e-9).astype(np.float32)
    w[384:512] += 1000
    w[512:640] = np.abs(w[512:640])
    w[512] = 0.0
    p, s, z = quant.int4_quantize_device(torch.from_numpy(w).to(DEV))
    wp, ws, wz = orc.int4_quantize(w)
    assert np.array_equal(p.cpu().numpy().view(np.uint32), wp)
    assert np.array_equal(s.cpu().numpy().view(np.uint16), ws)
    assert np.array_equal(z.cpu().numpy().view(np.uint16), wz)


def test_refusals():
    # tensor/int4_test.go:121-265: every validation branch refuses before anything is launched
    K, N = 64, 128
    _, p, s, z = quantized(1, K, N)
    q = to_int4(p, s, z, K * N)
    a = torch.zeros(K, device=DEV)
    with pytest.raises(T.Refused, match="must be u32"):
        T.int4_matvec(a, T.Int4(q.codes.float(), q.scales, q.zeros, q.weights))
    with pytest.raises(T.Refused, match="must be f16"):
        T.int4_matvec(a, T.Int4(q.codes, q.scales.float(), q.zeros, q.weights))
    with pytest.raises(T.Refused, match="declares 0 weights"):
        T.int4_matvec(a, T.Int4(q.codes, q.scales, q.zeros, 0))
    with pytest.raises(T.Refused, match="words"):
        T.int4_matvec(a, T.Int4(q.codes[:-1], q.scales, q.zeros, q.weights))
    with pytest.raises(T.Refused, match="groups"):
        T.int4_matvec(a, T.Int4(q.codes, q.scales[:-1], q.zeros, q.weights))
    with pytest.raises(T.Refused, match="zero plane"):
        T.int4_matvec(a, T.Int4(q.codes, q.scales, None, q.weights))
    with pytest.raises(T.Refused, match="reads f32"):
        T.int4_matvec(a.half(), q)
    with pytest.raises(T.Refused, match="takes a vector"):
        T.int4_matvec(torch.zeros(2, K, device=DEV), q)
    with pytest.raises(T.Refused, match="multiple of the first"):
        T.int4_matvec(torch.zeros(K + 1, device=DEV), q)
    with pytest.raises(T.Refused, match="batched form"):
        T.int4_matmul(a, q)
    # and at the C ABI: a lengths block that does not cover the shape launches nothing
    out = torch.zeros(N, device=DEV)
    with pytest.raises(_lib.AccelError, match="lengths block"):
        runtime.launch("QuantMatVecInt4", [a, q.codes, q.scales, q.zeros, out],
                       runtime.gemm_dims(0, N, K * 2))
