"""The decode-batch int4 kernel over prepacked weights (bulk copies, tensor memory, tcgen05)
against the oracle, through the C ABI: ab_int4_prepack, then QuantMatVecInt4Packed /
QuantMatMulInt4Packed by name.  Tolerance 1e-3 relative (max-norm) as for every int4 product, plus
the reference's per-element bound (internal/kernels/int4_test.go:99-182)."""
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
    if M == 1:
        runtime.launch("QuantMatVecInt4Packed", [x[0], packed, out], runtime.gemm_dims(0, N, K))
    else:
        runtime.launch("QuantMatMulInt4Packed", [x, packed, out], runtime.gemm_dims(M, N, K))
    torch.cuda.synchronize()
    quant.int4_stream_check()
    return out.cpu().numpy()


def oracle_product(a, p, s, z, M, K, N):
    if M == 1:
        return orc.quant_matvec_int4(a[0], p, s, z, N, K)[None, :]
    return orc.quant_matmul_int4(a, p, s, z, M, N, K)


@pytest.mark.parametrize("M,K,N", [(1, 4096, 4096), (1, 4096, 11008), (16, 4096, 11008), (16, 4096, 4096),
                                   (16, 11008, 4096), (8, 4096, 12288), (32, 4096, 11008), (20, 1024, 384),
                                   (3, 64, 128), (5, 100, 256), (16, 4100, 512), (40, 512, 256),
                                   (1, 4096, 32000)])
def test_matches_the_oracle(M, K, N):
    w = normal(2, (K, N), 0.02)
    w.reshape(-1)[3 * N:3 * N + 128] = 0.25          # constant groups: scale 0, value in the zero point
    w.reshape(-1)[K * N - 128:] = -0.125
    p, s, z = orc.int4_quantize(w)
    a = normal(1, (M, K))
    got = product(a, packed_of(p, s, z, K, N), M, K, N)
    # up to 48 rows: passes of the decode kernel; beyond: the tile kernel over the same stream
    assert ("stream kernel" if M <= 48 else "tile kernel") in runtime.last_selection()
    assert_close(got, oracle_product(a, p, s, z, M, K, N), GEMM_TOL, f"int4 packed M={M} K={K} N={N}")


@pytest.mark.parametrize("factor", [1e-4, 1e4, 1e-20, 1e20])
@pytest.mark.parametrize("M", [1, 16])
def test_activation_magnitude_does_not_matter(M, factor):
    # the f16 operand is scaled per row by an exact power of two, so tiny and huge activations keep
    # the accuracy of ordinary ones (the reference's f32 arithmetic is scale-invariant)
    K, N = 4096, 1024
    w = normal(4, (K, N), 0.02)
    p, s, z = orc.int4_quantize(w)
    a = normal(5, (M, K)) * np.float32(factor)
    if M > 1:
        a[1] *= np.float32(1e-3)                      # rows of very different magnitude in one call
    got = product(a, packed_of(p, s, z, K, N), M, K, N)
    want = oracle_product(a, p, s, z, M, K, N)
    for m in range(M):
        assert_close(got[m], want[m], GEMM_TOL, f"row {m} at activations x {factor:g}")


@pytest.mark.parametrize("std", [1e-5, 30.0])
def test_weight_magnitude_does_not_matter(std):
    M, K, N = 16, 2048, 512
    w = normal(6, (K, N), std)
    p, s, z = orc.int4_quantize(w)
    a = normal(7, (M, K))
    got = product(a, packed_of(p, s, z, K, N), M, K, N)
    assert_close(got, oracle_product(a, p, s, z, M, K, N), GEMM_TOL, f"weights of std {std:g}")


@pytest.mark.parametrize("M,K,N", [(1, 4096, 4096), (16, 4096, 11008)])
def test_per_element_bound(M, K, N):
    """|y - y_f64| <= (gamma(K) + 2^-11) * sum_k |a_k| |w_k| for EVERY output, not only against the
    largest one: gamma(K) is the reference's bound for its own f32 accumulation
    (internal/kernels/int4_test.go:99-182, specs/008-numerics.md), 2^-11 the one rounded operand."""
    w = normal(8, (K, N), 0.02)
    p, s, z = orc.int4_quantize(w)
    a = normal(9, (M, K))
    back = orc.int4_dequantize(p, s, z, w.size)
    want, mag = orc.matmul_definition_f64(a, back, M, N, K)
    got = product(a, packed_of(p, s, z, K, N), M, K, N)
    nu = (K - 1) * 2.0 ** -24
    bound = (nu / (1 - nu) + 2.0 ** -11) * mag
    assert np.all(np.abs(got - want) <= bound), float(np.max(np.abs(got - want) / mag))


def test_the_prepack_is_a_permutation_of_the_reference_planes():
    K, N = 192, 256
    w = normal(10, (K, N), 0.02)
    p, s, z = orc.int4_quantize(w)
    raw = packed_of(p, s, z, K, N).cpu().numpy().view(np.uint8)
    header = 256
    codes = np.array([orc.int4_nibble(p, i) for i in range(K * N)], np.uint8).reshape(K, N)
    pos = [0, 4, 1, 5, 2, 6, 3, 7]
    smax = orc.from_f16_bits(s).reshape(K, N // 128).max(axis=0)
    es = np.exp2(np.floor(np.log2(smax))).astype(np.float32)      # the header: 2^floor(log2(largest scale))
    for g in range(N // 128):
        for c in range(K // 64):
            blk = raw[header + (g * (K // 64) + c) * 4352:][:4352]
            words = blk[:4096].view(np.uint32).reshape(2, 128, 4)
            for h in range(2):
                for i in range(4):
                    for j in range(8):
                        k = 64 * c + 32 * h + 8 * i + j
                        got = (words[h, :, i] >> (4 * pos[j])) & 0xF
                        assert np.array_equal(got, codes[k, 128 * g:128 * g + 128]), (g, c, h, i, j)
            # scales are normalised by the group's power of two; rows whose codes sit four bits up
            # in the kernel's A operand carry 1/16 in their scale and 16 in their zero
            sc, zr = (blk[4096:4224].view(np.float16).astype(np.float32),
                      blk[4224:].view(np.float16).astype(np.float32))
            up = (np.arange(64) & 2) != 0
            s_ref = orc.from_f16_bits(s).reshape(K, N // 128)[64 * c:64 * c + 64, g]
            z_ref = orc.from_f16_bits(z).reshape(K, N // 128)[64 * c:64 * c + 64, g]
            assert np.array_equal(sc, s_ref / es[g] * np.where(up, 1 / 16, 1).astype(np.float32))
            assert np.array_equal(zr, z_ref * np.where(up & (s_ref != 0), 16, 1).astype(np.float32))
    assert np.array_equal(raw[:8].view(np.float32), es)


def test_the_three_output_form_equals_the_plain_product_bit_for_bit():
    """q | k | v side by side: one product whose column ranges land in three contiguous outputs."""
    M, K, N1, N2, N3 = 16, 1024, 512, 256, 256
    N = N1 + N2 + N3
    w = normal(12, (K, N), 0.02)
    p, s, z = orc.int4_quantize(w)
    packed = packed_of(p, s, z, K, N)
    a = torch.from_numpy(normal(13, (M, K))).to(DEV)
    whole = torch.empty(M, N, device=DEV)
    runtime.launch("QuantMatMulInt4Packed", [a, packed, whole], runtime.gemm_dims(M, N, K))
    o = [torch.full((M, n), float("nan"), device=DEV) for n in (N1, N2, N3)]
    import struct
    runtime.launch("QuantMatMulInt4PackedSplit3", [a, packed, *o], struct.pack("<IIIIIIII", M, N, K, N1, N2, 0, 0, 0))
    torch.cuda.synchronize()
    quant.int4_stream_check()
    assert torch.equal(torch.cat(o, dim=1), whole)


@pytest.mark.parametrize("M,K,F", [(16, 4096, 11008), (3, 512, 256), (1, 256, 128)])
def test_the_swiglu_epilogue_equals_the_product_followed_by_swiglu(M, K, F):
    """gate and up interleaved by 128-column group; out = SwiGLU(gate, up) from the epilogue against
    the two products' columns pulled apart and the SwiGLU kernel, and against the oracle."""
    wg, wu = normal(14, (K, F), 0.02), normal(15, (K, F), 0.02)
    qg, qu = orc.int4_quantize(wg), orc.int4_quantize(wu)
    G = F // 128
    inter = lambda x, y, per: np.stack([x.reshape(K, G, per), y.reshape(K, G, per)], axis=2).reshape(-1)
    p = inter(qg[0], qu[0], 16)
    s = inter(qg[1], qu[1], 1)
    z = inter(qg[2], qu[2], 1)
    packed = packed_of(p, s, z, K, 2 * F)
    a_np = normal(16, (M, K))
    a = torch.from_numpy(a_np).to(DEV)
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
    # the plain product may pick another K split (other order of the partial sums): equal within a few ulps
    assert_close(out.cpu().numpy(), want.cpu().numpy(), 1e-5, "SwiGLU epilogue against the chain")
    mm = (lambda q: orc.quant_matmul_int4(a_np, *q, M, F, K)) if M > 1 else \
        (lambda q: orc.quant_matvec_int4(a_np[0], *q, F, K)[None, :])
    assert_close(out.cpu().numpy(), orc.swiglu(mm(qg), mm(qu)), 2e-3, "SwiGLU epilogue against the oracle")


@pytest.mark.parametrize("M", [1, 16, 40])
def test_the_forms_that_take_the_rows_maxima_equal_the_plain_forms(M):
    """AddRMSNormAmax leaves every row's largest |norm| and the ...A products take it as a binding
    instead of running a kernel of their own for it: same factors, same kernels, so the results are
    bit-identical to AddRMSNorm followed by the plain packed products."""
    import struct
    K, F = 1024, 512
    rng = np.random.default_rng(33)
    x, delta = normal(40, (M, K)), normal(41, (M, K))
    gain = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    dx, dd, dg = (torch.from_numpy(t).to(DEV) for t in (x, delta, gain))
    s0, h0 = torch.empty(M, K, device=DEV), torch.empty(M, K, device=DEV)
    s1, h1 = torch.empty(M, K, device=DEV), torch.empty(M, K, device=DEV)
    amax = torch.full((M,), float("nan"), device=DEV)
    runtime.launch("AddRMSNorm", [dx, dd, dg, s0, h0], runtime.row_dims(M, K, 1e-5))
    runtime.launch("AddRMSNormAmax", [dx, dd, dg, s1, h1, amax], runtime.row_dims(M, K, 1e-5))
    torch.cuda.synchronize()
    assert torch.equal(s0, s1) and torch.equal(h0, h1)
    assert torch.equal(amax, h0.abs().max(dim=1).values)
    # plain, three-output and SwiGLU products, with and without the maxima
    N = 2 * F
    p, s, z = orc.int4_quantize(normal(42, (K, N), 0.02))
    packed = packed_of(p, s, z, K, N)
    a0, a1 = torch.empty(M, N, device=DEV), torch.full((M, N), float("nan"), device=DEV)
    runtime.launch("QuantMatMulInt4Packed", [h0, packed, a0], runtime.gemm_dims(M, N, K))
    runtime.launch("QuantMatMulInt4PackedA", [h0, amax, packed, a1], runtime.gemm_dims(M, N, K))
    assert torch.equal(a0, a1)
    u3 = struct.pack("<IIIIIIII", M, N, K, 512, 256, 0, 0, 0)
    o0 = [torch.empty(M, n, device=DEV) for n in (512, 256, 256)]
    o1 = [torch.full((M, n), float("nan"), device=DEV) for n in (512, 256, 256)]
    runtime.launch("QuantMatMulInt4PackedSplit3", [h0, packed, *o0], u3)
    runtime.launch("QuantMatMulInt4PackedSplit3A", [h0, amax, packed, *o1], u3)
    assert all(torch.equal(a, b) for a, b in zip(o0, o1))
    g0, g1 = torch.empty(M, F, device=DEV), torch.full((M, F), float("nan"), device=DEV)
    runtime.launch("QuantMatMulInt4PackedSwiGLU", [h0, packed, g0], runtime.gemm_dims(M, N, K))
    runtime.launch("QuantMatMulInt4PackedSwiGLUA", [h0, amax, packed, g1], runtime.gemm_dims(M, N, K))
    torch.cuda.synchronize()
    quant.int4_stream_check()
    assert torch.equal(g0, g1)


@pytest.mark.parametrize("M", [1, 5, 16, 33])
def test_row_maxima_in_parts(M):
    """The producer of a product's input may leave a row's largest magnitudes in parts (the attention
    kernels: one per head and warp; the SwiGLU product: one per 32 columns) and the product that
    follows takes the largest of a row's entries: bit-identical to the plain forms, whatever the
    split.  QuantMatMulInt4PackedSwiGLUAMax is the producer: its out equals ...SwiGLUA's and outmax
    holds the largest |out| of every 32 columns."""
    K, F = 1024, 512
    N = 2 * F
    p, s, z = orc.int4_quantize(normal(52, (K, N), 0.02))
    packed = packed_of(p, s, z, K, N)
    a = torch.from_numpy(normal(53, (M, K))).to(DEV)
    a[0, 7] = 300.0                                         # the maximum sits in one part only
    plain = torch.empty(M, N, device=DEV)
    runtime.launch("QuantMatMulInt4Packed", [a, packed, plain], runtime.gemm_dims(M, N, K))
    for parts in (1, 4, 32, 37):
        # a split of the columns into `parts` runs of unequal length; empty parts hold 0
        edges = np.unique(np.concatenate([[0, K], np.random.default_rng(parts).integers(0, K, parts - 1)]))
        amax = torch.zeros(M, parts, device=DEV)
        for i in range(len(edges) - 1):
            amax[:, i] = a[:, edges[i]:edges[i + 1]].abs().amax(dim=1)
        out = torch.full((M, N), float("nan"), device=DEV)
        runtime.launch("QuantMatMulInt4PackedA", [a, amax, packed, out], struct.pack("<IIII", M, N, K, parts))
        torch.cuda.synchronize()
        assert torch.equal(out, plain), parts
    one = a.abs().amax(dim=1).contiguous()
    g0, g1 = torch.empty(M, F, device=DEV), torch.full((M, F), float("nan"), device=DEV)
    gmax = torch.full((M, N // 64), float("nan"), device=DEV)
    runtime.launch("QuantMatMulInt4PackedSwiGLUA", [a, one, packed, g0], runtime.gemm_dims(M, N, K))
    runtime.launch("QuantMatMulInt4PackedSwiGLUAMax", [a, one, packed, g1, gmax], runtime.gemm_dims(M, N, K))
    torch.cuda.synchronize()
    quant.int4_stream_check()
    assert torch.equal(g0, g1)
    assert torch.equal(gmax, g1.view(M, F // 32, 32).abs().amax(dim=2))
    # and the product that reads it next
    K2 = F
    p2, s2, z2 = orc.int4_quantize(normal(54, (K2, 256), 0.02))
    packed2 = packed_of(p2, s2, z2, K2, 256)
    d0, d1 = torch.empty(M, 256, device=DEV), torch.full((M, 256), float("nan"), device=DEV)
    runtime.launch("QuantMatMulInt4Packed", [g1, packed2, d0], runtime.gemm_dims(M, 256, K2))
    runtime.launch("QuantMatMulInt4PackedA", [g1, gmax, packed2, d1], struct.pack("<IIII", M, 256, K2, N // 64))
    torch.cuda.synchronize()
    assert torch.equal(d0, d1)


def test_the_form_that_leaves_maxima_refuses_the_batch_kernel():
    M, K, N = 64, 256, 512
    p, s, z = orc.int4_quantize(normal(55, (K, N), 0.02))
    packed = packed_of(p, s, z, K, N)
    a = torch.zeros(M, K, device=DEV)
    with pytest.raises(Exception, match="decode kernel"):
        runtime.launch("QuantMatMulInt4PackedSwiGLUAMax", [a, torch.zeros(M, device=DEV), packed,
                                                           torch.zeros(M, N // 2, device=DEV),
                                                           torch.zeros(M, N // 64, device=DEV)], runtime.gemm_dims(M, N, K))
