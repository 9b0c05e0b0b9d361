"""What can be checked without a GPU: the library loads, exports every symbol the header declares,
refuses what it must, and its host-side pieces (quantizer, f16, block pool, shard split) are
bit-identical to the oracle."""
import ctypes as C
import re
import struct
from pathlib import Path

import numpy as np
import pytest

import oracle as orc
from accel_b200 import _lib, quant, runtime
from accel_b200.blockpool import BlockPool

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "accel_b200.h").read_text()
    declared = set(re.findall(r"AB_API\s+[^;(]*?\b(ab_\w+)\s*\(", header))
    assert len(declared) >= 40
    L = C.CDLL(str(_lib.LIB_PATH))
    for name in declared:
        assert hasattr(L, name), f"{name} is declared in the header and missing from the library"
    bound = {s[0] for s in _lib.SYMBOLS}
    assert declared == bound, declared ^ bound


def test_kernel_registry_names_the_reference_kernels():
    names = set(runtime.kernel_names())
    for n in ["QuantMatVecInt4", "QuantMatMulInt4", "AttentionDecode", "AttentionDecodeF16",
              "AttentionDecodePaged", "AttentionDecodePagedF16", "AttentionDecodeBatched",
              "AttentionRagged", "AttentionRaggedF16", "GroupedMatVec", "GroupedMatMul",
              "SegmentOffsets", "ScatterRows", "ScatterRowsF16", "GatherRows", "RMSNorm", "RoPE",
              "SwiGLU", "ElemAdd", "SampleArgmax", "CastF32ToF16"]:
        assert n in names


def test_every_registered_kernel_is_documented_in_the_header():
    """include/accel_b200.h lists every kernel name ab_launch dispatches, with its bindings and uniform."""
    header = (ROOT / "include" / "accel_b200.h").read_text()
    words = set(re.findall(r"[A-Za-z0-9_]+", header))
    missing = [n for n in runtime.kernel_names() if n not in words]
    assert not missing, missing


def test_the_forms_with_row_maxima_are_registered_with_their_binding_counts():
    # AttentionDecodeBatchedMax: the seventh binding holds four maxima per head
    lens = [32 * 32 * 128, 1, 1, 32 * 256, 32, 32 * 32 * 128, 32 * 32 * 4]
    u = runtime.batched_dims(32, 32, 8, 128, 16, 256, 0.088)
    assert runtime.workspace_bytes("AttentionDecodeBatchedMax", lens, u) == \
        runtime.workspace_bytes("AttentionDecodeBatched", lens[:6], u)
    with pytest.raises(_lib.AccelError, match="takes 7 bindings"):
        runtime.workspace_bytes("AttentionDecodeBatchedMax", lens[:6], u)
    # the decode kernel takes its rows' maxima as a binding and needs no scratch for them
    M, K, N = 16, 4096, 11008
    packed_words = (_lib.lib().ab_int4_prepack_bytes(K, N) + 3) // 4
    assert runtime.workspace_bytes("QuantMatMulInt4PackedA", [M * K, M * 32, packed_words, M * N],
                                   struct.pack("<IIII", M, N, K, 32)) == 0
    assert runtime.workspace_bytes("QuantMatMulInt4Packed", [M * K, packed_words, M * N],
                                   runtime.gemm_dims(M, N, K)) > 0


def test_an_unknown_kernel_is_a_refusal_not_a_fallback():
    L = _lib.lib()
    lens = (C.c_uint32 * 1)(4)
    out = C.c_size_t(0)
    rc = L.ab_workspace_bytes(b"MatMulTiled", lens, 1, None, 0, C.byref(out))
    assert rc == _lib.AB_ERR_UNSUPPORTED
    assert b"no CPU fallback" in L.ab_last_error()
    assert L.ab_supports_kernel(None, b"QuantMatVecInt4", None) == _lib.AB_OK
    assert L.ab_supports_kernel(None, b"LinearAttention", None) == _lib.AB_ERR_UNSUPPORTED


def test_workspace_query_and_argument_checks_need_no_gpu():
    # QuantMatVecInt4 at K=4096, N=4096 adds its K splits inside a thread-block cluster: no scratch
    need = runtime.workspace_bytes("QuantMatVecInt4", [4096, 2097152, 131072, 131072, 4096],
                                   runtime.gemm_dims(0, 4096, 4096))
    assert need == 0
    # 16 rows against the 4096 x 32000 vocabulary matrix do not fit one wave of clusters: that
    # product splits K across CTAs and needs one partial [M, N] tile per split
    M, K, N = 16, 4096, 32000
    need = runtime.workspace_bytes("QuantMatMulInt4", [M * K, K * N // 8, K * N // 128, K * N // 128, M * N],
                                   runtime.gemm_dims(M, N, K))
    # (the partial tiles, then the rows' largest magnitudes and the activations scaled by them)
    assert need >= 2 * M * N * 4 + M * 4 + M * K * 4
    with pytest.raises(_lib.AccelError, match="takes 5 bindings"):
        runtime.workspace_bytes("QuantMatVecInt4", [1, 2], runtime.gemm_dims(0, 4096, 4096))
    with pytest.raises(_lib.AccelError, match="uniform block"):
        runtime.workspace_bytes("QuantMatVecInt4", [1, 2, 3, 4, 5], None)
    # batched attention: 16 partitions of 256 positions over a 4096-position reach
    need = runtime.workspace_bytes("AttentionDecodeBatched",
                                   [32 * 32 * 128, 1, 1, 32 * 256, 32, 32 * 32 * 128],
                                   runtime.batched_dims(32, 32, 8, 128, 16, 256, 0.088))
    assert need >= 32 * 32 * 16 * 128 * 4


def test_torch_cpu_tensors_are_refused():
    import torch
    with pytest.raises(_lib.AccelError, match="no CPU path"):
        runtime.launch("ElemAdd", [torch.zeros(4), torch.zeros(4), torch.zeros(4)])


@pytest.mark.parametrize("n", [128, 129, 8, 5, 128 * 300 + 77, 1 << 20])
def test_host_quantizer_is_bit_identical_to_the_oracle(n):
    rng = np.random.default_rng(n)
    w = (rng.standard_normal(n) * 0.02).astype(np.float32)
    if n > 1000:
        w[128:256] = 0.75                      # a constant group
        w[256:384] = w[256] + rng.standard_normal(128).astype(np.float32) * 1e-9   # underflow
        w[384:512] += 1000                     # large zero point
    got, want = quant.int4_quantize(w), orc.int4_quantize(w)
    for g, x in zip(got, want):
        assert np.array_equal(g, x)
    assert np.array_equal(quant.int4_dequantize(*got, n), orc.int4_dequantize(*want, n))
    for i in (0, 1, n // 2, n - 1):
        assert quant.int4_nibble(got[0], i) == orc.int4_nibble(want[0], i)


@pytest.mark.parametrize("n", [5, 64, 200, 4096 * 3 + 7])
def test_int8_host_quantizer_is_bit_identical_to_the_oracle(n, rng):
    w = (rng.standard_normal(n) * 0.3).astype(np.float32)
    q, s = quant.int8_quantize(w)
    oq, os_ = orc.int8_quantize(w)
    assert np.array_equal(q, oq) and np.array_equal(s, os_)
    assert np.array_equal(quant.int8_dequantize(q, s), orc.int8_dequantize(oq, os_))


def test_reference_packing_fixtures_through_the_c_abi():
    # quant/int4_test.go:261-286 and :225-253
    w = np.full(128, 0.5, np.float32)
    w[0], w[1] = 0, 10
    p, _, _ = quant.int4_quantize(w)
    assert quant.int4_nibble(p, 0) == 0 and quant.int4_nibble(p, 1) == 15 and int(p[0]) & 0xFF == 0xF0
    w = (np.arange(129) % 16).astype(np.float32) / 4
    p, s, z = quant.int4_quantize(w)
    assert p.size == 17 and quant.int4_dequantize(p, s, z, 129)[-1] == w[-1]
    for c in (0.0, 1.0, -2.5, 0.125):
        p, s, z = quant.int4_quantize(np.full(128, c, np.float32))
        assert np.all(quant.int4_dequantize(p, s, z, 128) == np.float32(c))


def test_f16_conversion_matches_the_oracle():
    L = _lib.lib()
    rng = np.random.default_rng(3)
    xs = (rng.standard_normal(20000) * np.exp(rng.uniform(-20, 12, 20000))).astype(np.float32)
    xs[:6] = [0.0, -0.0, 3.1e-8, 65520.0, np.inf, np.nan]
    want = orc.to_f16_bits(xs)
    for x, wbits in zip(xs, want):
        xf = C.c_float(float(x))
        got = L.ab_f32_to_f16(C.byref(xf))
        assert got == int(wbits), (x, got, wbits)
    out = C.c_float(0)
    for h in (0x0001, 0x03ff, 0x3c00, 0x7bff, 0xfc00, 0x8000):
        L.ab_f16_to_f32(h, C.byref(out))
        assert out.value == orc.from_f16_bits([h])[0]


def test_block_pool_through_the_c_abi():
    # tensor/blockpool_test.go:16-91, and agreement with the oracle's pool on a longer script
    p = BlockPool(4, 8)
    assert p.block_size() == 8 and p.available() == 4
    a = p.grow(None, 9)
    assert a == [1, 0] and p.available() == 2 and p.positions(a) == 16
    b = p.grow(a, 17)
    assert b[:2] == a and len(b) == 3
    assert len(p.grow(b, 20)) == 3 and p.available() == 1
    with pytest.raises(_lib.AccelError, match="does not evict"):
        p.grow(b, 100)
    p.free(b)
    assert p.available() == 4
    with pytest.raises(_lib.AccelError, match="already free"):
        p.free(b)
    for bad in ((0, 8), (4, 0)):
        with pytest.raises(_lib.AccelError):
            BlockPool(*bad)
    with pytest.raises(_lib.AccelError):
        p.grow(None, -1)

    rng = np.random.default_rng(11)
    mine, ref = BlockPool(64, 16), orc.BlockPool(64, 16)
    seqs_m, seqs_r = {}, {}
    for step in range(300):
        s = int(rng.integers(0, 8))
        if s in seqs_m and rng.random() < 0.3:
            mine.free(seqs_m.pop(s))
            ref.free(seqs_r.pop(s))
            continue
        n = int(rng.integers(1, 200))
        try:
            gm = mine.grow(seqs_m.get(s), n)
        except _lib.AccelError:
            with pytest.raises(ValueError):
                ref.grow(seqs_r.get(s), n)
            continue
        seqs_m[s], seqs_r[s] = gm, ref.grow(seqs_r.get(s), n)
        assert seqs_m[s] == seqs_r[s] and mine.available() == ref.available()


def test_column_split_is_group_aligned_and_covers_every_column():
    for n_cols in (4096, 11008, 32000, 14336, 128):
        for parts in (1, 2, 4, 8):
            edges = [quant.int4_column_split(n_cols, parts, r) for r in range(parts)]
            assert edges[0][0] == 0 and edges[-1][1] == n_cols
            for (b0, e0), (b1, _) in zip(edges, edges[1:]):
                assert e0 == b1
            assert all(b % 128 == 0 and e % 128 == 0 for b, e in edges)
            sizes = [e - b for b, e in edges]
            assert max(sizes) - min(sizes) <= 128
    with pytest.raises(_lib.AccelError):
        quant.int4_column_split(1000, 2, 0)


def test_group_aligned_shards_pack_bit_identically(rng):
    # a column shard re-indexed as its own [K, N_shard] matrix holds the same codes, scales and
    # zeros as those columns of the full matrix
    K, N = 24, 1280
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    full = quant.int4_quantize(w)
    codes = np.array([quant.int4_nibble(full[0], i) for i in range(K * N)]).reshape(K, N)
    for r in range(4):
        b, e = quant.int4_column_split(N, 4, r)
        shard = quant.int4_quantize(np.ascontiguousarray(w[:, b:e]))
        sc = np.array([quant.int4_nibble(shard[0], i) for i in range(K * (e - b))]).reshape(K, e - b)
        assert np.array_equal(sc, codes[:, b:e])
        assert np.array_equal(shard[1].reshape(K, -1), full[1].reshape(K, -1)[:, b // 128:e // 128])
        assert np.array_equal(shard[2].reshape(K, -1), full[2].reshape(K, -1)[:, b // 128:e // 128])


def test_buckets():
    # tensor/cache.go:166-246 and tensor/cache_test.go: sorted, no duplicates, smallest that fits,
    # a prompt past the largest bucket is an error rather than a truncation
    from accel_b200.driver import Buckets
    b = Buckets(512, 128, 256)
    assert b.sizes() == [128, 256, 512]
    assert [b.for_(n) for n in (1, 100, 128, 129, 256, 300, 512)] == [128, 128, 128, 256, 256, 512, 512]
    with pytest.raises(ValueError, match="exceeds the largest bucket"):
        b.for_(513)
    with pytest.raises(ValueError, match="a prompt of 0"):
        b.for_(0)
    with pytest.raises(ValueError, match="appears twice"):
        Buckets(128, 128)
    with pytest.raises(ValueError, match="at least one"):
        Buckets()
    with pytest.raises(ValueError, match="positive"):
        Buckets(0, 4)


def test_plan_identity_is_structure_not_shape():
    from accel_b200 import driver as D
    from accel_b200 import runtime as rt
    o = lambda slot, size: D.Operand(slot=slot, size=size)
    base = [D.Dispatch("RMSNorm", [o(1, 4096), o(2, 1024), o(3, 4096)], rt.row_dims(4, 256, 1e-5))]
    same = [D.Dispatch("RMSNorm", [o(1, 4096), o(2, 1024), o(3, 4096)], rt.row_dims(4, 256, 1e-5))]
    other_kernel = [D.Dispatch("ElemAdd", [o(1, 4096), o(2, 1024), o(3, 4096)])]
    other_uniform = [D.Dispatch("RMSNorm", [o(1, 4096), o(2, 1024), o(3, 4096)], rt.row_dims(4, 256, 1e-6))]
    other_wiring = [D.Dispatch("RMSNorm", [o(3, 4096), o(2, 1024), o(1, 4096)], rt.row_dims(4, 256, 1e-5))]
    ident = D.plan_identity(base, 3)
    assert ident == D.plan_identity(same, 3)
    for p in (other_kernel, other_uniform, other_wiring):
        assert D.plan_identity(p, 3) != ident
    assert D.plan_identity(base, 4) != ident
    # a host write's payload is set per submission and is not part of what the plan is
    hw = lambda payload: [D.HostWrite(o(1, 16), payload)]
    assert D.plan_identity(hw(b"\0" * 16), 1) == D.plan_identity(hw(b"\1" * 16), 1)
