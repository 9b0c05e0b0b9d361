"""CPU oracle for the quantized decode path.  TEST INFRASTRUCTURE ONLY.

`accel_oracle.c` restates the arithmetic of golang-design/accel's CPU backend for the int4 linear,
the paged decode attention, the grouped product and the support operators of a decode step, in the
reference's summation order.  This package compiles it with gcc and binds it with ctypes.

Nothing in the product package may import this module: it is loaded only by the test-suite, by the
smoke check and by the benchmark's CPU-baseline leg, and always as the checker or the reported
baseline, never as the thing shipped.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SRC = _HERE / "accel_oracle.c"
_LIB = _HERE / "_build" / "liboracle.so"

u32p = np.ctypeslib.ndpointer(dtype=np.uint32, flags="C_CONTIGUOUS")
u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
f64p = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")


def build(force: bool = False) -> Path:
    """Compile the restatement.  -ffp-contract=off keeps every product and sum a separate
    binary32 rounding, which is what the reference's lowering spells with explicit conversions."""
    if not force and _LIB.exists() and _LIB.stat().st_mtime >= _SRC.stat().st_mtime:
        return _LIB
    _LIB.parent.mkdir(exist_ok=True)
    cmd = ["gcc", "-O2", "-std=c11", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-fPIC",
           "-shared", "-fvisibility=hidden", str(_SRC), "-o", str(_LIB), "-lm"]
    subprocess.run(cmd, check=True)
    return _LIB


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(build()))
        L = _lib
        L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_int4_error_bound.restype = C.c_double
        L.orc_int4_nibble.restype = C.c_uint32
        L.orc_blockpool_new.restype = C.c_void_p
        L.orc_set_threads.argtypes = [C.c_int]
        L.orc_max_threads.restype = C.c_int
    return _lib


def threads() -> int:
    """How many host threads the OpenMP loops use right now."""
    return int(lib().orc_max_threads())


def host_cores() -> int:
    """Cores this process may run on (its affinity mask, else every core)."""
    try:
        return len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        return os.cpu_count() or 1


def set_threads(n: int | None = None) -> int:
    """Sets the OpenMP thread count of the loops (default: every core this process may use),
    whatever OMP_NUM_THREADS said when the library was loaded.  Returns the count in use."""
    lib().orc_set_threads(int(n) if n else host_cores())
    return threads()


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def _vp(a):
    return a.ctypes.data_as(C.c_void_p)


# ---------------------------------------------------------------- f16
def to_f16_bits(x) -> np.ndarray:
    x = _c(x, np.float32).ravel()
    out = np.empty(x.size, np.uint16)
    lib().orc_cast_f32_to_f16(_vp(x), _vp(out), C.c_size_t(x.size))
    return out


def from_f16_bits(h) -> np.ndarray:
    h = _c(h, np.uint16).ravel()
    out = np.empty(h.size, np.float32)
    lib().orc_cast_f16_to_f32(_vp(h), _vp(out), C.c_size_t(h.size))
    return out


# ---------------------------------------------------------------- int4
def int4_quantize(w, group: int = 128):
    w = _c(w, np.float32).ravel()
    n = w.size
    packed = np.zeros((n + 7) // 8, np.uint32)
    groups = (n + group - 1) // group
    scales = np.zeros(groups, np.uint16)
    zeros = np.zeros(groups, np.uint16)
    lib().orc_int4_quantize(_vp(w), C.c_size_t(n), _vp(packed), _vp(scales), _vp(zeros),
                            C.c_uint32(group))
    return packed, scales, zeros


def int4_nibble(packed, i: int) -> int:
    packed = _c(packed, np.uint32)
    return int(lib().orc_int4_nibble(_vp(packed), C.c_size_t(i)))


def int4_dequantize(packed, scales, zeros, n: int, group: int = 128) -> np.ndarray:
    packed, scales, zeros = _c(packed, np.uint32), _c(scales, np.uint16), _c(zeros, np.uint16)
    out = np.empty(n, np.float32)
    lib().orc_int4_dequantize(_vp(packed), _vp(scales), _vp(zeros), C.c_size_t(n), _vp(out),
                              C.c_uint32(group))
    return out


def int4_error_bound(x, term_scales, term_zeros) -> float:
    x, ts, tz = _c(x, np.float32), _c(term_scales, np.uint16), _c(term_zeros, np.uint16)
    assert x.size == ts.size == tz.size
    return float(lib().orc_int4_error_bound(_vp(x), _vp(ts), _vp(tz), C.c_size_t(x.size)))


def quant_matvec_int4(a, bq, bs, bz, N: int, K: int, group: int = 128) -> np.ndarray:
    a, bq, bs, bz = _c(a, np.float32), _c(bq, np.uint32), _c(bs, np.uint16), _c(bz, np.uint16)
    out = np.zeros(N, np.float32)
    lib().orc_quant_matvec_int4(C.c_uint32(N), C.c_uint32(K), _vp(a), _vp(bq), _vp(bs), _vp(bz),
                                _vp(out), C.c_uint32(group))
    return out


def quant_matmul_int4(a, bq, bs, bz, M: int, N: int, K: int, group: int = 128) -> np.ndarray:
    a, bq, bs, bz = _c(a, np.float32), _c(bq, np.uint32), _c(bs, np.uint16), _c(bz, np.uint16)
    out = np.zeros((M, N), np.float32)
    lib().orc_quant_matmul_int4(C.c_uint32(M), C.c_uint32(N), C.c_uint32(K), _vp(a), _vp(bq),
                                _vp(bs), _vp(bz), _vp(out), C.c_uint32(group))
    return out


# ---------------------------------------------------------------- int8
def int8_quantize(w):
    w = _c(w, np.float32).ravel()
    quants = np.zeros(w.size, np.int8)
    scales = np.zeros((w.size + 31) // 32, np.uint16)
    lib().orc_int8_quantize(_vp(w), C.c_size_t(w.size), _vp(quants), _vp(scales))
    return quants, scales


def int8_dequantize(quants, scales) -> np.ndarray:
    quants, scales = _c(quants, np.int8), _c(scales, np.uint16)
    out = np.empty(quants.size, np.float32)
    lib().orc_int8_dequantize(_vp(quants), _vp(scales), C.c_size_t(quants.size), _vp(out))
    return out


def quant_matvec_f32(a, bq, bs, N: int, K: int) -> np.ndarray:
    a, bq, bs = _c(a, np.float32), _c(bq, np.int8), _c(bs, np.uint16)
    out = np.zeros(N, np.float32)
    lib().orc_quant_matvec_f32(C.c_uint32(N), C.c_uint32(K), _vp(a), _vp(bq), _vp(bs), _vp(out))
    return out


def quant_matmul_tiled_f32(a, bq, bs, M: int, N: int, K: int) -> np.ndarray:
    a, bq, bs = _c(a, np.float32), _c(bq, np.int8), _c(bs, np.uint16)
    out = np.zeros((M, N), np.float32)
    lib().orc_quant_matmul_tiled_f32(C.c_uint32(M), C.c_uint32(N), C.c_uint32(K), _vp(a), _vp(bq),
                                     _vp(bs), _vp(out))
    return out


def matmul_definition_f64(a, w_dequant, M: int, N: int, K: int):
    a, w = _c(a, np.float32), _c(w_dequant, np.float32)
    want = np.zeros((M, N), np.float64)
    mag = np.zeros((M, N), np.float64)
    lib().orc_matmul_definition_f64(C.c_uint32(M), C.c_uint32(N), C.c_uint32(K), _vp(a), _vp(w),
                                    _vp(want), _vp(mag))
    return want, mag


# ---------------------------------------------------------------- attention
def _cache(k, v):
    k, v = np.ascontiguousarray(k), np.ascontiguousarray(v)
    assert k.dtype == v.dtype and k.dtype in (np.float32, np.uint16), \
        "cache is f32, or f16 carried as uint16 bit patterns"
    return k, v, int(k.dtype == np.uint16)


def attention_decode(q, k, v, lengths, q_heads, kv_heads, head_dim, scale, sgw=4):
    q, lengths = _c(q, np.float32), _c(lengths, np.uint32)
    k, v, f16 = _cache(k, v)
    out = np.zeros(q_heads * head_dim, np.float32)
    lib().orc_attention_decode(C.c_uint32(q_heads), C.c_uint32(kv_heads), C.c_uint32(head_dim),
                               C.c_float(scale), _vp(q), _vp(k), _vp(v), C.c_int(f16),
                               C.c_uint64(k.size), _vp(lengths), _vp(out), C.c_uint32(sgw))
    return out


def attention_decode_paged(q, k, v, pages, lengths, q_heads, kv_heads, head_dim, block, scale,
                           sgw=4):
    q, lengths, pages = _c(q, np.float32), _c(lengths, np.uint32), _c(pages, np.uint32)
    k, v, f16 = _cache(k, v)
    out = np.zeros(q_heads * head_dim, np.float32)
    lib().orc_attention_decode_paged(C.c_uint32(q_heads), C.c_uint32(kv_heads),
                                     C.c_uint32(head_dim), C.c_uint32(block), C.c_float(scale),
                                     _vp(q), _vp(k), _vp(v), C.c_int(f16), _vp(pages),
                                     C.c_uint32(pages.size), _vp(lengths), _vp(out),
                                     C.c_uint32(sgw))
    return out


def attention_decode_batched(q, k, v, pages, lengths, batch, q_heads, kv_heads, head_dim, block,
                             max_pages, scale, sgw=4):
    q, lengths, pages = _c(q, np.float32), _c(lengths, np.uint32), _c(pages, np.uint32)
    k, v, f16 = _cache(k, v)
    out = np.zeros(batch * q_heads * head_dim, np.float32)
    lib().orc_attention_decode_batched(C.c_uint32(batch), C.c_uint32(q_heads),
                                       C.c_uint32(kv_heads), C.c_uint32(head_dim),
                                       C.c_uint32(block), C.c_uint32(max_pages), C.c_float(scale),
                                       _vp(q), _vp(k), _vp(v), C.c_int(f16), _vp(pages),
                                       _vp(lengths), _vp(out), C.c_uint32(sgw))
    return out


def attention_ragged(q, k, v, pages, lengths, offsets, tokens, batch, q_heads, kv_heads, head_dim,
                     block, max_pages, scale):
    q, lengths = _c(q, np.float32), _c(lengths, np.uint32)
    pages, offsets = _c(pages, np.uint32), _c(offsets, np.uint32)
    k, v, f16 = _cache(k, v)
    out = np.zeros(tokens * q_heads * head_dim, np.float32)
    lib().orc_attention_ragged(C.c_uint32(tokens), C.c_uint32(batch), C.c_uint32(q_heads),
                               C.c_uint32(kv_heads), C.c_uint32(head_dim), C.c_uint32(block),
                               C.c_uint32(max_pages), C.c_float(scale), _vp(q), _vp(k), _vp(v),
                               C.c_int(f16), _vp(pages), _vp(lengths), _vp(offsets), _vp(out))
    return out


def attention_prefill(q, k, v, lengths, q_heads, kv_heads, head_dim, q_seq, base, scale):
    """AttentionPrefill(F16), internal/kernels/prefill.go:197: contiguous cache, one sequence."""
    q, lengths = _c(q, np.float32), _c(lengths, np.uint32)
    k, v, f16 = _cache(k, v)
    out = np.zeros(q_seq * q_heads * head_dim, np.float32)
    lib().orc_attention_prefill(C.c_uint32(q_heads), C.c_uint32(kv_heads), C.c_uint32(head_dim),
                                C.c_uint32(q_seq), C.c_uint32(base), C.c_float(scale), _vp(q), _vp(k), _vp(v),
                                C.c_int(f16), C.c_uint64(k.size), _vp(lengths), _vp(out))
    return out


def attention_prefill_paged(q, k, v, pages, lengths, q_heads, kv_heads, head_dim, q_seq, base, block, scale):
    """AttentionPrefillPaged(F16), internal/kernels/prefill.go:409, pagedprefillf16.go:31."""
    q, lengths, pages = _c(q, np.float32), _c(lengths, np.uint32), _c(pages, np.uint32)
    k, v, f16 = _cache(k, v)
    out = np.zeros(q_seq * q_heads * head_dim, np.float32)
    lib().orc_attention_prefill_paged(C.c_uint32(q_heads), C.c_uint32(kv_heads), C.c_uint32(head_dim),
                                      C.c_uint32(q_seq), C.c_uint32(base), C.c_uint32(block), C.c_float(scale),
                                      _vp(q), _vp(k), _vp(v), C.c_int(f16), _vp(pages), C.c_uint32(pages.size),
                                      _vp(lengths), _vp(out))
    return out


def attention_definition_f64(q, k, v, rows, q_heads, kv_heads, head_dim, scale):
    q, rows = _c(q, np.float32), _c(rows, np.uint32)
    k, v, f16 = _cache(k, v)
    out = np.zeros(q_heads * head_dim, np.float64)
    lib().orc_attention_definition_f64(C.c_uint32(q_heads), C.c_uint32(kv_heads),
                                       C.c_uint32(head_dim), C.c_double(scale), _vp(q), _vp(k),
                                       _vp(v), C.c_int(f16), _vp(rows), C.c_uint32(rows.size),
                                       _vp(out))
    return out


# ---------------------------------------------------------------- grouped
def segment_offsets(counts) -> np.ndarray:
    counts = _c(counts, np.uint32)
    out = np.zeros(counts.size + 1, np.uint32)
    lib().orc_segment_offsets(C.c_uint32(counts.size), _vp(counts), _vp(out))
    return out


def grouped_matvec(x, w, offsets, tokens, experts, K, N) -> np.ndarray:
    x, w, offsets = _c(x, np.float32), _c(w, np.float32), _c(offsets, np.uint32)
    out = np.zeros((tokens, N), np.float32)
    lib().orc_grouped_matvec(C.c_uint32(tokens), C.c_uint32(experts), C.c_uint32(K),
                             C.c_uint32(N), _vp(x), _vp(w), _vp(offsets), _vp(out))
    return out


def grouped_matmul(x, w, offsets, tokens, experts, K, N, out=None) -> np.ndarray:
    x, w, offsets = _c(x, np.float32), _c(w, np.float32), _c(offsets, np.uint32)
    if out is None:
        out = np.zeros((tokens, N), np.float32)
    lib().orc_grouped_matmul(C.c_uint32(experts), C.c_uint32(tokens), C.c_uint32(K),
                             C.c_uint32(N), _vp(x), _vp(w), _vp(offsets), _vp(out))
    return out


# ---------------------------------------------------------------- support operators
def scatter_rows(rows, ids, state, capacity=None):
    """In place on `state` ([capacity, width]; f32, or f16 as uint16 bit patterns)."""
    rows = np.ascontiguousarray(rows)
    ids = _c(ids, np.uint32)
    assert state.flags["C_CONTIGUOUS"] and state.dtype == rows.dtype
    width = rows.size // max(ids.size, 1)
    cap = state.size // width if capacity is None else capacity
    lib().orc_scatter_rows(C.c_uint32(ids.size), C.c_uint32(width), C.c_uint32(cap), _vp(rows),
                           _vp(ids), _vp(state), C.c_uint32(state.dtype.itemsize))
    return state


def gather_rows(table, ids, width, capacity=None) -> np.ndarray:
    table, ids = _c(table, np.float32), _c(ids, np.uint32)
    cap = table.size // width if capacity is None else capacity
    out = np.zeros((ids.size, width), np.float32)
    lib().orc_gather_rows(C.c_uint32(ids.size), C.c_uint32(width), C.c_uint32(cap), _vp(table),
                          _vp(ids), _vp(out))
    return out


def rmsnorm(x, w, eps) -> np.ndarray:
    x, w = _c(x, np.float32), _c(w, np.float32)
    rows, width = x.shape
    out = np.zeros_like(x)
    lib().orc_rmsnorm(C.c_uint32(rows), C.c_uint32(width), C.c_float(eps), _vp(x), _vp(w),
                      _vp(out))
    return out


def rope(x, positions, rotary_dim, base) -> np.ndarray:
    x = np.array(x, dtype=np.float32, order="C", copy=True)
    positions = _c(positions, np.uint32)
    rows, width = x.shape
    lib().orc_rope(C.c_uint32(rows), C.c_uint32(width), C.c_uint32(rotary_dim), C.c_float(base),
                   _vp(positions), _vp(x))
    return x


def swiglu(a, b) -> np.ndarray:
    a, b = _c(a, np.float32), _c(b, np.float32)
    out = np.zeros_like(a)
    lib().orc_swiglu(_vp(a), _vp(b), _vp(out), C.c_size_t(a.size))
    return out


def elem_add(a, b) -> np.ndarray:
    a, b = _c(a, np.float32), _c(b, np.float32)
    out = np.zeros_like(a)
    lib().orc_elem_add(_vp(a), _vp(b), _vp(out), C.c_size_t(a.size))
    return out


def sample_argmax(logits) -> np.ndarray:
    logits = _c(logits, np.float32)
    rows, vocab = logits.shape
    out = np.zeros(rows, np.uint32)
    lib().orc_sample_argmax(C.c_uint32(rows), C.c_uint32(vocab), _vp(logits), _vp(out))
    return out


# ---------------------------------------------------------------- sampling policy
def softmax(x) -> np.ndarray:
    x = _c(x, np.float32)
    rows, width = x.shape
    out = np.empty_like(x)
    lib().orc_softmax(C.c_uint32(rows), C.c_uint32(width), _vp(x), _vp(out))
    return out


def scale_rows(x, factors) -> np.ndarray:
    x, factors = _c(x, np.float32), _c(factors, np.float32)
    out = np.empty_like(x)
    lib().orc_scale_rows(C.c_uint32(x.shape[0]), C.c_uint32(x.shape[1]), _vp(x), _vp(factors), _vp(out))
    return out


def topk_mask(weights, k) -> np.ndarray:
    """TopKMaskRows when k is an array (one per row), TopKMask when it is a number."""
    w = _c(np.atleast_2d(weights), np.float32)
    out = np.empty_like(w)
    if np.ndim(k) == 0:
        lib().orc_topk_mask(C.c_uint32(w.shape[0]), C.c_uint32(w.shape[1]), _vp(w), None, C.c_uint32(int(k)), _vp(out))
    else:
        ks = _c(k, np.uint32)
        lib().orc_topk_mask(C.c_uint32(w.shape[0]), C.c_uint32(w.shape[1]), _vp(w), _vp(ks), C.c_uint32(0), _vp(out))
    return out.reshape(np.shape(weights))


def topp_mask(weights, p) -> np.ndarray:
    """TopPMaskRows when p is an array (one per row), TopPMask when it is a number."""
    w = _c(np.atleast_2d(weights), np.float32)
    out = np.empty_like(w)
    if np.ndim(p) == 0:
        lib().orc_topp_mask(C.c_uint32(w.shape[0]), C.c_uint32(w.shape[1]), _vp(w), None, C.c_float(float(p)), _vp(out))
    else:
        ps = _c(p, np.float32)
        lib().orc_topp_mask(C.c_uint32(w.shape[0]), C.c_uint32(w.shape[1]), _vp(w), _vp(ps), C.c_float(0), _vp(out))
    return out.reshape(np.shape(weights))


def sample_rows(probs, draws, factors=None) -> np.ndarray:
    """SampleRows (factors given: a zero factor takes the row's argmax) or SampleCategorical."""
    p = _c(np.atleast_2d(probs), np.float32)
    d = _c(np.atleast_1d(draws), np.float32)
    out = np.zeros(p.shape[0], np.uint32)
    f = _c(factors, np.float32) if factors is not None else None
    lib().orc_sample_rows(C.c_uint32(p.shape[0]), C.c_uint32(p.shape[1]), _vp(p), _vp(d),
                          _vp(f) if f is not None else None, _vp(out))
    return out


def logit_bias(logits, ids, values) -> np.ndarray:
    x, ids, values = _c(logits, np.float32), _c(ids, np.uint32), _c(values, np.float32)
    out = np.empty_like(x)
    lib().orc_logit_bias(C.c_uint32(x.shape[0]), C.c_uint32(x.shape[1]), C.c_uint32(ids.shape[1]), _vp(x),
                         _vp(ids), _vp(values), _vp(out))
    return out


def penalty_rows(logits, history, filled, repetition, presence, frequency):
    """PenaltyClearRows -> PenaltyCountRows -> PenaltyApplyRows.  Returns (penalised logits, counts)."""
    x = _c(np.atleast_2d(logits), np.float32)
    h = _c(np.atleast_2d(history), np.uint32)
    rows, vocab = x.shape
    f = _c(np.atleast_1d(filled), np.uint32)
    rep, pres, freq = (_c(np.atleast_1d(a), np.float32) for a in (repetition, presence, frequency))
    counts = np.zeros((rows, vocab), np.uint32)
    out = np.empty_like(x)
    lib().orc_penalty_rows(C.c_uint32(rows), C.c_uint32(vocab), C.c_uint32(h.shape[1]), _vp(x), _vp(h), _vp(f),
                           _vp(rep), _vp(pres), _vp(freq), _vp(counts), _vp(out))
    return out, counts


# ---------------------------------------------------------------- block pool
class BlockPool:
    """tensor/blockpool.go:46-133 restated; errors are ValueError with the reference's wording."""

    def __init__(self, blocks: int, positions_per_block: int):
        h = lib().orc_blockpool_new(C.c_int(blocks), C.c_int(positions_per_block))
        if not h:
            raise ValueError(f"a pool of {blocks} blocks of {positions_per_block} positions")
        self._h = C.c_void_p(h)
        self._blocks = blocks

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_blockpool_free_pool(self._h)
            self._h = None

    def block_size(self) -> int:
        return lib().orc_blockpool_block_size(self._h)

    def available(self) -> int:
        return lib().orc_blockpool_available(self._h)

    def grow(self, pages, n: int):
        pages = [] if pages is None else list(pages)
        buf = np.zeros(len(pages) + self._blocks + 1, np.uint32)
        buf[:len(pages)] = pages
        r = lib().orc_blockpool_grow(self._h, _vp(buf), C.c_int(len(pages)), C.c_int(n))
        if r == -1:
            raise ValueError(f"{n} positions")
        if r == -2:
            raise ValueError("the pool does not evict")
        return [int(x) for x in buf[:r]]

    def free(self, pages):
        arr = _c(list(pages), np.uint32)
        errs = lib().orc_blockpool_free(self._h, _vp(arr), C.c_int(arr.size))
        if errs:
            raise ValueError(f"{errs} block(s) already free")

    def positions(self, pages) -> int:
        return len(pages) * self.block_size()
