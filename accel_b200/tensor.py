"""Operator-level interface of the path, mirroring accel's `tensor` package: the same operator
names, argument meaning, validation and refusal wording as tensor/int4.go, tensor/attention.go,
tensor/grouped.go, tensor/state.go and tensor/ops.go, executed eagerly on torch-owned device
memory through the C ABI (accel records these into a plan; the plan form is `accel_b200.driver`).

A refused call raises `Refused` and launches nothing, as accel's builder records a failure and
poisons the result rather than running."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import runtime as rt
from .quant import INT4_GROUP

__all__ = ["Refused", "Int4", "int4_matvec", "int4_matmul", "AttentionOptions", "attention",
           "grouped_matvec", "grouped_matmul", "grouped_matmul_int4", "segment_offsets",
           "scatter_rows", "gather_rows", "rms_norm", "rope", "swiglu", "add", "argmax", "cast"]

U32 = torch.int32       # torch has no general uint32 arithmetic; the bits are what the kernels read


class Refused(ValueError):
    """An operator's validation failed (accel's Builder.fail)."""

    def __init__(self, op: str, why: str):
        super().__init__(f"accel/tensor: {op}: {why}")
        self.op = op


def _is_u32(t: torch.Tensor) -> bool:
    return t.dtype in (torch.int32, torch.uint32)


# ------------------------------------------------------------------------------- int4 linear
@dataclass
class Int4:
    """tensor.Int4 (tensor/int4.go:25): three flat planes and the weight count."""
    codes: torch.Tensor     # u32 words, eight weights each, low nibble first
    scales: torch.Tensor    # f16, one per 128 weights
    zeros: torch.Tensor     # f16, one per 128 weights
    weights: int


def _check_int4(q: Int4, what: str) -> str:
    # tensor/int4.go:41-78
    if q.codes is None or q.scales is None or q.zeros is None:
        return (f"{what} needs a code plane, a scale plane and a zero plane; the zero point is "
                "what makes four bits usable and is not optional")
    if not _is_u32(q.codes):
        return (f"{what} codes are {q.codes.dtype} and must be u32: eight weights per word, and "
                "a kernel cannot do arithmetic on a narrower type")
    if q.scales.dtype != torch.float16:
        return f"{what} scales are {q.scales.dtype} and must be f16"
    if q.zeros.dtype != torch.float16:
        return f"{what} zeros are {q.zeros.dtype} and must be f16"
    if q.weights <= 0:
        return (f"{what} declares {q.weights} weights; the count cannot be derived from the word "
                "count, because eight weights per word makes several matrices pack into the same "
                "words")
    want = (q.weights + 7) // 8
    if q.codes.numel() != want:
        return (f"{what} declares {q.weights} weights, which is {want} words, and the code plane "
                f"holds {q.codes.numel()}")
    groups = (q.weights + INT4_GROUP - 1) // INT4_GROUP
    for name, t in (("scales", q.scales), ("zeros", q.zeros)):
        if t.numel() != groups:
            return (f"{what} has {q.weights} weights, which is {groups} groups of {INT4_GROUP}, "
                    f"and {t.numel()} {name}")
    return ""


def int4_matvec(a: torch.Tensor, w: Int4) -> torch.Tensor:
    """tensor.Int4MatVec (tensor/int4.go:99): a f32[K] against a [K,N] int4 matrix -> f32[N]."""
    why = _check_int4(w, "the weight matrix")
    if why:
        raise Refused("Int4MatVec", why)
    if a.dtype != torch.float32:
        raise Refused("Int4MatVec", f"activations are {a.dtype} and this kernel reads f32")
    if a.dim() != 1:
        raise Refused("Int4MatVec", f"activations are {tuple(a.shape)}; a matvec takes a vector, "
                      "and a batch of them is Int4MatMul")
    k = a.shape[0]
    if k == 0 or w.weights % k != 0:
        raise Refused("Int4MatVec", f"activations are {k} long and the matrix holds {w.weights} "
                      "weights; the matrix is [K, N] with K the activation width, so the second "
                      "is a multiple of the first")
    n = w.weights // k
    out = torch.empty(n, dtype=torch.float32, device=a.device)
    rt.launch("QuantMatVecInt4", [a.contiguous(), w.codes, w.scales, w.zeros, out],
              rt.gemm_dims(0, n, k))
    return out


def int4_matmul(a: torch.Tensor, w: Int4) -> torch.Tensor:
    """tensor.Int4MatMul (tensor/int4.go:168): a f32[M,K] against a [K,N] int4 matrix -> f32[M,N]."""
    why = _check_int4(w, "the weight matrix")
    if why:
        raise Refused("Int4MatMul", why)
    if a.dtype != torch.float32:
        raise Refused("Int4MatMul", f"activations are {a.dtype} and this kernel reads f32")
    if a.dim() != 2:
        raise Refused("Int4MatMul", f"activations are {tuple(a.shape)}; this is the batched form "
                      "and takes [rows, K]. One row is Int4MatVec, which is the decode shape and "
                      "reads the matrix once per token")
    m, k = a.shape
    if k == 0 or w.weights % k != 0:
        raise Refused("Int4MatMul", f"activations are {k} wide and the matrix holds {w.weights} "
                      "weights; the matrix is [K, N] with K the activation width, so the second "
                      "is a multiple of the first")
    n = w.weights // k
    out = torch.empty((m, n), dtype=torch.float32, device=a.device)
    if m:
        rt.launch("QuantMatMulInt4", [a.contiguous(), w.codes, w.scales, w.zeros, out],
                  rt.gemm_dims(m, n, k))
    return out


# ------------------------------------------------------------------------------- int8 linear
@dataclass
class Quantized:
    """tensor.Quantized (tensor/quantized.go:17): the quant plane [K, N] (i8) and its scales (f16,
    one per 32 quants along the flat index)."""
    quants: torch.Tensor
    scales: torch.Tensor


def _check_quantized(q: Quantized, what: str) -> str:
    # tensor/quantized.go:25-52
    if q.quants.dtype != torch.int8:
        return f"{what} quants are {q.quants.dtype} and must be i8"
    if q.scales.dtype != torch.float16:
        return f"{what} scales are {q.scales.dtype} and must be f16"
    n = q.quants.numel()
    want = (n + 31) // 32
    if q.scales.numel() != want:
        return (f"{what} has {n} quants, which is {want} blocks of 32, and {q.scales.numel()} scales")
    return ""


def quant_matmul(x: torch.Tensor, w: Quantized) -> torch.Tensor:
    """tensor.QuantMatMul (tensor/quantized.go:72) for f32 activations: one row takes the
    matrix-vector kernel, more rows the tiled one, as the reference selects them."""
    if w.quants is None or w.scales is None:
        raise Refused("QuantMatMul", "the weight needs both a quant plane and a scale plane")
    why = _check_quantized(w, "the weight")
    if why:
        raise Refused("QuantMatMul", why)
    if x.dtype != torch.float32:
        raise Refused("QuantMatMul", f"activations are {x.dtype}; this backend runs the f32-activation "
                      "kernels of the int8 path (QuantMatVecF32, QuantMatMulTiledF32)")
    if x.dim() != 2 or w.quants.dim() != 2:
        raise Refused("QuantMatMul", f"operands are {tuple(x.shape)} and {tuple(w.quants.shape)}; "
                      "v0 multiplies two matrices")
    if x.shape[1] != w.quants.shape[0]:
        raise Refused("QuantMatMul", f"{tuple(x.shape)} times {tuple(w.quants.shape)}: the contracted "
                      f"axes are {x.shape[1]} and {w.quants.shape[0]}")
    m, k = x.shape
    n = w.quants.shape[1]
    out = torch.empty((m, n), dtype=torch.float32, device=x.device)
    if m == 0:
        return out
    name = "QuantMatVecF32" if m == 1 else "QuantMatMulTiledF32"
    rt.launch(name, [x.contiguous(), w.quants.contiguous(), w.scales, out], rt.gemm_dims(m, n, k))
    return out


# ------------------------------------------------------------------------------- attention
@dataclass
class AttentionOptions:
    """tensor.AttentionOptions (tensor/attention.go:15).  `scale` stands for the named f32 scalar
    the reference reads at submit time."""
    lengths: Optional[torch.Tensor] = None
    pages: Optional[torch.Tensor] = None
    block: int = 0
    scale: float = 1.0
    query_extents: Optional[torch.Tensor] = None
    base: Optional[int] = None     # stands for BaseName: the cache position of a prefill's first query token


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, opts: AttentionOptions) -> torch.Tensor:
    """tensor.Attention (tensor/attention.go:124).  q's rank selects the kernel: [qHeads, D] one
    token; [batch, 1, qHeads, D] with Pages the batched decode (f32 cache; an f16 cache runs the
    batched-f16 extension); [tokens, qHeads, D] with QueryExtents the ragged step; [qSeq, qHeads, D]
    without it a causal prefill of one sequence (Base required; paged when Pages is set).
    k and v are the caches, [capacity, kvHeads, D], f32 or f16."""
    op = "Attention"
    if q.dtype != torch.float32:
        raise Refused(op, f"q is {q.dtype} and the registered kernels read an f32 query")
    if k.dtype != v.dtype:
        raise Refused(op, f"the key cache is {k.dtype} and the value cache is {v.dtype}; one kernel "
                      "reads both, so they are the same dtype")
    if k.dtype not in (torch.float32, torch.float16):
        raise Refused(op, f"the cache is {k.dtype}; the registered kernels read f32 or f16")
    f16 = k.dtype == torch.float16
    if not q.is_contiguous():
        raise Refused(op, "q is a strided view and the registered kernels index it contiguously")
    rank = q.dim()
    if rank not in (2, 3, 4):
        raise Refused(op, f"q is {tuple(q.shape)}; it is [qHeads, headDim] for one token, "
                      "[qSeq, qHeads, headDim] for a prefill, or [batch, qSeq, qHeads, headDim] "
                      "for several sequences stepping together")
    batch, q_seq = 1, 1
    batched = rank == 4
    ragged = prefill = False
    if rank == 4:
        batch, q_seq = q.shape[0], q.shape[1]
    if opts.query_extents is not None:
        if rank != 3:
            raise Refused(op, f"q is {tuple(q.shape)} and QueryExtents is set; a ragged step is "
                          "the flat [tokens, qHeads, headDim] form")
        if not _is_u32(opts.query_extents):
            raise Refused(op, f"QueryExtents is {opts.query_extents.dtype}; it is a count per "
                          "sequence, which is u32")
        ragged = True
        batch = opts.query_extents.numel()
        if batch == 0:
            raise Refused(op, "QueryExtents is empty; it is one count per sequence and a step has "
                          "at least one sequence")
    elif rank == 3:
        prefill, q_seq = True, q.shape[0]
    if k.dim() != 3 or tuple(k.shape) != tuple(v.shape):
        raise Refused(op, f"the key cache is {tuple(k.shape)} and the value cache is "
                      f"{tuple(v.shape)}; both are [capacity, kvHeads, headDim] and equal")
    q_heads, head_dim = q.shape[-2], q.shape[-1]
    kv_heads = k.shape[1]
    if k.shape[2] != head_dim:
        raise Refused(op, f"q's head is {head_dim} wide and the cache's is {k.shape[2]}")
    if kv_heads == 0 or q_heads % kv_heads != 0:
        raise Refused(op, f"{q_heads} query heads over {kv_heads} key/value heads; several query "
                      "heads share one cache entry, so the first is a multiple of the second")
    if opts.lengths is None:
        raise Refused(op, "Lengths is required: it holds how much of each sequence's cache is "
                      "real, one entry per sequence. A single sequence binds one element")
    if not _is_u32(opts.lengths):
        raise Refused(op, f"Lengths is {opts.lengths.dtype} and a cache length is u32")
    if opts.pages is not None:
        if not _is_u32(opts.pages):
            raise Refused(op, f"Pages is {opts.pages.dtype} and a page table is u32")
        if opts.block <= 0:
            raise Refused(op, f"Pages is set and Block is {opts.block}; a page table addresses "
                          "blocks, so how many positions one holds is required")
    if opts.lengths.numel() != batch:
        raise Refused(op, f"Lengths holds {opts.lengths.numel()} entries and this step has {batch} "
                      "sequence(s); it is one length per sequence")
    k, v = k.contiguous(), v.contiguous()
    scale = float(opts.scale)

    if prefill:
        if opts.base is None:
            raise Refused(op, "a prefill needs BaseName: the position of its first query token within "
                          "the cache, which is what the causal mask is measured from")
        out = torch.empty((q_seq, q_heads, head_dim), dtype=torch.float32, device=q.device)
        if q_seq == 0:
            return out
        if opts.pages is not None:
            if opts.pages.dim() != 1:
                raise Refused(op, f"Pages is {tuple(opts.pages.shape)}; a prefill is one sequence, whose "
                              "page table is one row of block ids")
            rt.launch("AttentionPrefillPagedF16" if f16 else "AttentionPrefillPaged",
                      [q, k, v, opts.pages.contiguous(), opts.lengths, out],
                      rt.paged_prefill_dims(q_heads, kv_heads, head_dim, q_seq, int(opts.base), opts.block, scale))
        else:
            rt.launch("AttentionPrefillF16" if f16 else "AttentionPrefill", [q, k, v, opts.lengths, out],
                      rt.prefill_dims(q_heads, kv_heads, head_dim, q_seq, int(opts.base), scale))
        return out
    if ragged:
        if opts.pages is None:
            raise Refused(op, f"a ragged step of {batch} sequences needs Pages: they have "
                          "different lengths, so a contiguous cache would pad every sequence to "
                          "the longest")
        if opts.pages.dim() != 2 or opts.pages.shape[0] != batch:
            raise Refused(op, f"Pages is {tuple(opts.pages.shape)} and QueryExtents names {batch} "
                          "sequences; a page table is [batch, maxPages]")
        tokens = q.shape[0]
        offsets = segment_offsets(opts.query_extents)
        out = torch.empty((tokens, q_heads, head_dim), dtype=torch.float32, device=q.device)
        if tokens:
            rt.launch("AttentionRaggedF16" if f16 else "AttentionRagged",
                      [q, k, v, opts.pages.contiguous(), opts.lengths, offsets, out],
                      rt.batched_dims(batch, q_heads, kv_heads, head_dim, opts.block,
                                      opts.pages.shape[1], scale))
        return out
    if batched:
        if opts.pages is None:
            raise Refused(op, f"a batch of {batch} sequences needs Pages: they have different "
                          "lengths, so a contiguous cache would pad every sequence to the longest")
        if q_seq != 1:
            raise Refused(op, f"q is {tuple(q.shape)}: the rectangular batched form takes one "
                          "token per sequence. A batched prefill is the ragged form")
        if opts.pages.dim() != 2 or opts.pages.shape[0] != batch:
            raise Refused(op, f"Pages is {tuple(opts.pages.shape)} and the batch is {batch}; a "
                          "batched page table is [batch, maxPages], one row of block ids per "
                          "sequence")
        out = torch.empty((batch, q_heads, head_dim), dtype=torch.float32, device=q.device)
        if batch:
            rt.launch("AttentionDecodeBatchedF16" if f16 else "AttentionDecodeBatched",
                      [q, k, v, opts.pages.contiguous(), opts.lengths, out],
                      rt.batched_dims(batch, q_heads, kv_heads, head_dim, opts.block,
                                      opts.pages.shape[1], scale))
        return out
    out = torch.empty((q_heads, head_dim), dtype=torch.float32, device=q.device)
    if opts.pages is not None:
        rt.launch("AttentionDecodePagedF16" if f16 else "AttentionDecodePaged",
                  [q, k, v, opts.pages.contiguous(), opts.lengths, out],
                  rt.paged_dims(q_heads, kv_heads, head_dim, opts.block, scale))
    else:
        rt.launch("AttentionDecodeF16" if f16 else "AttentionDecode",
                  [q, k, v, opts.lengths, out], rt.attn_dims(q_heads, kv_heads, head_dim, scale))
    return out


# ------------------------------------------------------------------------------- grouped
def segment_offsets(counts: torch.Tensor) -> torch.Tensor:
    """tensor/segment.go: exclusive prefix sum counts[R] -> offsets[R+1], on the device."""
    rows = counts.numel()
    offsets = torch.empty(rows + 1, dtype=counts.dtype, device=counts.device)
    rt.launch("SegmentOffsets", [counts.contiguous(), offsets], rt.segment_dims(rows))
    return offsets


def _check_grouped(op: str, x, w, counts):
    if counts is None:
        raise Refused(op, "counts is nil; it is one token count per expert and is what says "
                      "which rows belong to which weight matrix")
    for name, t, ok in (("x", x, x.dtype == torch.float32), ("w", w, w.dtype == torch.float32),
                        ("counts", counts, _is_u32(counts))):
        if not ok:
            raise Refused(op, f"{name} is {t.dtype} and this kernel reads "
                          f"{'u32' if name == 'counts' else 'f32'}")
    if x.dim() != 2:
        raise Refused(op, f"x is {tuple(x.shape)}; it is [tokens, K] with the tokens of every "
                      "expert end to end")
    if w.dim() != 3:
        raise Refused(op, f"w is {tuple(w.shape)}; it is [experts, K, N], one matrix per expert")
    if w.shape[1] != x.shape[1]:
        raise Refused(op, f"x is {tuple(x.shape)} and w is {tuple(w.shape)}; every expert "
                      "contracts against the same width, so w's second axis is x's second")
    if counts.numel() != w.shape[0]:
        raise Refused(op, f"counts holds {counts.numel()} entries and w has {w.shape[0]} experts; "
                      "it is one token count per expert")
    if w.shape[0] == 0:
        raise Refused(op, "w declares no experts")


def grouped_matvec(x, w, counts) -> torch.Tensor:
    """tensor.GroupedMatVec (tensor/grouped.go:48): rows past the counts' sum come out zero."""
    _check_grouped("GroupedMatVec", x, w, counts)
    tokens, k = x.shape
    experts, _, n = w.shape
    offsets = segment_offsets(counts)
    out = torch.empty((tokens, n), dtype=torch.float32, device=x.device)
    if tokens * n:
        rt.launch("GroupedMatVec", [x.contiguous(), w.contiguous(), offsets, out],
                  rt.grouped_dims(experts, k, n))
    return out


def grouped_matmul(x, w, counts, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """tensor.GroupedMatMul (tensor/grouped.go:138): rows past the counts' sum are not written."""
    _check_grouped("GroupedMatMul", x, w, counts)
    tokens, k = x.shape
    experts, _, n = w.shape
    offsets = segment_offsets(counts)
    if out is None:
        out = torch.zeros((tokens, n), dtype=torch.float32, device=x.device)
    if tokens * n:
        rt.launch("GroupedMatMul", [x.contiguous(), w.contiguous(), offsets, out],
                  rt.grouped_tiled_dims(experts, tokens, k, n))
    return out


def grouped_matmul_int4(x, w: Int4, experts: int, counts, out=None) -> torch.Tensor:
    """No reference operator: GroupedMatMul over int4 expert matrices.  `w` holds the experts'
    planes end to end, each [K,N] matrix quantized on its own; w.weights = experts*K*N."""
    op = "GroupedMatMulInt4"
    if x.dtype != torch.float32 or x.dim() != 2:
        raise Refused(op, f"x is {x.dtype} {tuple(x.shape)}; it is f32 [tokens, K]")
    tokens, k = x.shape
    if experts <= 0 or w.weights % experts or (w.weights // experts) % k:
        raise Refused(op, f"{w.weights} weights do not divide into {experts} matrices of K={k}")
    per = w.weights // experts
    if per % INT4_GROUP:
        raise Refused(op, f"each expert holds {per} weights, not a whole number of groups, so the "
                      "experts' planes would not be separable")
    n = per // k
    if counts.numel() != experts:
        raise Refused(op, f"counts holds {counts.numel()} entries for {experts} experts")
    offsets = segment_offsets(counts)
    if out is None:
        out = torch.zeros((tokens, n), dtype=torch.float32, device=x.device)
    if tokens * n:
        rt.launch(op, [x.contiguous(), w.codes, w.scales, w.zeros, offsets, out],
                  rt.grouped_tiled_dims(experts, tokens, k, n))
    return out


# ------------------------------------------------------------------------------- support operators
def scatter_rows(state: torch.Tensor, rows: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """tensor.ScatterRows (tensor/state.go:206): state[ids[r]] = rows[r], in place; an id at or past
    the capacity drops its row.  Returns the state, which is what a following Attention must read."""
    if rows.dtype != state.dtype:
        raise Refused("ScatterRows", f"rows are {rows.dtype} and the state is {state.dtype}; "
                      "they are the same dtype")
    if state.dtype not in (torch.float32, torch.float16):
        raise Refused("ScatterRows", f"the state is {state.dtype}; f32 or f16")
    if not _is_u32(ids):
        raise Refused("ScatterRows", f"ids are {ids.dtype} and a row index is u32")
    capacity = state.shape[0]
    width = state.numel() // max(capacity, 1)
    n = ids.numel()
    if rows.numel() != n * width:
        raise Refused("ScatterRows", f"{n} ids and rows of {tuple(rows.shape)} against a state "
                      f"row of {width}")
    if n:
        rt.launch("ScatterRowsF16" if state.dtype == torch.float16 else "ScatterRows",
                  [rows.contiguous(), ids.contiguous(), state], rt.row_params(n, width, capacity))
    return state


def gather_rows(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """tensor.GatherRows (tensor/ops.go:50): out[r] = table[ids[r]], zeros for an id out of range."""
    if table.dim() != 2 or table.dtype not in (torch.float32, torch.float16):
        raise Refused("GatherRows", f"the table is {table.dtype} {tuple(table.shape)}; it is "
                      "[rows, width], f32 or f16")
    if not _is_u32(ids):
        raise Refused("GatherRows", f"ids are {ids.dtype} and a row index is u32")
    capacity, width = table.shape
    out = torch.empty((ids.numel(), width), dtype=torch.float32, device=table.device)
    if ids.numel():
        rt.launch("GatherRowsF16" if table.dtype == torch.float16 else "GatherRows",
                  [table.contiguous(), ids.contiguous(), out],
                  rt.row_params(ids.numel(), width, capacity))
    return out


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """tensor.RMSNorm (tensor/ops.go:105) over the last axis."""
    if x.dtype != torch.float32 or w.dtype != torch.float32:
        raise Refused("RMSNorm", f"x is {x.dtype} and w is {w.dtype}; this kernel reads f32")
    width = x.shape[-1]
    if w.numel() != width:
        raise Refused("RMSNorm", f"x's rows are {width} wide and w holds {w.numel()}")
    x = x.contiguous()
    out = torch.empty_like(x)
    rows = x.numel() // max(width, 1)
    if rows:
        rt.launch("RMSNorm", [x, w.contiguous(), out], rt.row_dims(rows, width, eps))
    return out


def rope(x: torch.Tensor, positions: torch.Tensor, rotary_dim: int, base: float) -> torch.Tensor:
    """tensor.RoPE (tensor/ops.go:208): interleaved pairs over the first rotary_dim elements of each
    row, one position per row; works on a copy, as the reference does."""
    if x.dtype != torch.float32 or x.dim() != 2:
        raise Refused("RoPE", f"x is {x.dtype} {tuple(x.shape)}; it is f32 [rows, width]")
    rows, width = x.shape
    if rotary_dim <= 0 or rotary_dim % 2 or rotary_dim > width:
        raise Refused("RoPE", f"RotaryDim is {rotary_dim} over rows of {width}; it is even and at "
                      "most the width")
    if not _is_u32(positions) or positions.numel() != rows:
        raise Refused("RoPE", f"positions are {positions.dtype}[{positions.numel()}]; one u32 per "
                      f"row, {rows} of them")
    out = x.contiguous().clone()
    if rows:
        rt.launch("RoPE", [positions.contiguous(), out], rt.rope_params(rows, width, rotary_dim, base))
    return out


def _same(op, a, b):
    if a.dtype != torch.float32 or b.dtype != torch.float32:
        raise Refused(op, f"the operands are {a.dtype} and {b.dtype}; this kernel reads f32")
    if tuple(a.shape) != tuple(b.shape):
        raise Refused(op, f"the operands are {tuple(a.shape)} and {tuple(b.shape)}; they are the "
                      "same shape")


def swiglu(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """tensor.SwiGLU (tensor/elementwise.go:161): silu(a) * b."""
    _same("SwiGLU", a, b)
    out = torch.empty_like(a, memory_format=torch.contiguous_format)
    if a.numel():
        rt.launch("SwiGLU", [a.contiguous(), b.contiguous(), out])
    return out


def add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """tensor.Add (tensor/elementwise.go:88)."""
    _same("Add", a, b)
    out = torch.empty_like(a, memory_format=torch.contiguous_format)
    if a.numel():
        rt.launch("ElemAdd", [a.contiguous(), b.contiguous(), out])
    return out


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """tensor.Argmax (tensor/sample.go:157): per row, ties to the lowest index; u32 out."""
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise Refused("Argmax", f"logits are {logits.dtype} {tuple(logits.shape)}; f32 [rows, vocab]")
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=U32, device=logits.device)
    if rows:
        rt.launch("SampleArgmax", [logits.contiguous(), out], rt.sample_dims(vocab, rows))
    return out


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """tensor.Cast (tensor/ops.go:285) between f32 and f16, narrowing with the reference's rounding."""
    if x.dtype == dtype:
        return x
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    if x.dtype == torch.float32 and dtype == torch.float16:
        name = "CastF32ToF16"
    elif x.dtype == torch.float16 and dtype == torch.float32:
        name = "CastF16ToF32"
    else:
        raise Refused("Cast", f"{x.dtype} to {dtype}; f32 and f16 are built")
    if x.numel():
        rt.launch(name, [x.contiguous(), out])
    return out


# ------------------------------------------------------------------------------- sampling policy
@dataclass
class RowPenalties:
    """tensor.RowPenalties (tensor/rowsample.go): per-row history rings [rows, capacity] of token ids
    (u32), how much of each is filled, the counts scratch [rows, vocab] (u32, rebuilt every step)
    and the three strengths per row."""
    history: torch.Tensor
    counts: torch.Tensor
    filled: torch.Tensor
    repetition: torch.Tensor
    presence: torch.Tensor
    frequency: torch.Tensor


@dataclass
class RowSampling:
    """tensor.RowSampling: every parameter is one value per row.  factor is the inverse temperature,
    0 for a greedy row; top_k / top_p None leaves the node out; bias is (ids u32 [rows, slots],
    values f32 [rows, slots])."""
    factor: Optional[torch.Tensor] = None
    top_k: Optional[torch.Tensor] = None
    top_p: Optional[torch.Tensor] = None
    bias: Optional[tuple] = None
    penalties: Optional[RowPenalties] = None


def softmax(x: torch.Tensor) -> torch.Tensor:
    """tensor.Softmax over the last axis (internal/kernels/norm.go:94)."""
    if x.dtype != torch.float32 or x.dim() < 1 or x.shape[-1] == 0:
        raise Refused("Softmax", f"x is {x.dtype} {tuple(x.shape)}; the kernel reads f32 rows")
    rows, width = x.numel() // x.shape[-1], x.shape[-1]
    out = torch.empty_like(x)
    if rows:
        rt.launch("Softmax", [x.contiguous(), out], rt.row_dims(rows, width, 0.0))
    return out


def sample_rows(logits: torch.Tensor, draws: torch.Tensor, o: RowSampling) -> torch.Tensor:
    """tensor.SampleRows (tensor/rowsample.go): logits [rows, vocab] f32 -> one token id per row.
    bias -> penalties -> x factor -> softmax -> top-k -> top-p -> draw (or the argmax of a row whose
    factor is 0), each a kernel of its own as the reference records them."""
    op = "SampleRows"
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.shape[1] == 0:
        raise Refused(op, f"logits are {logits.dtype} {tuple(logits.shape)}; they are f32 [rows, vocab]")
    rows, vocab = logits.shape
    if o.factor is None:
        raise Refused(op, "Factor is nil; every row needs its inverse temperature, and zero is how a "
                      "row asks for the argmax")
    if draws is None:
        raise Refused(op, "draws is nil; every stochastic row draws against its own uniform, and the "
                      "greedy rows ignore theirs")
    for name, t, u32 in (("Factor", o.factor, False), ("TopK", o.top_k, True), ("TopP", o.top_p, False),
                         ("draws", draws, False)):
        if t is None:
            continue
        if (u32 and not _is_u32(t)) or (not u32 and t.dtype != torch.float32):
            raise Refused(op, f"{name} is {t.dtype} and the kernels read {'u32' if u32 else 'f32'}")
        if t.numel() != rows:
            raise Refused(op, f"{name} holds {t.numel()} entries and the logits hold {rows} rows; there "
                          "is exactly one per row")
    dims = rt.row_sample_dims(vocab, rows)
    x = logits.contiguous()
    dev = x.device
    new = lambda: torch.empty((rows, vocab), dtype=torch.float32, device=dev)
    if rows == 0:
        return torch.empty(0, dtype=torch.int32, device=dev)
    if o.bias is not None:
        ids, values = o.bias
        if not _is_u32(ids) or values.dtype != torch.float32 or ids.numel() != values.numel() or ids.numel() % rows:
            raise Refused(op, "Bias.IDs (u32) and Bias.Values (f32) are both [rows, slots]")
        y = new()
        rt.launch("LogitBias", [x, ids.contiguous(), values.contiguous(), y],
                  rt.row_sample_dims(vocab, rows, 0, ids.numel() // rows))
        x = y
    if o.penalties is not None:
        p = o.penalties
        if not _is_u32(p.history) or not _is_u32(p.counts) or not _is_u32(p.filled):
            raise Refused(op, "the history, the counts and the filled lengths are u32")
        if p.counts.numel() != rows * vocab or p.history.numel() % rows or p.history.numel() == 0:
            raise Refused(op, f"the counts hold {p.counts.numel()} entries for {rows} rows of {vocab}, the "
                          f"history {p.history.numel()}; they are [rows, vocab] and [rows, capacity]")
        cap = p.history.numel() // rows
        pd = rt.row_sample_dims(vocab, rows, cap)
        rt.launch("PenaltyClearRows", [p.counts], pd)
        rt.launch("PenaltyCountRows", [p.history.contiguous(), p.filled, p.counts], pd)
        y = new()
        rt.launch("PenaltyApplyRows", [x, p.counts, p.repetition, p.presence, p.frequency, y], pd)
        x = y
    y = new()
    rt.launch("ScaleRows", [x, o.factor, y], dims)
    x = softmax(y)
    if o.top_k is not None:
        y = new()
        rt.launch("TopKMaskRows", [x, o.top_k, y], dims)
        x = y
    if o.top_p is not None:
        y = new()
        rt.launch("TopPMaskRows", [x, o.top_p, y], dims)
        x = y
    out = torch.empty(rows, dtype=torch.int32, device=dev)
    rt.launch("SampleRows", [x, draws, o.factor, out], dims)
    return out
