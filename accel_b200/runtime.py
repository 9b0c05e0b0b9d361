"""Direct dispatch of the sm_100a kernels on torch-owned device memory.

torch supplies device memory and streams; every computation is one `ab_launch` through the C ABI.
The binding order, the lengths block and the std140 uniform bytes are the reference's
(internal/kernels/accel_kernels.go codecs; specs/061-ptx-target.md:152-159)."""
from __future__ import annotations

import ctypes as C
import struct
from typing import Optional, Sequence

import torch

from . import _lib

# ---------------------------------------------------------------- std140 uniform blocks


def gemm_dims(M: int, N: int, K: int) -> bytes:                 # GEMMDims, gemm.go:11
    return struct.pack("<IIII", M, N, K, 0)


def attn_dims(q_heads, kv_heads, head_dim, scale) -> bytes:     # AttnDims
    return struct.pack("<IIIf", q_heads, kv_heads, head_dim, scale)


def paged_dims(q_heads, kv_heads, head_dim, block, scale) -> bytes:     # PagedDims, paged.go:16
    return struct.pack("<IIIIfIII", q_heads, kv_heads, head_dim, block, scale, 0, 0, 0)


def batched_dims(batch, q_heads, kv_heads, head_dim, block, max_pages, scale) -> bytes:
    # BatchedDims / RaggedDims, batched.go:13, ragged.go:17
    return struct.pack("<IIIIIIfI", batch, q_heads, kv_heads, head_dim, block, max_pages, scale, 0)


def prefill_dims(q_heads, kv_heads, head_dim, q_seq, base, scale) -> bytes:         # PrefillDims, prefill.go:18
    return struct.pack("<IIIIIfII", q_heads, kv_heads, head_dim, q_seq, base, scale, 0, 0)


def paged_prefill_dims(q_heads, kv_heads, head_dim, q_seq, base, block, scale) -> bytes:
    # PagedPrefillDims, prefill.go:368
    return struct.pack("<IIIIIIfI", q_heads, kv_heads, head_dim, q_seq, base, block, scale, 0)


def grouped_dims(experts, K, N) -> bytes:                       # GroupedDims, grouped.go:10
    return struct.pack("<IIII", experts, K, N, 0)


def grouped_tiled_dims(experts, tokens, K, N) -> bytes:         # GroupedTiledDims
    return struct.pack("<IIII", experts, tokens, K, N)


def segment_dims(rows) -> bytes:                                # SegmentDims, segment.go
    return struct.pack("<IIII", rows, 0, 0, 0)


def row_params(rows, width, capacity) -> bytes:                 # RowParams, elementwise.go
    return struct.pack("<IIII", rows, width, capacity, 0)


def row_dims(rows, width, eps) -> bytes:                        # RowDims, norm.go
    return struct.pack("<IIfI", rows, width, eps, 0)


def rope_params(rows, width, rotary_dim, base) -> bytes:        # RoPEParams, elementwise.go
    return struct.pack("<IIIf", rows, width, rotary_dim, base)


def sample_dims(vocab, rows) -> bytes:                          # SampleDims, sample.go
    return struct.pack("<IIII", vocab, rows, 0, 0)


def row_sample_dims(vocab, rows, history=0, slots=0) -> bytes:  # RowSampleDims, rowsample.go:25
    return struct.pack("<IIII", vocab, rows, history, slots)


def top_dims(vocab, k=0, p=0.0) -> bytes:                        # TopDims, topk.go:10
    return struct.pack("<IIfI", vocab, k, p, 0)


def penalty_dims(vocab, history, count, repetition, presence, frequency) -> bytes:   # PenaltyDims, penalty.go:15
    return struct.pack("<IIIfffII", vocab, history, count, repetition, presence, frequency, 0, 0)


# ---------------------------------------------------------------- launch
_workspaces: dict = {}


def kernel_names():
    L = _lib.lib()
    return [L.ab_kernel_name(i).decode() for i in range(L.ab_kernel_count())]


def workspace_bytes(name: str, lengths: Sequence[int], uniform: Optional[bytes]) -> int:
    L = _lib.lib()
    lens = (C.c_uint32 * len(lengths))(*lengths)
    out = C.c_size_t(0)
    ub = uniform or b""
    _lib.check(L.ab_workspace_bytes(name.encode(), lens, len(lengths), ub if ub else None,
                                    len(ub), C.byref(out)))
    return out.value


def _workspace(device: torch.device, need: int) -> Optional[torch.Tensor]:
    if need == 0:
        return None
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def launch(name: str, bindings: Sequence[torch.Tensor], uniform: Optional[bytes] = None,
           lengths: Optional[Sequence[int]] = None, workspace: Optional[torch.Tensor] = None):
    """One dispatch of reference kernel `name` on the current stream of the tensors' device.
    `lengths` defaults to each tensor's element count."""
    L = _lib.lib()
    if not bindings:
        raise ValueError("no bindings")
    dev = bindings[0].device
    if dev.type != "cuda":
        raise _lib.AccelError(_lib.AB_ERR_NO_DEVICE, f"{name}: bindings live on {dev}; this backend "
                              "runs on a CUDA device and has no CPU path")
    for t in bindings:
        if t.device != dev or not t.is_contiguous():
            raise ValueError(f"{name}: every binding is a contiguous tensor on {dev}")
    lens = list(lengths) if lengths is not None else [t.numel() for t in bindings]
    ub = uniform or b""
    if workspace is None:
        workspace = _workspace(dev, workspace_bytes(name, lens, uniform))
    ptrs = (C.c_void_p * len(bindings))(*[t.data_ptr() for t in bindings])
    clens = (C.c_uint32 * len(lens))(*lens)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        rc = L.ab_launch(name.encode(), C.c_void_p(stream), ptrs, clens, len(bindings),
                         ub if ub else None, len(ub),
                         C.c_void_p(workspace.data_ptr()) if workspace is not None else None,
                         workspace.numel() if workspace is not None else 0)
    _lib.check(rc)


def last_selection() -> str:
    return _lib.lib().ab_last_selection().decode()


def launch_count() -> int:
    """Kernels this library has launched (or recorded into a capture) so far in this process."""
    return int(_lib.lib().ab_launch_count())
