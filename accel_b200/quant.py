"""quant.Int4Quantize and friends (quant/int4.go:71-175) through the C ABI."""
from __future__ import annotations

import numpy as np
import torch

from . import _lib, runtime

INT4_GROUP = 128      # quant.Int4Group
INT4_MAX = 15         # quant.Int4Max


def _vp(a: np.ndarray):
    return a.ctypes.data


def int4_quantize(w) -> tuple:
    """Host-side packing: (packed u32[ceil(n/8)], scales f16 bits u16[groups], zeros u16[groups])."""
    w = np.ascontiguousarray(w, dtype=np.float32).ravel()
    n = w.size
    packed = np.zeros((n + 7) // 8, np.uint32)
    groups = (n + INT4_GROUP - 1) // INT4_GROUP
    scales = np.zeros(groups, np.uint16)
    zeros = np.zeros(groups, np.uint16)
    _lib.check(_lib.lib().ab_int4_quantize(_vp(w), n, _vp(packed), _vp(scales), _vp(zeros)))
    return packed, scales, zeros


def int4_nibble(packed, i: int) -> int:
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    return int(_lib.lib().ab_int4_nibble(_vp(packed), i))


def int4_dequantize(packed, scales, zeros, n: int) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    scales = np.ascontiguousarray(scales, dtype=np.uint16)
    zeros = np.ascontiguousarray(zeros, dtype=np.uint16)
    out = np.zeros(n, np.float32)
    _lib.check(_lib.lib().ab_int4_dequantize(_vp(packed), _vp(scales), _vp(zeros), n, _vp(out)))
    return out


def int4_quantize_device(w: torch.Tensor) -> tuple:
    """The same packing computed on the GPU, bit-identical to the host routine.  Returns
    (packed int32 view of the u32 words, scales float16, zeros float16) on w's device."""
    w = w.contiguous().view(-1)
    n = w.numel()
    packed = torch.empty((n + 7) // 8, dtype=torch.int32, device=w.device)
    groups = (n + INT4_GROUP - 1) // INT4_GROUP
    scales = torch.empty(groups, dtype=torch.float16, device=w.device)
    zeros = torch.empty(groups, dtype=torch.float16, device=w.device)
    runtime.launch("Int4Quantize", [w, packed, scales, zeros])
    return packed, scales, zeros


def int4_column_split(n_cols: int, parts: int, rank: int) -> tuple:
    """Columns [begin, end) of shard `rank`: boundaries on multiples of 128 so a shard's packing is
    bit-identical to the same columns of the unsharded matrix."""
    import ctypes as C
    b, e = C.c_uint32(0), C.c_uint32(0)
    _lib.check(_lib.lib().ab_int4_column_split(n_cols, parts, rank, C.byref(b), C.byref(e)))
    return b.value, e.value
