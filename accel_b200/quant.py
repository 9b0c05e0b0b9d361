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


INT8_BLOCK = 32       # quant.Int8Block
INT8_MAX = 127        # quant.Int8Max


def int8_quantize(w) -> tuple:
    """quant.Int8Quantize (quant/quant.go:60): (quants i8[n], scales f16 bits u16[ceil(n/32)])."""
    w = np.ascontiguousarray(w, dtype=np.float32).ravel()
    quants = np.zeros(w.size, np.int8)
    scales = np.zeros((w.size + INT8_BLOCK - 1) // INT8_BLOCK, np.uint16)
    _lib.check(_lib.lib().ab_int8_quantize(_vp(w), w.size, _vp(quants), _vp(scales)))
    return quants, scales


def int8_dequantize(quants, scales) -> np.ndarray:
    """quant.Int8Dequantize (quant/quant.go:128)."""
    quants = np.ascontiguousarray(quants, dtype=np.int8)
    scales = np.ascontiguousarray(scales, dtype=np.uint16)
    out = np.zeros(quants.size, np.float32)
    _lib.check(_lib.lib().ab_int8_dequantize(_vp(quants), _vp(scales), quants.size, _vp(out)))
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


def int4_prepack(codes: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, K: int, N: int) -> torch.Tensor:
    """The load-time permutation of a device-resident int4 matrix [K, N] (N a multiple of 128) into
    the stream layout the decode-batch kernels read (QuantMatVecInt4Packed / QuantMatMulInt4Packed).
    Returns an int32 tensor holding the packed bytes."""
    import ctypes as C
    L = _lib.lib()
    nbytes = int(L.ab_int4_prepack_bytes(K, N))
    if nbytes == 0:
        raise _lib.AccelError(_lib.AB_ERR_INVALID, f"int4_prepack: K={K} N={N}; N must be a multiple of 128")
    out = torch.empty(nbytes // 4, dtype=torch.int32, device=codes.device)
    with torch.cuda.device(codes.device):
        stream = torch.cuda.current_stream(codes.device).cuda_stream
        _lib.check(L.ab_int4_prepack(C.c_void_p(stream), C.c_void_p(codes.data_ptr()), C.c_void_p(scales.data_ptr()),
                                     C.c_void_p(zeros.data_ptr()), K, N, C.c_void_p(out.data_ptr())))
    return out


def int4_stream_check() -> None:
    """Raises AB_ERR_TIMEOUT when a bounded device-side wait of the prepacked kernels has run out."""
    _lib.check(_lib.lib().ab_int4_stream_error())
