"""ctypes binding of libaccelb200.so.  There is no fallback: if the library is missing or an entry
point fails, the caller gets an exception, never a CPU result."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libaccelb200.so"

AB_OK = 0
AB_ERR_INVALID = -1
AB_ERR_UNSUPPORTED = -2
AB_ERR_OOM = -3
AB_ERR_DEVICE_LOST = -4
AB_ERR_BUSY = -5
AB_ERR_CUDA = -6
AB_ERR_NO_DEVICE = -7
AB_ERR_TIMEOUT = -8

AB_MEMORY_DEVICE = 0
AB_MEMORY_HOST_VISIBLE = 1
AB_OP_COPY, AB_OP_HOST_WRITE, AB_OP_DISPATCH = 0, 1, 2


class AccelError(RuntimeError):
    """A negative ab_status, with the library's message."""

    def __init__(self, code: int, message: str):
        super().__init__(f"{message} (ab_status {code})")
        self.code = code
        self.message = message


class DeviceLost(AccelError):
    pass


class Info(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("token", C.c_uint8 * 16), ("total_memory", C.c_uint64),
                ("sm_count", C.c_uint32), ("cc_major", C.c_uint32), ("cc_minor", C.c_uint32),
                ("max_shared_per_block", C.c_uint32), ("storage_offset_alignment", C.c_uint32),
                ("subgroup_size", C.c_uint32)]


class OpenOpts(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("lose_at_submission", C.c_int32),
                ("use_graphs", C.c_int32)]


class Operand(C.Structure):
    _fields_ = [("block", C.c_void_p), ("slot", C.c_uint32), ("_pad", C.c_uint32),
                ("offset", C.c_uint64), ("size", C.c_uint64)]


class Node(C.Structure):
    _fields_ = [("op", C.c_int32), ("barrier_before", C.c_int32), ("kernel", C.c_char_p),
                ("digest", C.c_char_p), ("count", C.c_uint32 * 3), ("n_bindings", C.c_int32),
                ("bindings", C.POINTER(Operand)), ("uniform", C.c_void_p),
                ("uniform_bytes", C.c_uint64), ("payload", C.c_void_p),
                ("payload_bytes", C.c_uint64)]


class Plan(C.Structure):
    _fields_ = [("nodes", C.POINTER(Node)), ("n_nodes", C.c_int32), ("n_slots", C.c_int32),
                ("collect_timings", C.c_int32), ("max_in_flight", C.c_int32)]


class SlotBinding(C.Structure):
    _fields_ = [("slot", C.c_uint32), ("_pad", C.c_uint32), ("block", C.c_void_p),
                ("offset", C.c_uint64)]


# Every symbol include/accel_b200.h declares: (name, restype, argtypes)
_P = C.c_void_p
SYMBOLS = [
    ("ab_error_string", C.c_char_p, [C.c_int]),
    ("ab_last_error", C.c_char_p, []),
    ("ab_init", C.c_int, []),
    ("ab_device_count", C.c_int, [C.POINTER(C.c_int)]),
    ("ab_device_info", C.c_int, [C.c_int, C.POINTER(Info)]),
    ("ab_open", C.c_int, [C.c_int, C.POINTER(OpenOpts), C.POINTER(_P)]),
    ("ab_close", C.c_int, [_P]),
    ("ab_lost", C.c_int, [_P]),
    ("ab_alloc", C.c_int, [_P, C.c_int, C.c_size_t, C.c_char_p, C.POINTER(_P)]),
    ("ab_block_bytes", _P, [_P]),
    ("ab_block_device_ptr", _P, [_P]),
    ("ab_block_import", C.c_int, [_P, _P, C.c_size_t, C.POINTER(_P)]),
    ("ab_block_size", C.c_size_t, [_P]),
    ("ab_block_write", C.c_int, [_P, C.c_size_t, _P, C.c_size_t]),
    ("ab_block_read", C.c_int, [_P, C.c_size_t, _P, C.c_size_t]),
    ("ab_block_free", C.c_int, [_P]),
    ("ab_supports_kernel", C.c_int, [_P, C.c_char_p, C.c_char_p]),
    ("ab_compile", C.c_int, [_P, C.POINTER(Plan), C.POINTER(_P)]),
    ("ab_exec_rebind", C.c_int, [_P, C.POINTER(SlotBinding), C.c_int]),
    ("ab_exec_set_uniform", C.c_int, [_P, C.c_int, C.c_int, _P, C.c_size_t]),
    ("ab_exec_set_payload", C.c_int, [_P, C.c_int, _P, C.c_size_t]),
    ("ab_exec_submit", C.c_int, [_P, C.POINTER(_P)]),
    ("ab_exec_close", C.c_int, [_P]),
    ("ab_fence_wait", C.c_int, [_P]),
    ("ab_fence_done", C.c_int, [_P]),
    ("ab_fence_elapsed_ns", C.c_uint64, [_P]),
    ("ab_fence_free", None, [_P]),
    ("ab_kernel_count", C.c_int, []),
    ("ab_kernel_name", C.c_char_p, [C.c_int]),
    ("ab_workspace_bytes", C.c_int, [C.c_char_p, _P, C.c_int, _P, C.c_size_t,
                                     C.POINTER(C.c_size_t)]),
    ("ab_launch", C.c_int, [C.c_char_p, _P, _P, _P, C.c_int, _P, C.c_size_t, _P, C.c_size_t]),
    ("ab_quant_matmul_int4_noalloc", C.c_int, [_P, _P, _P, _P, _P, _P, C.c_uint32, C.c_uint32,
                                               C.c_uint32]),
    ("ab_last_selection", C.c_char_p, []),
    ("ab_launch_count", C.c_uint64, []),
    ("ab_peer_allreduce_buffer_bytes", C.c_size_t, [C.c_uint32]),
    ("ab_peer_allreduce_state_bytes", C.c_size_t, []),
    ("ab_peer_allreduce_f32", C.c_int, [_P, C.POINTER(_P), _P, C.c_int, C.c_int, _P, _P, C.c_uint32,
                                        C.c_uint32]),
    ("ab_peer_allreduce_add_rmsnorm_f32", C.c_int, [_P, C.POINTER(_P), _P, C.c_int, C.c_int, _P, _P, _P, _P, _P,
                                                    C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]),
    ("ab_peer_allreduce_region_offset_bytes", C.c_size_t, [C.c_uint32]),
    ("ab_peer_allreduce_inplace_f32", C.c_int, [_P, C.POINTER(_P), _P, C.c_int, C.c_int, C.c_size_t, _P, C.c_uint32,
                                                C.c_size_t]),
    ("ab_peer_allreduce_inplace_add_rmsnorm_f32", C.c_int, [_P, C.POINTER(_P), _P, C.c_int, C.c_int, C.c_size_t, _P, _P,
                                                            _P, _P, C.c_uint32, C.c_uint32, C.c_uint32, C.c_size_t]),
    ("ab_peer_allreduce_inplace_add_rmsnorm_amax_f32", C.c_int, [_P, C.POINTER(_P), _P, C.c_int, C.c_int, C.c_size_t, _P, _P,
                                                                 _P, _P, C.c_uint32, C.c_uint32, C.c_uint32, C.c_size_t, _P]),
    ("ab_peer_allreduce_error", C.c_int, [_P, C.POINTER(C.c_uint32)]),
    ("ab_peer_allreduce_set_spin_limit", C.c_int, [_P, C.c_uint32]),
    ("ab_peer_allreduce_clear_error", C.c_int, [_P]),
    ("ab_group_open", C.c_int, [_P, C.c_int, C.c_uint32, C.POINTER(_P)]),
    ("ab_group_close", C.c_int, [_P]),
    ("ab_group_size", C.c_int, [_P]),
    ("ab_group_ordinal", C.c_int, [_P, C.c_int]),
    ("ab_group_buffer", _P, [_P, C.c_int]),
    ("ab_group_state", _P, [_P, C.c_int]),
    ("ab_group_stream", _P, [_P, C.c_int]),
    ("ab_group_peer_table", _P, [_P]),
    ("ab_group_all_reduce_f32", C.c_int, [_P, _P, _P, C.c_uint32]),
    ("ab_group_synchronize", C.c_int, [_P]),
    ("ab_int4_quantize", C.c_int, [_P, C.c_size_t, _P, _P, _P]),
    ("ab_int4_nibble", C.c_uint32, [_P, C.c_size_t]),
    ("ab_int4_dequantize", C.c_int, [_P, _P, _P, C.c_size_t, _P]),
    ("ab_int8_quantize", C.c_int, [_P, C.c_size_t, _P, _P]),
    ("ab_int8_dequantize", C.c_int, [_P, _P, C.c_size_t, _P]),
    ("ab_f32_to_f16", C.c_uint16, [_P]),
    ("ab_f16_to_f32", None, [C.c_uint16, _P]),
    ("ab_blockpool_new", C.c_int, [C.c_int, C.c_int, C.POINTER(_P)]),
    ("ab_blockpool_close", None, [_P]),
    ("ab_blockpool_block_size", C.c_int, [_P]),
    ("ab_blockpool_available", C.c_int, [_P]),
    ("ab_blockpool_grow", C.c_int, [_P, _P, C.c_int, C.c_int]),
    ("ab_blockpool_free", C.c_int, [_P, _P, C.c_int]),
    ("ab_blockpool_positions", C.c_int, [_P, C.c_int]),
    ("ab_int4_prepack_bytes", C.c_size_t, [C.c_uint32, C.c_uint32]),
    ("ab_int4_prepack", C.c_int, [_P, _P, _P, _P, C.c_uint32, C.c_uint32, _P]),
    ("ab_int4_stream_error", C.c_int, []),
    ("ab_int4_column_split", C.c_int, [C.c_uint32, C.c_int, C.c_int, C.POINTER(C.c_uint32),
                                       C.POINTER(C.c_uint32)]),
]

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m accel_b200.build` (needs nvcc). "
                "accel_b200 has no CPU path and will not run without it.")
        L = C.CDLL(str(LIB_PATH))
        for name, res, args in SYMBOLS:
            fn = getattr(L, name)      # AttributeError here = the header and the library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc: int) -> int:
    """Raises on a negative status; returns non-negative results unchanged."""
    if rc >= 0:
        return rc
    msg = lib().ab_last_error().decode("utf-8", "replace")
    if rc == AB_ERR_DEVICE_LOST:
        raise DeviceLost(rc, msg)
    raise AccelError(rc, msg)
