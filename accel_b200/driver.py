"""The driver seam through the C ABI: Device / Block / Executable / Fence, shaped like accel's
internal/driver (driver.go:149-238, plan.go:31-428).  This is the binding a Go backend package
would make with purego; here it is ctypes, so the tests and the end-to-end benchmark drive the
library exactly as accel would: host buffers in, a compiled plan submitted, host buffers out."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Union

import numpy as np

from . import _lib
from ._lib import AccelError, DeviceLost  # noqa: F401  (re-exported)

MEMORY_DEVICE = _lib.AB_MEMORY_DEVICE
MEMORY_HOST_VISIBLE = _lib.AB_MEMORY_HOST_VISIBLE


def device_count() -> int:
    n = C.c_int(0)
    _lib.check(_lib.lib().ab_device_count(C.byref(n)))
    return n.value


def device_info(ordinal: int = 0) -> dict:
    info = _lib.Info()
    _lib.check(_lib.lib().ab_device_info(ordinal, C.byref(info)))
    return {"name": info.name.decode(), "token": bytes(info.token), "total_memory": info.total_memory,
            "sm_count": info.sm_count, "cc": (info.cc_major, info.cc_minor),
            "max_shared_per_block": info.max_shared_per_block,
            "storage_offset_alignment": info.storage_offset_alignment,
            "subgroup_size": info.subgroup_size}


class Block:
    """driver.Block: Write and Read are synchronous; bytes() is None for device memory."""

    def __init__(self, dev: "Device", handle):
        self.dev, self._h = dev, handle

    @property
    def size(self) -> int:
        return _lib.lib().ab_block_size(self._h)

    @property
    def device_ptr(self) -> int:
        return _lib.lib().ab_block_device_ptr(self._h) or 0

    def bytes(self) -> Optional[int]:
        return _lib.lib().ab_block_bytes(self._h)

    def write(self, offset: int, src: np.ndarray):
        src = np.ascontiguousarray(src)
        _lib.check(_lib.lib().ab_block_write(self._h, offset, src.ctypes.data, src.nbytes))

    def read(self, offset: int, dst: np.ndarray):
        assert dst.flags["C_CONTIGUOUS"]
        _lib.check(_lib.lib().ab_block_read(self._h, offset, dst.ctypes.data, dst.nbytes))
        return dst

    def free(self):
        """Refused (AB_ERR_BUSY) while a live executable still names the block."""
        if self._h:
            _lib.check(_lib.lib().ab_block_free(self._h))
            self._h = None


@dataclass
class Operand:
    """driver.Operand: a fixed block or a 1-based slot, plus offset and size in bytes."""
    block: Optional[Block] = None
    slot: int = 0
    offset: int = 0
    size: int = 0


@dataclass
class Dispatch:
    kernel: str
    bindings: Sequence[Operand]
    uniform: Optional[bytes] = None
    count: Sequence[int] = (1, 1, 1)


@dataclass
class Copy:
    src: Operand
    dst: Operand


@dataclass
class HostWrite:
    dst: Operand
    payload: bytes


class Fence:
    def __init__(self, handle):
        self._h = handle

    def wait(self):
        try:
            _lib.check(_lib.lib().ab_fence_wait(self._h))
        finally:
            pass

    def done(self) -> bool:
        return _lib.check(_lib.lib().ab_fence_done(self._h)) == 1

    def elapsed_ns(self) -> int:
        return _lib.lib().ab_fence_elapsed_ns(self._h)

    def free(self):
        if self._h:
            _lib.lib().ab_fence_free(self._h)
            self._h = None

    __del__ = free


class Executable:
    """driver.Executable: Rebind is all-or-nothing; Submit begins the work and returns."""

    def __init__(self, dev: "Device", handle, keep):
        self.dev, self._h, self._keep = dev, handle, keep

    def rebind(self, bindings: Sequence[tuple]):
        """bindings: (slot, Block, offset) triples."""
        arr = (_lib.SlotBinding * len(bindings))()
        for i, (slot, block, off) in enumerate(bindings):
            arr[i].slot, arr[i].block, arr[i].offset = slot, block._h, off
        _lib.check(_lib.lib().ab_exec_rebind(self._h, arr, len(bindings)))

    def set_uniform(self, node: int, data: bytes, index: int = 0):
        _lib.check(_lib.lib().ab_exec_set_uniform(self._h, node, index, data, len(data)))

    def set_payload(self, node: int, data: bytes):
        _lib.check(_lib.lib().ab_exec_set_payload(self._h, node, data, len(data)))

    def submit(self) -> Fence:
        h = C.c_void_p()
        _lib.check(_lib.lib().ab_exec_submit(self._h, C.byref(h)))
        return Fence(h)

    def close(self):
        if self._h:
            _lib.lib().ab_exec_close(self._h)
            self._h = None


class Device:
    """driver.Device opened through Adapter.Open."""

    def __init__(self, ordinal: int = 0, lose_at_submission: int = 0, use_graphs: bool = False):
        _lib.check(_lib.lib().ab_init())
        opts = _lib.OpenOpts(C.sizeof(_lib.OpenOpts), lose_at_submission, int(use_graphs))
        h = C.c_void_p()
        _lib.check(_lib.lib().ab_open(ordinal, C.byref(opts), C.byref(h)))
        self._h = h
        self.ordinal = ordinal

    def alloc(self, nbytes: int, kind: int = MEMORY_DEVICE, label: str = "") -> Block:
        h = C.c_void_p()
        _lib.check(_lib.lib().ab_alloc(self._h, kind, nbytes, label.encode(), C.byref(h)))
        return Block(self, h)

    def upload(self, arr: np.ndarray, label: str = "") -> Block:
        arr = np.ascontiguousarray(arr)
        b = self.alloc(max(arr.nbytes, 1), MEMORY_DEVICE, label)
        if arr.nbytes:
            b.write(0, arr)
        return b

    def lost(self) -> bool:
        return _lib.lib().ab_lost(self._h) == _lib.AB_ERR_DEVICE_LOST

    def supports_kernel(self, name: str) -> bool:
        return _lib.lib().ab_supports_kernel(self._h, name.encode(), None) == _lib.AB_OK

    def compile(self, nodes: Sequence[Union[Dispatch, Copy, HostWrite]], n_slots: int = 0,
                collect_timings: bool = False) -> Executable:
        """GraphCompiler.Compile: validates everything knowable now."""
        keep: List[object] = []
        arr = (_lib.Node * len(nodes))()

        def operands(ops):
            oa = (_lib.Operand * len(ops))()
            for i, o in enumerate(ops):
                oa[i].block = o.block._h if o.block is not None else None
                oa[i].slot, oa[i].offset, oa[i].size = o.slot, o.offset, o.size
            keep.append(oa)
            return oa

        for i, nd in enumerate(nodes):
            if isinstance(nd, Dispatch):
                arr[i].op = _lib.AB_OP_DISPATCH
                arr[i].kernel = nd.kernel.encode()
                arr[i].count[0], arr[i].count[1], arr[i].count[2] = nd.count
                arr[i].n_bindings = len(nd.bindings)
                arr[i].bindings = operands(nd.bindings)
                if nd.uniform:
                    buf = C.create_string_buffer(nd.uniform, len(nd.uniform))
                    keep.append(buf)
                    arr[i].uniform = C.cast(buf, C.c_void_p)
                    arr[i].uniform_bytes = len(nd.uniform)
            elif isinstance(nd, Copy):
                arr[i].op = _lib.AB_OP_COPY
                arr[i].n_bindings = 2
                arr[i].bindings = operands([nd.src, nd.dst])
            elif isinstance(nd, HostWrite):
                arr[i].op = _lib.AB_OP_HOST_WRITE
                arr[i].n_bindings = 1
                arr[i].bindings = operands([nd.dst])
                buf = C.create_string_buffer(nd.payload, len(nd.payload))
                keep.append(buf)
                arr[i].payload = C.cast(buf, C.c_void_p)
                arr[i].payload_bytes = len(nd.payload)
            else:
                raise TypeError(f"node {i} is {type(nd)}; this is a compute-only backend")
        plan = _lib.Plan(arr, len(nodes), n_slots, int(collect_timings), 0)
        h = C.c_void_p()
        _lib.check(_lib.lib().ab_compile(self._h, C.byref(plan), C.byref(h)))
        return Executable(self, h, keep)

    def close(self):
        if self._h:
            _lib.check(_lib.lib().ab_close(self._h))
            self._h = None
