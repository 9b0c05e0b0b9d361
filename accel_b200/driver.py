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

    def import_ptr(self, device_ptr: int, nbytes: int) -> Block:
        """A block over device memory the caller owns (a torch tensor's storage, say); the caller
        keeps that memory alive for as long as a plan names the block."""
        h = C.c_void_p()
        _lib.check(_lib.lib().ab_block_import(self._h, C.c_void_p(device_ptr), nbytes, C.byref(h)))
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
                collect_timings: bool = False, max_in_flight: int = 0) -> Executable:
        """GraphCompiler.Compile: validates everything knowable now.  max_in_flight is
        CompileOptions.MaxInFlight (tensor/compile.go:19-27): zero means one submission at a time."""
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
        plan = _lib.Plan(arr, len(nodes), n_slots, int(collect_timings), int(max_in_flight))
        h = C.c_void_p()
        _lib.check(_lib.lib().ab_compile(self._h, C.byref(plan), C.byref(h)))
        return Executable(self, h, keep)

    def close(self):
        if self._h:
            _lib.check(_lib.lib().ab_close(self._h))
            self._h = None


# ---------------------------------------------------------------------------- plan cache, buckets
@dataclass
class CompileOptions:
    """tensor.CompileOptions (tensor/compile.go:15-28)."""
    label: str = ""
    max_in_flight: int = 0


def plan_identity(nodes: Sequence[Union[Dispatch, Copy, HostWrite]], n_slots: int) -> bytes:
    """A digest of a recorded plan's structure: every node's kind, kernel name, workgroup count,
    uniform bytes, payload size and operands (block handle or slot, offset, size), in order.  Two
    plans with the same shapes and different kernels or wiring have different identities: "shape
    alone is never a sufficient key" (tensor/cache.go:50-56)."""
    import hashlib
    h = hashlib.sha256()

    def put(*items):
        for it in items:
            b = it if isinstance(it, bytes) else str(it).encode()
            h.update(len(b).to_bytes(8, "little"))
            h.update(b)

    def operand(o: Operand):
        put("slot" if o.block is None else "block", o.slot if o.block is None else (o.block._h.value or 0),
            o.offset, o.size)

    put("accel_b200 plan identity v1", n_slots, len(nodes))
    for nd in nodes:
        if isinstance(nd, Dispatch):
            put("dispatch", nd.kernel, *nd.count, nd.uniform or b"", len(nd.bindings))
            for o in nd.bindings:
                operand(o)
        elif isinstance(nd, Copy):
            put("copy")
            operand(nd.src)
            operand(nd.dst)
        elif isinstance(nd, HostWrite):
            put("host-write", len(nd.payload))        # the payload's bytes are set per submission
            operand(nd.dst)
        else:
            raise TypeError(f"a plan node is {type(nd)}")
    return h.digest()


class PlanCache:
    """tensor.PlanCache (tensor/cache.go:16-164): compiled executables kept by what they are, so a
    caller whose shape varies compiles each distinct plan once.  Never evicts: a plan owns
    transient device memory a caller may be about to submit against, so the cache grows until
    close(); a caller who needs a bound gives it a bounded set of shapes (Buckets)."""

    def __init__(self, dev: "Device"):
        import threading
        self.dev = dev
        self._mu = threading.Lock()
        self._plans: dict = {}
        self._closed = False
        self.compiles = 0

    def _key(self, identity: bytes, opts: CompileOptions) -> bytes:
        # tensor/cache.go:70-110: the graph, the device's identity, and every option that changes
        # what compiling produces; the label is left out (two plans differing only in what they are
        # called are the same plan)
        import hashlib
        h = hashlib.sha256()
        h.update(b"accel/tensor plan key v1")
        h.update(identity)
        h.update(device_info(self.dev.ordinal)["token"])
        h.update(b"opts v3")
        h.update(f"max-in-flight={opts.max_in_flight}".encode())
        return h.digest()

    def compile(self, record, opts: Optional[CompileOptions] = None) -> Executable:
        """`record()` returns (nodes, n_slots): recording is cheap and is the only way to learn the
        identity; what a hit saves is everything after it (validation, workspaces, the lowering)."""
        opts = opts or CompileOptions()
        with self._mu:
            if self._closed:
                raise AccelError(_lib.AB_ERR_INVALID, "the plan cache is closed")
            nodes, n_slots = record()
            k = self._key(plan_identity(nodes, n_slots), opts)
            hit = self._plans.get(k)
            if hit is not None:
                return hit
            exe = self.dev.compile(nodes, n_slots, max_in_flight=opts.max_in_flight)
            self.compiles += 1
            self._plans[k] = exe
            return exe

    def __len__(self) -> int:
        with self._mu:
            return len(self._plans)

    def close(self):
        with self._mu:
            if self._closed:
                return
            self._closed = True
            for exe in self._plans.values():
                exe.close()
            self._plans = {}


class Buckets:
    """tensor.Buckets (tensor/cache.go:166-246): a sorted set of sequence lengths a caller compiles
    plans for; a prompt runs in the smallest bucket that fits."""

    def __init__(self, *sizes: int):
        if not sizes:
            raise ValueError("a bucket set needs at least one size")
        out = sorted(int(s) for s in sizes)
        for i, s in enumerate(out):
            if s <= 0:
                raise ValueError(f"bucket {i} is {s}, and a length is positive")
            if i and out[i] == out[i - 1]:
                raise ValueError(f"bucket size {s} appears twice")
        self._sizes = out

    def sizes(self) -> List[int]:
        return list(self._sizes)

    def for_(self, n: int) -> int:
        """The smallest bucket that holds n tokens; a prompt longer than the largest bucket is an
        error rather than a truncation."""
        import bisect
        if n <= 0:
            raise ValueError(f"a prompt of {n} tokens")
        i = bisect.bisect_left(self._sizes, n)
        if i == len(self._sizes):
            raise ValueError(f"a prompt of {n} tokens exceeds the largest bucket, {self._sizes[-1]}; add a "
                             "bucket or split the prompt, because truncating it would answer a different question")
        return self._sizes[i]
