"""One-shot all-reduce over NVLink peer memory for the tensor-parallel decode step.

`PeerAllReduce` owns this rank's buffer (flags + two data halves), maps every peer's buffer, and
launches `ab_peer_allreduce_f32` (csrc/peer_allreduce.cu) on the caller's stream.  The mapping is
done by torch's symmetric-memory allocator (CUDA virtual-memory handles exchanged between the
ranks of a process group); the kernel only sees the resulting pointers.  Multicast objects are
not used: the library's loads and stores are plain peer accesses.

accel is single-device: there is no reference counterpart (the tensor-parallel layer sits above
the per-device plan, see decode.py)."""
from __future__ import annotations

import ctypes as C
import os

import torch
import torch.distributed as dist

from . import _lib


class PeerAllReduce:
    def __init__(self, capacity_floats: int, device: torch.device, group=None, regions=()):
        """Collective: every rank of `group` (default: the world) constructs one, with the same
        capacity (the largest element count a copying call will carry) and the same `regions`
        (element counts of caller-owned parts of the buffer for the in-place calls).  Without a
        process group the object is a single rank (the sum is a copy through its own buffer)."""
        L = _lib.lib()
        self.capacity = (int(capacity_floats) + 3) // 4 * 4
        at = int(L.ab_peer_allreduce_region_offset_bytes(self.capacity))
        self._region_at = []
        for n in regions:
            at = (at + 255) // 256 * 256
            self._region_at.append((at, int(n)))
            at += int(n) * 4
        self.nbytes = nbytes = (at + 255) // 256 * 256
        if not dist.is_initialized():
            self.group, self.rank, self.world = None, 0, 1
            self._buf = torch.zeros(nbytes // 4, dtype=torch.float32, device=device)
            self._ptrs = (C.c_void_p * 1)(self._buf.data_ptr())
            self._state = torch.zeros(int(L.ab_peer_allreduce_state_bytes()) // 4, dtype=torch.int32, device=device)
            return
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        if self.world > 8:
            raise _lib.AccelError(_lib.AB_ERR_INVALID, f"PeerAllReduce: {self.world} ranks (at most 8)")
        try:
            symm.set_backend("CUDA")
        except Exception:
            pass                                   # already chosen by an earlier allocation
        self._buf = symm.empty(nbytes // 4, dtype=torch.float32, device=device)
        self._buf.zero_()
        self._hdl = symm.rendezvous(self._buf, self.group)
        ptrs = [int(p) for p in self._hdl.buffer_ptrs]
        if len(ptrs) != self.world or ptrs[self.rank] != self._buf.data_ptr():
            raise _lib.AccelError(_lib.AB_ERR_INVALID, "PeerAllReduce: the allocator's peer table does not "
                                  "match this rank's buffer")
        self._ptrs = (C.c_void_p * self.world)(*ptrs)
        self._state = torch.zeros(int(L.ab_peer_allreduce_state_bytes()) // 4, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(self.group)                   # every rank's flags are zero before any call

    def all_reduce_(self, t: torch.Tensor, stream=None) -> torch.Tensor:
        """Sums `t` (f32, contiguous, a multiple of 4 elements, at most the capacity) over the
        ranks in place; every rank ends with the same bits."""
        if t.dtype != torch.float32 or not t.is_contiguous() or not t.is_cuda:
            raise _lib.AccelError(_lib.AB_ERR_INVALID, "PeerAllReduce: a contiguous f32 CUDA tensor is required")
        s = stream if stream is not None else torch.cuda.current_stream(t.device)
        _lib.check(_lib.lib().ab_peer_allreduce_f32(
            C.c_void_p(s.cuda_stream), self._ptrs, C.c_void_p(self._state.data_ptr()), self.rank, self.world,
            C.c_void_p(t.data_ptr()), C.c_void_p(t.data_ptr()), t.numel(), self.capacity))
        return t

    def region(self, i: int) -> torch.Tensor:
        """Region i of this rank's own buffer: write the partial result here (it is an ordinary
        device tensor), then call one of the in-place forms."""
        at, n = self._region_at[i]
        return self._buf[at // 4:at // 4 + n]

    def all_reduce_region(self, i: int, out: torch.Tensor, stream=None) -> torch.Tensor:
        """out = sum over the ranks of region i (out.numel() elements, a multiple of 4)."""
        at, n = self._region_at[i]
        if out.numel() > n or out.dtype != torch.float32 or not out.is_contiguous():
            raise _lib.AccelError(_lib.AB_ERR_INVALID, "PeerAllReduce: out must be contiguous f32 within the region")
        s = stream if stream is not None else torch.cuda.current_stream(out.device)
        _lib.check(_lib.lib().ab_peer_allreduce_inplace_f32(
            C.c_void_p(s.cuda_stream), self._ptrs, C.c_void_p(self._state.data_ptr()), self.rank, self.world, at,
            C.c_void_p(out.data_ptr()), out.numel(), self.nbytes))
        return out

    def all_reduce_region_add_rms_norm(self, i: int, residual, gain, sum_out, norm_out, eps: float, stream=None,
                                       amax_out=None):
        """sum_out = residual + (sum over the ranks of region i), norm_out = RMSNorm(sum_out) * gain;
        amax_out [rows] f32 (optional) receives every row's largest |norm_out|."""
        import struct
        at, n = self._region_at[i]
        rows, width = residual.shape
        if rows * width > n:
            raise _lib.AccelError(_lib.AB_ERR_INVALID, "PeerAllReduce: the rows do not fit the region")
        s = stream if stream is not None else torch.cuda.current_stream(residual.device)
        p = lambda x: C.c_void_p(x.data_ptr())
        eps_bits = struct.unpack("<I", struct.pack("<f", eps))[0]
        _lib.check(_lib.lib().ab_peer_allreduce_inplace_add_rmsnorm_amax_f32(
            C.c_void_p(s.cuda_stream), self._ptrs, p(self._state), self.rank, self.world, at, p(residual), p(gain),
            p(sum_out), p(norm_out), rows, width, eps_bits, self.nbytes,
            p(amax_out) if amax_out is not None else None))

    def all_reduce_add_rms_norm(self, t, residual, gain, sum_out, norm_out, eps: float, stream=None):
        """sum_out = residual + all-reduce(t), norm_out = RMSNorm(sum_out) * gain, in one launch;
        t, residual, sum_out, norm_out are [rows, width] f32, gain [width]."""
        import struct
        rows, width = t.shape
        s = stream if stream is not None else torch.cuda.current_stream(t.device)
        p = lambda x: C.c_void_p(x.data_ptr())
        eps_bits = struct.unpack("<I", struct.pack("<f", eps))[0]
        _lib.check(_lib.lib().ab_peer_allreduce_add_rmsnorm_f32(
            C.c_void_p(s.cuda_stream), self._ptrs, p(self._state), self.rank, self.world, p(t), p(residual),
            p(gain), p(sum_out), p(norm_out), rows, width, eps_bits, self.capacity))

    def check(self) -> None:
        """Synchronous: raises when a call of this rank gave up waiting for its peers."""
        _lib.check(_lib.lib().ab_peer_allreduce_error(C.c_void_p(self._state.data_ptr()), None))

    def set_spin_limit(self, polls: int) -> None:
        """How long a call waits for its peers before giving up, in polls of a flag (0: the
        default, about a second)."""
        _lib.check(_lib.lib().ab_peer_allreduce_set_spin_limit(C.c_void_p(self._state.data_ptr()), int(polls)))

    def clear_error(self) -> None:
        _lib.check(_lib.lib().ab_peer_allreduce_clear_error(C.c_void_p(self._state.data_ptr())))

    @property
    def error_word(self) -> torch.Tensor:
        """The device word that holds the 1-based number of the call that gave up (0: none); a
        caller that already reads results back every step can read this beside them."""
        return self._state[3:4]
