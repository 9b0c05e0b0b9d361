"""ab_group_*: N devices of one process opened together (peer access, peer buffers, states, streams,
the pointer table) and the one-shot all-reduce driven over them from one host thread, with no
process group and no symmetric-memory allocator underneath.  Needs at least two GPUs."""
import ctypes as C

import pytest
import torch

from accel_b200 import _lib

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_a_group_of_devices_all_reduces_without_a_process_group():
    L = _lib.lib()
    n = 4 if torch.cuda.device_count() >= 4 else 2
    ords = (C.c_int * n)(*range(n))
    g = C.c_void_p()
    _lib.check(L.ab_group_open(ords, n, 16 * 4096, C.byref(g)))
    try:
        assert L.ab_group_size(g) == n and [L.ab_group_ordinal(g, r) for r in range(n)] == list(range(n))
        assert all(L.ab_group_buffer(g, r) and L.ab_group_state(g, r) and L.ab_group_stream(g, r) for r in range(n))
        for call in range(3):                                  # several calls: the epochs stay aligned
            xs = [torch.randn(16, 4096, device=f"cuda:{r}", generator=torch.Generator(f"cuda:{r}").manual_seed(10 * call + r))
                  for r in range(n)]
            outs = [torch.empty_like(x) for x in xs]
            for r in range(n):
                torch.cuda.synchronize(r)
            ins = (C.c_void_p * n)(*[x.data_ptr() for x in xs])
            dst = (C.c_void_p * n)(*[o.data_ptr() for o in outs])
            _lib.check(L.ab_group_all_reduce_f32(g, ins, dst, 16 * 4096))
            _lib.check(L.ab_group_synchronize(g))
            want = xs[0].cpu().clone()
            for r in range(1, n):
                want += xs[r].cpu()                            # rank order, as the kernel adds
            for r in range(n):
                assert torch.equal(outs[r].cpu(), want), (call, r)
    finally:
        L.ab_group_close(g)


def test_a_group_refuses_a_device_named_twice():
    L = _lib.lib()
    g = C.c_void_p()
    ords = (C.c_int * 2)(0, 0)
    with pytest.raises(_lib.AccelError, match="named twice"):
        _lib.check(L.ab_group_open(ords, 2, 1024, C.byref(g)))
