"""The one-shot peer all-reduce: as a single rank on one GPU (the kernel's copy, flag, sum and
epoch logic, eagerly and from a graph), and across every GPU of the box against NCCL when there
are at least two (child processes under torchrun, one rank per GPU)."""
import os
import subprocess
import sys

import pytest
import torch

from accel_b200 import _lib
from accel_b200.peer import PeerAllReduce

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_single_rank_is_a_copy_and_replays_from_a_graph():
    dev = torch.device("cuda:0")
    ar = PeerAllReduce(70000, dev)
    for n in (4, 1024, 65536, 70000):
        x = torch.randn(n, device=dev)
        want = x.clone()
        ar.all_reduce_(x)
        assert torch.equal(x, want)
    y = torch.randn(4096, device=dev)
    want = y * 4                  # two replays (capture itself runs nothing)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            ar.all_reduce_(y)
            y.mul_(2)
        g.replay()
        g.replay()
    torch.cuda.synchronize()
    assert torch.allclose(y, want)
    ar.check()


def test_a_wait_that_runs_out_reports_a_timeout_and_the_next_call_stays_aligned():
    """Two "ranks" whose buffers both live on this GPU; rank 1 never calls.  Rank 0's wait is given
    2^14 polls: the kernel must return, leave the output alone, record call 1 as timed out, and
    still count the call, so that call 2 (for which rank 1's signal and data are put in place by
    hand) sums correctly.  A wait that gives up is an ordinary return: nothing here can hang."""
    import ctypes as C
    dev = torch.device("cuda:0")
    L = _lib.lib()
    cap, n = 1024, 512
    nbytes = int(L.ab_peer_allreduce_buffer_bytes(cap))
    bufs = [torch.zeros(nbytes // 4, dtype=torch.float32, device=dev) for _ in range(2)]
    state = torch.zeros(int(L.ab_peer_allreduce_state_bytes()) // 4, dtype=torch.int32, device=dev)
    ptrs = (C.c_void_p * 2)(bufs[0].data_ptr(), bufs[1].data_ptr())
    sp = C.c_void_p(state.data_ptr())
    _lib.check(L.ab_peer_allreduce_set_spin_limit(sp, 1 << 14))
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    x = torch.randn(n, device=dev)
    out = torch.full((n,), -7.0, device=dev)
    _lib.check(L.ab_peer_allreduce_f32(stream, ptrs, sp, 0, 2, C.c_void_p(x.data_ptr()),
                                       C.c_void_p(out.data_ptr()), n, cap))
    torch.cuda.synchronize()
    assert torch.all(out == -7.0), "a call that gave up must not write its output"
    failed = C.c_uint32(0)
    rc = L.ab_peer_allreduce_error(sp, C.byref(failed))
    assert rc == _lib.AB_ERR_TIMEOUT and failed.value == 1
    with pytest.raises(_lib.AccelError, match="gave up waiting"):
        _lib.check(rc)
    assert int(state[0]) == 1, "the call counter advances even when the call gave up"

    # call 2 uses data half 0 (epoch & 1): rank 1's part and its flag for call 2, placed by hand
    _lib.check(L.ab_peer_allreduce_clear_error(sp))
    other = torch.randn(n, device=dev)
    bufs[1][64:64 + n] = other                                   # behind the 64 flag words
    bufs[0].view(torch.int32)[1] = 2                             # flag[rank 1] in rank 0's buffer
    torch.cuda.synchronize()
    _lib.check(L.ab_peer_allreduce_f32(stream, ptrs, sp, 0, 2, C.c_void_p(x.data_ptr()),
                                       C.c_void_p(out.data_ptr()), n, cap))
    torch.cuda.synchronize()
    assert L.ab_peer_allreduce_error(sp, None) == 0
    assert torch.equal(out, x + other)
    assert int(state[0]) == 2


def test_refusals():
    dev = torch.device("cuda:0")
    ar = PeerAllReduce(1024, dev)
    with pytest.raises(_lib.AccelError, match="multiple of 4"):
        ar.all_reduce_(torch.zeros(6, device=dev))
    with pytest.raises(_lib.AccelError, match="capacity"):
        ar.all_reduce_(torch.zeros(2048, device=dev))
    with pytest.raises(_lib.AccelError, match="contiguous f32"):
        ar.all_reduce_(torch.zeros(8, device=dev, dtype=torch.float16))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_matches_nccl_across_the_gpus_of_the_box():
    n = min(torch.cuda.device_count(), 8)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                          "--master-addr", "127.0.0.1", "--master-port", "29611",
                          os.path.join(HERE, "peer_allreduce_check.py")],
                         env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, (out.stdout[-1500:], out.stderr[-3000:])
    assert "OK world=" in out.stdout
