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
