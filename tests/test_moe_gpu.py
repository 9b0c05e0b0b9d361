"""The expert-parallel grouped int4 FFN on a B200: one rank against the oracle (dequantize per
expert, reference GroupedMatMul, SwiGLU, GroupedMatMul), and across the GPUs of the box against one
rank, bit for bit, when there are at least two (child processes under torchrun)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import oracle_ops
from accel_b200 import moe
from util import GEMM_TOL, assert_close

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
DEV = "cuda:0"


def test_one_rank_matches_the_oracle():
    E, D, FFN, rows = 4, 256, 384, 150
    gpu = moe.ExpertParallelFFN(E, D, FFN, DEV, seed=8, std=0.05)          # quantized on the device
    cpu = moe.ExpertParallelFFN(E, D, FFN, "cpu", seed=8, std=0.05, ops=oracle_ops, quantize=oracle_ops.quantize)
    for a, b in ((gpu.gate, cpu.gate), (gpu.up, cpu.up), (gpu.down, cpu.down)):   # same experts, same packing
        assert torch.equal(a.codes.cpu(), b.codes) and torch.equal(a.scales.cpu(), b.scales)
        assert torch.equal(a.zeros.cpu(), b.zeros)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(rows, D, generator=g)
    expert = torch.randint(0, E, (rows,), generator=g, dtype=torch.int32)
    expert[expert == 1] = 0                                               # expert 1 gets no rows
    got = gpu.forward(x.to(DEV), expert.to(DEV)).cpu().numpy()
    want = cpu.forward(x, expert).numpy()
    assert_close(got, want, 2 * GEMM_TOL, "expert-parallel FFN, one rank")   # two products deep
    assert gpu.forward(x[:0].to(DEV), expert[:0].to(DEV)).shape == (0, D)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_ranks_reproduce_one_rank_bit_for_bit():
    n = 8 if torch.cuda.device_count() >= 8 else (4 if torch.cuda.device_count() >= 4 else 2)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                          "--master-addr", "127.0.0.1", "--master-port", "29613",
                          os.path.join(HERE, "moe_ep_check.py")],
                         env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, (out.stdout[-1500:], out.stderr[-3000:])
    assert "OK world=" in out.stdout
