"""Run under torchrun by test_moe_gpu.py (one rank per GPU): the expert-parallel FFN across the
GPUs of the box against the same layer on one rank (every rank also builds all experts locally
to have the single-rank answer for its own rows)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, __file__.rsplit("/", 2)[0])
from accel_b200 import moe  # noqa: E402

E, D, FFN = 8, 512, 1024


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    ep = moe.ExpertParallelFFN(E, D, FFN, dev, seed=21, std=0.05)
    g = torch.Generator().manual_seed(100 + rank)
    rows = 300 + 37 * rank
    x = torch.randn(rows, D, generator=g).to(dev)
    expert = torch.randint(0, E, (rows,), generator=g, dtype=torch.int32).to(dev)
    got = ep.forward(x, expert)
    # the single-rank answer: a second object that owns every expert and ignores the process group
    alone = moe.ExpertParallelFFN(E, D, FFN, dev, seed=21, std=0.05, parallel=False)
    want = alone.forward(x, expert)
    torch.cuda.synchronize()
    assert torch.equal(got, want), float((got - want).abs().max())
    if rank == 0:
        print(f"OK world={world} rows={rows} max|y|={float(want.abs().max()):.3f}", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)


if __name__ == "__main__":
    main()
