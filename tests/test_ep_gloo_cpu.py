"""Expert-parallel wiring with two gloo ranks on CPU: counts exchange, the two all-to-alls, the
regrouping by local expert and its inverse, with the oracle standing in for the grouped kernels.
A routed row is multiplied on its own, so two ranks must reproduce one rank bit for bit."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle_ops
from accel_b200 import moe

E, D, FFN = 4, 128, 256


def _rows(rank, world, total=22):
    """Each rank holds a different number of routed rows; the union is the same for any world."""
    g = torch.Generator().manual_seed(5)
    x = torch.randn(total, D, generator=g)
    expert = torch.randint(0, E, (total,), generator=g, dtype=torch.int32)
    expert[:3] = 2                                        # one expert gets a run of rows, one may get none
    cut = [0, total] if world == 1 else [0, 9, total]
    return x[cut[rank]:cut[rank + 1]].contiguous(), expert[cut[rank]:cut[rank + 1]].contiguous()


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    ffn = moe.ExpertParallelFFN(E, D, FFN, "cpu", seed=3, std=0.05, ops=oracle_ops, quantize=oracle_ops.quantize)
    assert list(ffn.local) == [2 * rank, 2 * rank + 1]
    x, expert = _rows(rank, world)
    out = ffn.forward(x, expert)
    empty = ffn.forward(x[:0], expert[:0]) if rank == 1 else ffn.forward(x, expert)   # a rank with no rows
    q.put((rank, out.numpy(), empty.shape[0]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_expert_parallel_ffn_equals_one_rank():
    one = moe.ExpertParallelFFN(E, D, FFN, "cpu", seed=3, std=0.05, ops=oracle_ops, quantize=oracle_ops.quantize)
    x, expert = _rows(0, 1)
    want = one.forward(x, expert).numpy()
    assert np.abs(want).max() > 0

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict()
    for _ in range(2):
        r, out, n_empty = q.get(timeout=300)
        got[r] = out
        assert n_empty in (0, out.shape[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    both = np.concatenate([got[0], got[1]])
    assert both.shape == want.shape
    assert np.array_equal(both, want)


def test_expert_ranges():
    assert list(moe.expert_range(8, 8, 3)) == [3]
    assert list(moe.expert_range(8, 2, 1)) == [4, 5, 6, 7]
    try:
        moe.expert_range(8, 3, 0)
    except ValueError as e:
        assert "do not divide" in str(e)
    else:
        raise AssertionError("8 experts over 3 ranks was accepted")
