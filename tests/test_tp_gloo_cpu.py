"""Tensor-parallel wiring with two gloo ranks on CPU: the shard plan, the group-aligned weight
shards and the two all-reduces per layer, run through the decode step with the oracle standing in
for the kernels.  The sharded step must reproduce the unsharded one: the row-parallel products are
partial sums added in a different order, so logits agree to f32 rounding and greedy tokens are
equal."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle_ops
from accel_b200 import decode as dec


def _cfg():
    return dec.ModelConfig(layers=2, d_model=256, n_heads=4, n_kv_heads=4, head_dim=64, ffn=640,
                           vocab=640, block=8)      # 5 groups: the two ranks hold 3 and 2


def _run_steps(engine, steps, batch):
    for s in range(batch):
        engine.reserve(s, steps + 1)
    engine.upload_pages()
    engine.prepare()
    tok = np.arange(batch) + 3
    toks, logits = [], []
    for _ in range(steps):
        engine.set_inputs(tok)
        engine.run_step()
        engine.lengths_host += 1
        tok = engine.next_tokens.numpy().copy()
        toks.append(tok)
        logits.append(engine.full_logits().numpy().copy())
    return np.array(toks), np.array(logits)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    cfg = _cfg()
    shard = dec.Shard.plan(cfg, world, rank)
    model = dec.DecodeModel(cfg, shard, "cpu", seed=11, quantize=oracle_ops.quantize, std=0.08)
    eng = dec.DecodeEngine(model, 2, max_context=32, ops=oracle_ops)
    toks, logits = _run_steps(eng, 6, 2)
    if rank == 0:
        q.put((toks, logits, len(shard.ffn), len(shard.vocab)))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_tensor_parallel_step_matches_the_unsharded_step():
    cfg = _cfg()
    one = dec.DecodeEngine(dec.DecodeModel(cfg, dec.Shard.plan(cfg, 1, 0), "cpu", seed=11,
                                           quantize=oracle_ops.quantize, std=0.08),
                           2, max_context=32, ops=oracle_ops)
    want_toks, want_logits = _run_steps(one, 6, 2)

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    toks, logits, ffn_local, vocab_local = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # 640 = 5 groups -> 3 + 2; 768 = 6 groups -> 3 + 3: uneven and even group-aligned splits
    assert ffn_local == 384 and vocab_local == 384
    assert np.array_equal(toks, want_toks)
    assert np.max(np.abs(logits - want_logits)) <= 2e-5 * np.max(np.abs(want_logits))


def test_shard_plan_covers_the_7b_shape_at_every_degree():
    cfg = dec.ModelConfig()
    for tp in (1, 2, 4, 8):
        shards = [dec.Shard.plan(cfg, tp, r) for r in range(tp)]
        assert sum(len(s.heads) for s in shards) == 32
        assert sum(len(s.ffn) for s in shards) == 11008 and sum(len(s.vocab) for s in shards) == 32000
        for s in shards:
            assert s.ffn.start % 128 == 0 and s.ffn.stop % 128 == 0
            assert s.vocab.start % 128 == 0 and s.vocab.stop % 128 == 0
            assert list(s.heads) == list(s.kv_heads)
    assert [len(dec.Shard.plan(cfg, 8, r).ffn) for r in range(8)] == [1408] * 6 + [1280] * 2
