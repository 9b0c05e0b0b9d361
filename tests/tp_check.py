"""Run under torchrun by test_decode_gpu.py (one rank per GPU): the tensor-parallel decode step on
the GPUs of the box against the unsharded step on one GPU, for both collectives (the process
group's all-reduce and this library's peer all-reduce with the fused residual add and RMSNorm),
eagerly and replayed from a captured graph."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, __file__.rsplit("/", 2)[0])
from accel_b200 import decode as dec  # noqa: E402


def run(engine, steps, batch, graph):
    engine.fill_context(11, seed=2)
    for s in range(batch):
        engine.reserve(s, 11 + steps + 2)
    engine.upload_pages()
    first = np.arange(batch) + 7
    toks, logits = [], []
    if graph:
        engine.set_inputs(first)
        engine.capture(warmup=1)
        engine.set_inputs(first)
        for _ in range(steps):
            engine.run_step()
            toks.append(engine.next_tokens.cpu().numpy().copy())
            logits.append(engine.full_logits().cpu().numpy().copy())
            engine.advance_on_device()
    else:
        tok = first
        for _ in range(steps):
            tok = engine.step(tok)
            toks.append(tok.copy())
            logits.append(engine.full_logits().cpu().numpy().copy())
    return np.array(toks), np.array(logits)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    cfg = dec.ModelConfig(layers=2, d_model=512, n_heads=8, n_kv_heads=8, head_dim=64, ffn=1280, vocab=1024, block=16)
    batch, steps = 4, 5
    one = dec.DecodeEngine(dec.DecodeModel(cfg, dec.Shard.plan(cfg, 1, 0), dev, seed=13, std=0.08), batch, max_context=64)
    want_t, want_l = run(one, steps, batch, graph=False)
    model = dec.DecodeModel(cfg, dec.Shard.plan(cfg, world, rank), dev, seed=13, std=0.08)
    scale = float(np.abs(want_l).max())
    report = []
    for collective in ("nccl", "peer"):
        for graph in (False, True):
            eng = dec.DecodeEngine(model, batch, max_context=64, group=dist.group.WORLD, collective=collective)
            got_t, got_l = run(eng, steps, batch, graph)
            err = float(np.abs(got_l - want_l).max()) / scale
            # greedy tokens agree wherever the unsharded top two logits are clearly apart
            top2 = np.sort(want_l, axis=2)[:, :, -2:]
            clear = (top2[:, :, 1] - top2[:, :, 0]) > 1e-3 * scale
            assert err < 5e-4, (collective, graph, err)
            assert np.array_equal(got_t[clear], want_t[clear]), (collective, graph)
            if eng._peer is not None:
                eng._peer.check()
            report.append(f"{collective}/{'graph' if graph else 'eager'}={err:.1e}")
    if rank == 0:
        print(f"OK world={world} logits_rel_err " + " ".join(report), flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)


if __name__ == "__main__":
    main()
