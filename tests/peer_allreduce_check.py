"""Run under torchrun by test_peer_allreduce_gpu.py (one rank per GPU): the one-shot peer
all-reduce against the process group's all-reduce, eagerly and replayed from a CUDA graph."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, __file__.rsplit("/", 2)[0])
from accel_b200.peer import PeerAllReduce  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    ar = PeerAllReduce(16 * 32000, dev, regions=(16 * 4096, 16 * 4096, 1000))
    worst = 0.0
    for n in (4, 65536, 16 * 32000, 1000 * 4):
        for it in range(5):
            g = torch.Generator(device=dev).manual_seed(1000 * rank + it)
            x = torch.randn(n, device=dev, generator=g)
            want = x.clone()
            dist.all_reduce(want)
            got = ar.all_reduce_(x.clone())
            torch.cuda.synchronize()
            worst = max(worst, float((got - want).abs().max() / want.abs().max().clamp_min(1e-30)))
            gathered = [torch.empty_like(got) for _ in range(world)]
            dist.all_gather(gathered, got)
            assert all(torch.equal(gathered[0], t) for t in gathered), "ranks disagree on the bits"
    # the fused form: residual + all-reduce, then RMSNorm, against the plain call and torch
    from accel_b200 import runtime as rt
    for rows, width in ((16, 4096), (3, 1000), (16, 256)):
        g = torch.Generator(device=dev).manual_seed(77 + rank)
        part = torch.randn(rows, width, device=dev, generator=g)
        g0 = torch.Generator(device=dev).manual_seed(5)              # the same on every rank
        res = torch.randn(rows, width, device=dev, generator=g0)
        gain = torch.rand(width, device=dev, generator=g0) + 0.5
        s1, n1 = torch.empty_like(part), torch.empty_like(part)
        ar.all_reduce_add_rms_norm(part, res, gain, s1, n1, 1e-5)
        summed = ar.all_reduce_(part.clone())
        s2, n2 = torch.empty_like(part), torch.empty_like(part)
        rt.launch("AddRMSNorm", [res, summed, gain, s2, n2], rt.row_dims(rows, width, 1e-5))
        torch.cuda.synchronize()
        assert torch.equal(s1, s2) and torch.equal(n1, n2), (rows, width)
    # the in-place forms: the partial result is written into a region of the rank's own buffer
    for which, (rows, width) in ((0, (16, 4096)), (1, (5, 1000)), (0, (16, 4096))):
        g = torch.Generator(device=dev).manual_seed(300 + 10 * which + rank)
        part = torch.randn(rows, width, device=dev, generator=g)
        g0 = torch.Generator(device=dev).manual_seed(6)
        res = torch.randn(rows, width, device=dev, generator=g0)
        gain = torch.rand(width, device=dev, generator=g0) + 0.5
        ar.region(which)[:rows * width].copy_(part.view(-1))
        plain = ar.all_reduce_region(which, torch.empty(rows * width, device=dev)).view(rows, width)
        other = 1 - which                          # a region is rewritten only after another call
        ar.region(other)[:rows * width].copy_(part.view(-1))
        s1, n1 = torch.empty_like(part), torch.empty_like(part)
        ar.all_reduce_region_add_rms_norm(other, res, gain, s1, n1, 1e-5)
        copied = ar.all_reduce_(part.clone())
        s2, n2 = torch.empty_like(part), torch.empty_like(part)
        rt.launch("AddRMSNorm", [res, copied, gain, s2, n2], rt.row_dims(rows, width, 1e-5))
        torch.cuda.synchronize()
        assert torch.equal(plain, copied) and torch.equal(s1, s2) and torch.equal(n1, n2), (which, rows, width)
    # 64 calls per replay, as a decode step makes them
    x = torch.randn(16, 4096, device=dev)
    ref = x.clone()
    for _ in range(64 * 3 + 64):
        dist.all_reduce(ref)
        ref /= world
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        def body():
            for _ in range(64):
                ar.all_reduce_(x)
                x.div_(world)
        body()                                   # warm-up: 64 calls
        s.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=s):
            body()
        for _ in range(3):
            gr.replay()
    torch.cuda.synchronize()
    ar.check()
    err = float((x - ref).abs().max() / ref.abs().max())

    if rank == 0:
        print(f"OK world={world} worst_rel_err={worst:.3e} replayed_rel_err={err:.3e}", flush=True)
    assert worst < 1e-5 and err < 1e-4
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)


if __name__ == "__main__":
    main()
