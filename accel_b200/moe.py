"""Expert-parallel grouped int4 FFN (a MoE layer's expert half) over the ranks of one box.

The reference's GroupedMatMul (tensor/grouped.go:138) takes rows sorted by expert and the per-expert
counts, on one device.  Expert parallelism sits above it, as tensor parallelism sits above the
linears: rank r owns experts [r*E/W, (r+1)*E/W) with their gate, up and down matrices (each
quantized on its own, so nothing constrains the split), and a layer is

    sort rows by expert -> exchange counts -> all-to-all of the rows -> regroup by local expert
    -> GroupedMatMulInt4 (gate, up) -> SwiGLU -> GroupedMatMulInt4 (down)
    -> undo the regrouping -> all-to-all back -> undo the sort

The two all-to-alls are the process group's (NCCL over NVLink on GPUs, gloo in the CPU tests); the
split sizes come from the exchanged counts, which is the one host synchronisation per layer.  Each
routed row is multiplied on its own whatever rows surround it, so the result does not depend on
the number of ranks: the tests compare W ranks with one, bit for bit.

accel is single-device: no reference counterpart for the parallel part."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from . import runtime as rt

I32 = torch.int32


@dataclass
class ExpertWeights:
    """The int4 planes of the local experts' [K, N] matrices, end to end in expert order."""
    codes: torch.Tensor
    scales: torch.Tensor
    zeros: torch.Tensor
    K: int
    N: int
    packed: Optional[torch.Tensor] = None     # the experts' load-time prepacks, end to end (CUDA only)


def expert_range(experts: int, world: int, rank: int) -> range:
    if experts % world:
        raise ValueError(f"{experts} experts do not divide over {world} ranks")
    per = experts // world
    return range(rank * per, (rank + 1) * per)


class ExpertParallelFFN:
    def __init__(self, experts: int, d_model: int, ffn: int, device, group=None, seed: int = 77,
                 std: float = 0.02, ops=rt, quantize=None, init_on_device: bool = False,
                 parallel: bool = True):
        """init_on_device: draw the random weights with the device's generator (fast at full size;
        the values then depend on the device type, not on the number of ranks).
        parallel=False: own every expert and ignore the process group (the single-rank answer)."""
        import torch.distributed as dist
        self.group = group
        on = parallel and dist.is_initialized()
        self.world = dist.get_world_size(group) if on else 1
        self.rank = dist.get_rank(group) if on else 0
        self.E, self.d, self.ffn, self.ops = experts, d_model, ffn, ops
        self.device = torch.device(device)
        self.local = expert_range(experts, self.world, self.rank)
        self._init_dev = self.device if init_on_device else torch.device("cpu")
        self.use_packed = True         # False: the kernel over quant.Int4Quantize's planes as they are
        if quantize is None:
            from . import quant
            quantize = quant.int4_quantize_device
        self.gate = self._make(seed, 0, d_model, ffn, std, quantize)
        self.up = self._make(seed, 1, d_model, ffn, std, quantize)
        self.down = self._make(seed, 2, ffn, d_model, std, quantize)

    def _make(self, seed, which, K, N, std, quantize) -> ExpertWeights:
        """Expert e's matrix depends on (seed, which, e) only, so every world size holds the same
        experts."""
        planes = []
        for e in self.local:
            g = torch.Generator(device=self._init_dev).manual_seed(seed * 1000003 + which * 1009 + e)
            w = (torch.randn(K, N, generator=g, device=self._init_dev) * std).to(self.device)
            planes.append(quantize(w))
        cat = lambda i: torch.cat([p[i].reshape(-1) for p in planes])
        packed = None
        if self.device.type == "cuda" and self.ops is rt and N % 128 == 0 and K % 4 == 0:
            # the permutation the tcgen05 tile kernel streams (each expert's matrix on its own)
            from . import quant
            packed = torch.cat([quant.int4_prepack(c, s_, z, K, N).view(torch.uint8).reshape(-1) for c, s_, z in planes])
        return ExpertWeights(cat(0), cat(1), cat(2), K, N, packed)

    # -- the pieces, separately testable ---------------------------------------------------
    def _grouped(self, x, w: ExpertWeights, counts, out):
        n_local = len(self.local)
        offsets = torch.zeros(n_local + 1, dtype=I32, device=x.device)
        self.ops.launch("SegmentOffsets", [counts, offsets], rt.segment_dims(n_local))
        if w.packed is not None and self.use_packed:
            self.ops.launch("GroupedMatMulInt4Packed", [x, w.packed.view(I32), offsets, out],
                            rt.grouped_tiled_dims(n_local, x.shape[0], w.K, w.N))
            return out
        self.ops.launch("GroupedMatMulInt4", [x, w.codes, w.scales, w.zeros, offsets, out],
                        rt.grouped_tiled_dims(n_local, x.shape[0], w.K, w.N))
        return out

    def local_experts(self, x_sorted: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
        """Rows sorted by LOCAL expert with their counts -> the experts' outputs, same order."""
        rows = x_sorted.shape[0]
        z = lambda n: torch.zeros((rows, n), dtype=torch.float32, device=x_sorted.device)
        if rows == 0:
            return z(self.d)
        gate = self._grouped(x_sorted, self.gate, counts, z(self.ffn))
        up = self._grouped(x_sorted, self.up, counts, z(self.ffn))
        act = z(self.ffn)
        self.ops.launch("SwiGLU", [gate, up, act])
        return self._grouped(act, self.down, counts, z(self.d))

    def forward(self, x: torch.Tensor, expert: torch.Tensor) -> torch.Tensor:
        """x: this rank's routed rows [R, d_model] f32; expert: their expert ids [R] (0 .. E-1).
        Returns the experts' outputs for those rows, in the rows' order."""
        import torch.distributed as dist
        R, W, per = x.shape[0], self.world, len(self.local)
        expert = expert.to(torch.int64)
        order = torch.argsort(expert, stable=True)
        xs = x[order].contiguous()
        counts = torch.bincount(expert, minlength=self.E).to(I32)              # [E] = [W, per]
        if W == 1:
            ys = self.local_experts(xs, counts)
        else:
            # 1. counts: rank s tells rank r how many rows it sends for each of r's experts
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts, group=self.group)        # [W(src), per]
            send_rows = counts.view(W, per).sum(1).tolist()                      # host sync
            recv_mat = recv_counts.view(W, per).cpu()
            recv_rows = recv_mat.sum(1).tolist()
            # 2. rows
            got = torch.empty((sum(recv_rows), self.d), dtype=torch.float32, device=x.device)
            dist.all_to_all_single(got, xs, output_split_sizes=recv_rows, input_split_sizes=send_rows,
                                   group=self.group)
            # 3. arrived ordered by (source, expert): regroup by (expert, source)
            src = torch.repeat_interleave(torch.arange(W), torch.tensor(recv_rows))
            exp_of = torch.repeat_interleave(torch.arange(per).repeat(W), recv_mat.reshape(-1))
            regroup = torch.argsort(exp_of * W + src, stable=True).to(x.device)
            local_counts = recv_mat.sum(0).to(I32).to(x.device)
            out_local = self.local_experts(got[regroup].contiguous(), local_counts)
            # 4. back the way they came
            back = torch.empty_like(out_local)
            back[regroup] = out_local
            ys = torch.empty((R, self.d), dtype=torch.float32, device=x.device)
            dist.all_to_all_single(ys, back, output_split_sizes=send_rows, input_split_sizes=recv_rows,
                                   group=self.group)
        out = torch.empty_like(ys)
        out[order] = ys
        return out
