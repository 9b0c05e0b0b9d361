"""A Llama-style decode step built from the path's operators: what a caller of accel's tensor API
records once and submits per token (docs/tutorial/09-a-decode-step.md, 11-batching-sequences.md),
with every linear an int4 product and the KV cache paged.

Per layer:  RMSNorm -> Int4MatMul x3 (q,k,v) -> RoPE(q), RoPE(k) -> ScatterRows(K), ScatterRows(V)
            -> Attention (batched paged decode) -> Int4MatMul (wo) -> Add -> RMSNorm
            -> Int4MatMul (gate), Int4MatMul (up) -> SwiGLU -> Int4MatMul (down) -> Add
then        RMSNorm -> Int4MatMul (lm_head) -> Argmax.

Every operator is one dispatch by reference kernel name through `ops.launch` (the C ABI's
ab_launch); torch supplies device memory, streams, CUDA-graph capture and the NCCL process group.

Tensor parallelism (one process per GPU): wq/wk/wv, gate/up and lm_head are split by output
columns on 128-column group boundaries, so each shard's packing is bit-identical to the same
columns of the unsharded matrix; heads and their KV cache follow the q/k/v split; wo and down are
split by rows and their partial sums are all-reduced; the page table, lengths and norm gains are
replicated.  The reference is single-device: sharding is an extension above the per-device plan."""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import List, Optional

import numpy as np
import torch

from . import runtime as rt
from .blockpool import BlockPool
from .quant import int4_column_split

I32 = torch.int32


@dataclass
class ModelConfig:
    layers: int = 32
    d_model: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 32
    head_dim: int = 128
    ffn: int = 11008
    vocab: int = 32000
    eps: float = 1e-5
    rope_base: float = 10000.0
    block: int = 16               # positions per KV page
    cache_dtype: torch.dtype = torch.float32

    def int4_weights(self) -> int:
        d, f = self.d_model, self.ffn
        qkv = d * self.n_heads * self.head_dim + 2 * d * self.n_kv_heads * self.head_dim
        per_layer = qkv + self.n_heads * self.head_dim * d + 3 * d * f
        return self.layers * per_layer + d * self.vocab


@dataclass
class Shard:
    """What rank `rank` of `tp` owns."""
    tp: int
    rank: int
    heads: range          # query heads
    kv_heads: range
    ffn: range            # columns of gate/up = rows of down
    vocab: range

    @staticmethod
    def plan(cfg: ModelConfig, tp: int, rank: int) -> "Shard":
        if cfg.n_heads % tp or cfg.n_kv_heads % tp:
            raise ValueError(f"{cfg.n_heads} query and {cfg.n_kv_heads} KV heads do not divide over {tp} ranks")
        if (cfg.n_heads // tp * cfg.head_dim) % 128:
            raise ValueError("a rank's q/k/v columns must be whole 128-column groups")
        hq, hk = cfg.n_heads // tp, cfg.n_kv_heads // tp
        fb, fe = int4_column_split(cfg.ffn, tp, rank)
        vb, ve = int4_column_split(cfg.vocab, tp, rank)
        return Shard(tp, rank, range(rank * hq, (rank + 1) * hq), range(rank * hk, (rank + 1) * hk),
                     range(fb, fe), range(vb, ve))


@dataclass
class Int4Matrix:
    codes: torch.Tensor      # int32 view of the u32 words, flat [K*N/8]
    scales: torch.Tensor     # f16 flat [K*N/128]
    zeros: torch.Tensor
    K: int
    N: int

    @property
    def nbytes(self) -> int:
        return self.codes.numel() * 4 + self.scales.numel() * 2 + self.zeros.numel() * 2


@dataclass
class PackedMatrix:
    """An int4 matrix in the decode kernels' stream layout (quant.int4_prepack)."""
    packed: torch.Tensor     # int32 words
    K: int
    N: int

    @property
    def nbytes(self) -> int:
        return self.packed.numel() * 4


def pack(m: Int4Matrix) -> PackedMatrix:
    from .quant import int4_prepack
    return PackedMatrix(int4_prepack(m.codes, m.scales, m.zeros, m.K, m.N), m.K, m.N)


def concat_columns(mats) -> Int4Matrix:
    """[K, N1 | N2 | ...]: matrices of equal K side by side (whole 128-column groups each)."""
    K = mats[0].K
    c = torch.cat([m.codes.view(K, m.N // 8) for m in mats], dim=1).contiguous().view(-1)
    s = torch.cat([m.scales.view(K, m.N // 128) for m in mats], dim=1).contiguous().view(-1)
    z = torch.cat([m.zeros.view(K, m.N // 128) for m in mats], dim=1).contiguous().view(-1)
    return Int4Matrix(c, s, z, K, sum(m.N for m in mats))


def interleave_groups(a: Int4Matrix, b: Int4Matrix) -> Int4Matrix:
    """[K, 2N] whose 128-column groups alternate a's and b's: group 2j is a's group j, 2j + 1 is b's."""
    K, G = a.K, a.N // 128
    assert (b.K, b.N) == (a.K, a.N)
    c = torch.stack([a.codes.view(K, G, 16), b.codes.view(K, G, 16)], dim=2).contiguous().view(-1)
    s = torch.stack([a.scales.view(K, G), b.scales.view(K, G)], dim=2).contiguous().view(-1)
    z = torch.stack([a.zeros.view(K, G), b.zeros.view(K, G)], dim=2).contiguous().view(-1)
    return Int4Matrix(c, s, z, K, 2 * a.N)


def shard_columns(codes, scales, zeros, K, N, b, e) -> Int4Matrix:
    """Columns [b, e) of a packed [K, N] matrix; b and e are multiples of 128."""
    c = codes.view(K, N // 8)[:, b // 8:e // 8].contiguous().view(-1)
    s = scales.view(K, N // 128)[:, b // 128:e // 128].contiguous().view(-1)
    z = zeros.view(K, N // 128)[:, b // 128:e // 128].contiguous().view(-1)
    return Int4Matrix(c, s, z, K, e - b)


def shard_rows(codes, scales, zeros, K, N, b, e) -> Int4Matrix:
    """Rows [b, e) of a packed [K, N] matrix with N a multiple of 128 (groups never cross a row)."""
    c = codes.view(K, N // 8)[b:e].contiguous().view(-1)
    s = scales.view(K, N // 128)[b:e].contiguous().view(-1)
    z = zeros.view(K, N // 128)[b:e].contiguous().view(-1)
    return Int4Matrix(c, s, z, e - b, N)


class Layer:
    # wqkv, wo_p, wgu, wd_p: the same matrices prepacked for the decode kernels (GPU models): q | k | v
    # side by side, gate and up interleaved by 128-column group
    __slots__ = ("g1", "g2", "wq", "wk", "wv", "wo", "wg", "wu", "wd", "wqkv", "wo_p", "wgu", "wd_p")


class DecodeModel:
    """Random-init weights of the given shape, quantized with quant.Int4Quantize.  Every rank draws
    the full matrix from the same seed, quantizes it and keeps its shard, so the shards of all
    ranks together are bit-for-bit the unsharded model."""

    def __init__(self, cfg: ModelConfig, shard: Shard, device, seed: int = 1234, ops=rt,
                 quantize=None, std: float = 0.02, prepack: bool = True):
        self.cfg, self.shard, self.device = cfg, shard, torch.device(device)
        d, D = cfg.d_model, cfg.head_dim
        gen = torch.Generator(device=self.device)
        if quantize is None:
            from .quant import int4_quantize_device as quantize
        self._quantize = quantize

        def full(k, n, tag):
            gen.manual_seed(seed * 1000003 + tag)
            w = torch.randn((k, n), generator=gen, device=self.device, dtype=torch.float32) * std
            return self._quantize(w)

        def gain(tag):
            gen.manual_seed(seed * 1000003 + tag)
            return 1.0 + 0.1 * torch.randn(d, generator=gen, device=self.device, dtype=torch.float32)

        hq, hk, fr, vr = shard.heads, shard.kv_heads, shard.ffn, shard.vocab
        self.layers: List[Layer] = []
        for li in range(cfg.layers):
            L = Layer()
            t = 100 * li
            L.g1, L.g2 = gain(t + 1), gain(t + 2)
            nq, nkv = cfg.n_heads * D, cfg.n_kv_heads * D
            L.wq = shard_columns(*full(d, nq, t + 3), d, nq, hq.start * D, hq.stop * D)
            L.wk = shard_columns(*full(d, nkv, t + 4), d, nkv, hk.start * D, hk.stop * D)
            L.wv = shard_columns(*full(d, nkv, t + 5), d, nkv, hk.start * D, hk.stop * D)
            L.wo = shard_rows(*full(nq, d, t + 6), nq, d, hq.start * D, hq.stop * D)
            L.wg = shard_columns(*full(d, cfg.ffn, t + 7), d, cfg.ffn, fr.start, fr.stop)
            L.wu = shard_columns(*full(d, cfg.ffn, t + 8), d, cfg.ffn, fr.start, fr.stop)
            L.wd = shard_rows(*full(cfg.ffn, d, t + 9), cfg.ffn, d, fr.start, fr.stop)
            self.layers.append(L)
        self.g_final = gain(999001)
        self.lm_head = shard_columns(*full(d, cfg.vocab, 999002), d, cfg.vocab, vr.start, vr.stop)
        gen.manual_seed(seed * 1000003 + 999003)
        self.embedding = torch.randn((cfg.vocab, d), generator=gen, device=self.device,
                                     dtype=torch.float32)
        self.packed = False
        if prepack and self.device.type == "cuda":
            self.prepack()

    def prepack(self, keep_planes: bool = True):
        """The load-time permutation of every matrix into the decode kernels' stream layout; q, k and
        v become one matrix (one product, three outputs), gate and up one matrix whose groups
        alternate (one product with SwiGLU in its epilogue).  keep_planes=False drops the
        reference-layout planes of the layers afterwards (the oracle-side step and the unfused
        path need them; a serving process does not)."""
        for L in self.layers:
            L.wqkv = pack(concat_columns([L.wq, L.wk, L.wv]))
            L.wo_p = pack(L.wo)
            L.wgu = pack(interleave_groups(L.wg, L.wu))
            L.wd_p = pack(L.wd)
            if not keep_planes:
                L.wq = L.wk = L.wv = L.wo = L.wg = L.wu = L.wd = None
        self.lm_head_p = pack(self.lm_head)
        self.packed = True

    @classmethod
    def from_host(cls, cfg: ModelConfig, device, layers, g_final, lm_head, embedding,
                  shard: Optional[Shard] = None) -> "DecodeModel":
        """A model from quantized planes held on the host (what a weight loader hands over).
        `layers` is a list of dicts with the gains "g1", "g2" (f32 [d]) and the matrices "wq",
        "wk", "wv", "wo", "wg", "wu", "wd", each a (codes u32, scales f16 bits, zeros f16 bits)
        triple of the unsharded [K, N] matrix in quant.Int4Quantize's layout; `lm_head` is such a
        triple, `embedding` f32 [vocab, d].  The shard's columns and rows are cut here."""
        self = cls.__new__(cls)
        dev = torch.device(device)
        sh = shard if shard is not None else Shard.plan(cfg, 1, 0)
        self.cfg, self.shard, self.device, self._quantize = cfg, sh, dev, None
        d, D = cfg.d_model, cfg.head_dim
        nq, nkv = cfg.n_heads * D, cfg.n_kv_heads * D

        def planes(t):
            c, s, z = (np.ascontiguousarray(a) for a in t)
            return (torch.from_numpy(c.view(np.int32)).to(dev), torch.from_numpy(s.view(np.float16)).to(dev),
                    torch.from_numpy(z.view(np.float16)).to(dev))

        f32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(dev)
        hq, hk, fr, vr = sh.heads, sh.kv_heads, sh.ffn, sh.vocab
        self.layers = []
        for src in layers:
            L = Layer()
            L.g1, L.g2 = f32(src["g1"]), f32(src["g2"])
            L.wq = shard_columns(*planes(src["wq"]), d, nq, hq.start * D, hq.stop * D)
            L.wk = shard_columns(*planes(src["wk"]), d, nkv, hk.start * D, hk.stop * D)
            L.wv = shard_columns(*planes(src["wv"]), d, nkv, hk.start * D, hk.stop * D)
            L.wo = shard_rows(*planes(src["wo"]), nq, d, hq.start * D, hq.stop * D)
            L.wg = shard_columns(*planes(src["wg"]), d, cfg.ffn, fr.start, fr.stop)
            L.wu = shard_columns(*planes(src["wu"]), d, cfg.ffn, fr.start, fr.stop)
            L.wd = shard_rows(*planes(src["wd"]), cfg.ffn, d, fr.start, fr.stop)
            self.layers.append(L)
        self.g_final = f32(g_final)
        self.lm_head = shard_columns(*planes(lm_head), d, cfg.vocab, vr.start, vr.stop)
        self.embedding = f32(embedding)
        self.packed = False
        if dev.type == "cuda":
            self.prepack()
        return self

    def int4_bytes(self) -> int:
        """Bytes of int4 weights one step streams (either layout: the prepack is a permutation)."""
        if self.packed:
            return self.lm_head_p.nbytes + sum(m.nbytes for L in self.layers for m in (L.wqkv, L.wo_p, L.wgu, L.wd_p))
        n = self.lm_head.nbytes
        for L in self.layers:
            n += sum(m.nbytes for m in (L.wq, L.wk, L.wv, L.wo, L.wg, L.wu, L.wd))
        return n


def _u(fmt, *v) -> bytes:
    return struct.pack(fmt, *v)


class DecodeEngine:
    """The recorded step and its state: per-layer paged K/V pools (one state per layer, as the
    reference sizes them), the page table from a BlockPool, and static buffers so the step can be
    captured once as a CUDA graph and replayed."""

    def __init__(self, model: DecodeModel, batch: int, max_context: int, ops=rt, group=None,
                 collective: str = "nccl", use_packed: Optional[bool] = None):
        """collective: how the row-parallel products are summed over the ranks: "nccl" (the
        process group's all-reduce) or "peer" (this library's one-shot kernel over NVLink peer
        memory, peer.PeerAllReduce; GPUs only), or "skip": one rank of a sharded model run on its
        own with the sums over ranks left out (its results are NOT the model's: this is for
        timing and profiling one rank's kernels on one GPU, where a profiler may not wrap a
        multi-rank launch)."""
        cfg, sh = model.cfg, model.shard
        self.model, self.cfg, self.shard, self.ops, self.group = model, cfg, sh, ops, group
        self.collective = collective
        self._peer = None
        # fused support kernels (AddRMSNorm, RopeScatterQKV: extensions of this library, each
        # bit-identical to the chain of reference operators it replaces); an operator table that
        # only knows the reference names, like the oracle's, gets the chain
        self.fuse = ops is rt
        # prepacked weights and the kernels that read them (q | k | v and gate | up as one product each)
        self.use_packed = ops is rt and getattr(model, "packed", False) and use_packed is not False
        self.batch = batch
        dev = model.device
        self.dev = dev
        B, d, D = batch, cfg.d_model, cfg.head_dim
        self.hq, self.hk = len(sh.heads), len(sh.kv_heads)
        self.max_pages = (max_context + cfg.block - 1) // cfg.block
        pool_blocks = B * self.max_pages
        self.capacity = pool_blocks * cfg.block
        self.pool = BlockPool(pool_blocks, cfg.block)
        self.page_rows: List[List[int]] = [[] for _ in range(B)]
        self.lengths_host = np.zeros(B, np.int64)
        kv_shape = (self.capacity, self.hk, D)
        self.k_cache = [torch.zeros(kv_shape, dtype=cfg.cache_dtype, device=dev) for _ in range(cfg.layers)]
        self.v_cache = [torch.zeros(kv_shape, dtype=cfg.cache_dtype, device=dev) for _ in range(cfg.layers)]

        z = lambda *s, dt=torch.float32: torch.zeros(s, dtype=dt, device=dev)
        # per-step inputs (the small buffers a caller writes each step: token, q and k positions,
        # slot, length; docs/tutorial/11-batching-sequences.md:83-103).  They are views of one
        # buffer, each starting on a 256-byte boundary, so one host-to-device copy fills them all.
        sizes = [B, B * self.hq, B * self.hk, B, B]
        starts, at = [], 0
        for n in sizes:
            starts.append(at)
            at += (n + 63) // 64 * 64
        self.inputs = z(at, dt=I32)
        self._in_starts, self._in_sizes = starts, sizes
        view = lambda i: self.inputs[starts[i]:starts[i] + sizes[i]]
        self.tokens, self.pos_q, self.pos_k, self.slots = view(0), view(1), view(2), view(3)
        self.lengths = view(4)               # length AFTER this step's token is appended
        self.pages = z(B, self.max_pages, dt=I32)
        # activations
        self.x, self.h, self.x2 = z(B, d), z(B, d), z(B, d)
        self.q, self.k, self.v = z(B, self.hq * D), z(B, self.hk * D), z(B, self.hk * D)
        self.attn = z(B, self.hq * D)
        self.proj = z(B, d)
        self.gate, self.up, self.act = z(B, len(sh.ffn)), z(B, len(sh.ffn)), z(B, len(sh.ffn))
        self.logits_local = z(B, len(sh.vocab))
        # with the vocabulary split over ranks the step exchanges each rank's (largest logit,
        # index) per row, not the logits; full_logits() gathers them when a caller wants them
        self.logits = self.logits_local if sh.tp == 1 else None
        self.top_pairs = z(B, sh.tp, 2)          # every rank's (value, index) per row, after the exchange
        self._my_pairs = z(B, sh.tp, 2)          # this rank's slot filled, the others zero
        self.next_tokens = z(B, dt=I32)
        self.h_amax = z(B)                       # every row's largest |h|, left by the norm kernels for the products
        # the same for the inputs of wo and down, in parts: one entry per head and warp of the attention
        # kernel, one per 32 columns of the SwiGLU product; the product that follows takes the largest
        self.attn_max = z(B, self.hq * 4)
        self.act_max = z(B, max(len(sh.ffn) // 32, 1))
        self._proj = [self.proj, self.proj]      # where wo and down write their partial results
        if sh.tp > 1 and collective == "peer":
            # the row-parallel products write straight into this rank's peer buffer: two regions
            # used alternately (wo, down), a third for the vocabulary logits
            from .peer import PeerAllReduce
            self._peer = PeerAllReduce(4, dev, group, regions=(B * d, B * d, B * sh.tp * 2))
            self._proj = [self._peer.region(0).view(B, d), self._peer.region(1).view(B, d)]
            self._my_pairs = self._peer.region(2).view(B, sh.tp, 2)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.overlap = True          # run the independent linears of a layer side by side
        self._side: List[torch.cuda.Stream] = []
        self.launches_per_step = 0
        self._pin = None

    # ------------------------------------------------------------------ cache bookkeeping (host)
    def reserve(self, seq: int, n_positions: int):
        """Grow sequence `seq`'s page row to address n_positions (tensor.BlockPool.Grow)."""
        self.page_rows[seq] = self.pool.grow(self.page_rows[seq], n_positions)

    def upload_pages(self):
        host = np.zeros((self.batch, self.max_pages), np.int32)
        for s, row in enumerate(self.page_rows):
            host[s, :len(row)] = row
        self.pages.copy_(torch.from_numpy(host))

    def fill_context(self, context: int, seed: int = 7):
        """Stands in for a prefill: reserves pages for `context` positions per sequence and fills
        those K/V rows with seeded N(0,1) values (f32 or f16 as the cache is)."""
        for s in range(self.batch):
            self.reserve(s, context)
        self.upload_pages()
        gen = torch.Generator(device=self.dev)
        rows = torch.tensor([self.page_rows[s][j // self.cfg.block] * self.cfg.block + j % self.cfg.block
                             for s in range(self.batch) for j in range(context)],
                            dtype=torch.long, device=self.dev)
        for li in range(self.cfg.layers):
            for ci, cache in enumerate((self.k_cache[li], self.v_cache[li])):
                gen.manual_seed(seed * 7919 + li * 2 + ci)
                # every rank draws all KV heads and keeps its own, so shards agree with tp = 1
                full = torch.randn((rows.numel(), self.cfg.n_kv_heads, self.cfg.head_dim),
                                   generator=gen, device=self.dev, dtype=torch.float32)
                part = full[:, self.shard.kv_heads.start:self.shard.kv_heads.stop]
                cache[rows] = part.to(cache.dtype)
        self.lengths_host[:] = context

    def prefill(self, prompts: np.ndarray, chunk: int = 256) -> float:
        """Runs the prompts [batch, T] (token ids) through the model and leaves their K/V in the paged
        cache: the real fill of the context a decode loop starts from.  Every sequence advances
        `chunk` positions at a time, so a product sees batch x chunk rows of activations (the
        batch kernels over the same prepacked weights), RoPE and the scatter into the pages are the
        decode step's fused kernel over those rows, and attention is the paged causal prefill
        kernel, one launch per sequence and layer (internal/kernels/prefill.go:409: row s sees the
        positions <= Base + s).  Pages for T positions are reserved here.  The row-parallel
        products of a sharded model are summed by the process group.  Returns the seconds it took
        (device time)."""
        if not (self.use_packed and self.fuse):
            raise ValueError("prefill runs on the prepacked weights and the fused support kernels")
        cfg, B, D, d = self.cfg, self.batch, self.cfg.head_dim, self.cfg.d_model
        self._count = 0
        prompts = np.asarray(prompts)
        T = prompts.shape[1]
        assert prompts.shape[0] == B and T > 0
        base0 = int(self.lengths_host[0])
        assert np.all(self.lengths_host == base0), "prefill starts every sequence at the same position"
        for sq in range(B):
            self.reserve(sq, base0 + T)
        self.upload_pages()
        dev, blk = self.dev, cfg.block
        f16 = cfg.cache_dtype == torch.float16
        z = lambda *sh, dt=torch.float32: torch.zeros(sh, dtype=dt, device=dev)
        S = min(chunk, T)
        M = B * S
        x, x2, h, proj = z(M, d), z(M, d), z(M, d), z(M, d)
        q, k, v = z(M, self.hq * D), z(M, self.hk * D), z(M, self.hk * D)
        attn, act = z(M, self.hq * D), z(M, len(self.shard.ffn))
        scale = float(np.float32(1.0) / np.float32(np.sqrt(D)))
        launch = self.ops.launch
        pages_of = [self.pages[sq].clone() for sq in range(B)]     # own allocations: a row of the table may start anywhere
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for p0 in range(base0, base0 + T, S):
            s_now = min(S, base0 + T - p0)
            m = B * s_now
            pos = p0 + np.arange(s_now)
            toks = torch.from_numpy(np.ascontiguousarray(prompts[:, p0 - base0:p0 - base0 + s_now]).reshape(-1).astype(np.int32)).to(dev)
            rows_pos = np.tile(pos, B)                                        # row b * s_now + s -> position
            slots = np.concatenate([[self.page_rows[sq][p // blk] * blk + p % blk for p in pos] for sq in range(B)])
            pos_q = torch.from_numpy(np.repeat(rows_pos, self.hq).astype(np.int32)).to(dev)
            pos_k = torch.from_numpy(np.repeat(rows_pos, self.hk).astype(np.int32)).to(dev)
            slots_t = torch.from_numpy(slots.astype(np.int32)).to(dev)
            kv_len = torch.full((1,), p0 + s_now, dtype=I32, device=dev)
            xa, xb = x[:m], x2[:m]
            launch("GatherRows", [self.model.embedding, toks, xa], _u("<IIII", m, d, cfg.vocab, 0))
            norm_u = _u("<IIfI", m, d, cfg.eps, 0)
            for li, lay in enumerate(self.model.layers):
                if li == 0:
                    launch("RMSNorm", [xa, lay.g1, h[:m]], norm_u)
                else:
                    self._all_reduce(proj[:m])
                    launch("AddRMSNorm", [xa, proj[:m], lay.g1, xb, h[:m]], norm_u)
                    xa, xb = xb, xa
                w = lay.wqkv
                launch("QuantMatMulInt4PackedSplit3", [h[:m], w.packed, q[:m], k[:m], v[:m]],
                       _u("<IIIIIIII", m, w.N, w.K, self.hq * D, self.hk * D, 0, 0, 0))
                launch("RopeScatterQKVF16" if f16 else "RopeScatterQKV",
                       [pos_q, pos_k, slots_t, q[:m], k[:m], v[:m], self.k_cache[li], self.v_cache[li]],
                       _u("<IIIIIIfI", m, self.hq, self.hk, D, D, self.capacity, cfg.rope_base, 0))
                for sq in range(B):
                    rows = slice(sq * s_now, (sq + 1) * s_now)
                    launch("AttentionPrefillPagedF16" if f16 else "AttentionPrefillPaged",
                           [q[rows], self.k_cache[li], self.v_cache[li], pages_of[sq], kv_len, attn[rows]],
                           _u("<IIIIIIfI", self.hq, self.hk, D, s_now, p0, blk, scale, 0))
                self._linear(attn[:m], lay.wo_p, proj[:m])
                self._all_reduce(proj[:m])
                launch("AddRMSNorm", [xa, proj[:m], lay.g2, xb, h[:m]], norm_u)
                xa, xb = xb, xa
                w = lay.wgu
                launch("QuantMatMulInt4PackedSwiGLU", [h[:m], w.packed, act[:m]], _u("<IIII", m, w.N, w.K, 0))
                self._linear(act[:m], lay.wd_p, proj[:m])
        t1.record()
        t1.synchronize()
        self.lengths_host += T
        return t0.elapsed_time(t1) / 1e3

    def step_inputs_host(self, token_ids: np.ndarray) -> np.ndarray:
        """The per-step host buffers for the CURRENT lengths, laid out as `self.inputs` is:
        tokens | positions of q rows | positions of k rows | slots | lengths + 1."""
        B, blk = self.batch, self.cfg.block
        pos = self.lengths_host.astype(np.int64)
        slots = np.empty(B, np.int64)
        for s in range(B):
            p = int(pos[s])
            if p // blk >= len(self.page_rows[s]):
                raise RuntimeError(f"sequence {s} has no page for position {p}; reserve() first")
            slots[s] = self.page_rows[s][p // blk] * blk + p % blk
        out = np.zeros(self.inputs.numel(), np.int32)
        parts = [np.asarray(token_ids, np.int64), np.repeat(pos, self.hq), np.repeat(pos, self.hk),
                 slots, pos + 1]
        for st, part in zip(self._in_starts, parts):
            out[st:st + part.size] = part
        return out

    def set_inputs(self, token_ids: np.ndarray):
        """Writes the per-step inputs for the current lengths (synchronous; for setup and tests)."""
        self.inputs.copy_(torch.from_numpy(self.step_inputs_host(token_ids)))

    def advance_on_device(self):
        """Feeds the step's sampled tokens back as the next step's inputs without leaving the
        device: next position = current length, its slot from the page table, length + 1."""
        self.ops.launch("DecodeStepInputs",
                        [self.next_tokens, self.pages, self.tokens, self.pos_q, self.pos_k,
                         self.slots, self.lengths],
                        _u("<IIIIIIII", self.batch, self.hq, self.hk, self.cfg.block,
                           self.max_pages, 0, 0, 0))
        self.lengths_host += 1

    # ------------------------------------------------------------------ the recorded step
    def _launch(self, name, bindings, uniform=None):
        self.ops.launch(name, bindings, uniform)
        self._count += 1

    def _linear(self, a, w, out):
        M = a.shape[0]
        if isinstance(w, PackedMatrix):
            self._launch("QuantMatMulInt4Packed", [a, w.packed, out], _u("<IIII", M, w.N, w.K, 0))
            return
        self._launch("QuantMatMulInt4", [a, w.codes, w.scales, w.zeros, out],
                     _u("<IIII", M, w.N, w.K, 0))

    def _parallel(self, branches):
        """Runs independent branches of the step on side streams (graph branches once captured);
        the first stays on the current stream.  On a CPU stand-in they simply run in order."""
        if self.dev.type != "cuda" or not self.overlap or len(branches) == 1:
            for fn in branches:
                fn()
            return
        main = torch.cuda.current_stream(self.dev)
        while len(self._side) < len(branches) - 1:
            self._side.append(torch.cuda.Stream(device=self.dev))
        for st in self._side[:len(branches) - 1]:
            st.wait_stream(main)
        branches[0]()
        for fn, st in zip(branches[1:], self._side):
            with torch.cuda.stream(st):
                fn()
        for st in self._side[:len(branches) - 1]:
            main.wait_stream(st)

    def _all_reduce(self, t):
        if self.shard.tp > 1 and self.collective != "skip":
            import torch.distributed as dist
            dist.all_reduce(t, group=self.group)

    def record_step(self):
        """Issues one decode step on the current stream.  Reads tokens/pos/slots/lengths/pages,
        appends this token's K/V, writes next_tokens."""
        cfg, B, D, d = self.cfg, self.batch, self.cfg.head_dim, self.cfg.d_model
        self._count = 0
        count = getattr(self.ops, "launch_count", lambda: 0)
        kernels0 = count()
        L = self._launch
        scale = float(np.float32(1.0) / np.float32(np.sqrt(D)))
        L("GatherRows", [self.model.embedding, self.tokens, self.x], _u("<IIII", B, d, cfg.vocab, 0))
        x, x2 = self.x, self.x2
        f16 = cfg.cache_dtype == torch.float16
        rp = _u("<IIII", B, self.hk * D, self.capacity, 0)
        scatter = "ScatterRowsF16" if f16 else "ScatterRows"
        norm_u = _u("<IIfI", B, d, cfg.eps, 0)

        # with the prepacked products the norm kernels also leave every row's largest |h|, and the
        # products that read h take it as a binding instead of running a kernel of their own for it
        h_has_amax = False
        # the decode kernel (fewer than 49 rows) is the one that takes maxima in parts and leaves them
        maxima = self.use_packed and self.fuse and B <= 48

        def add_norm(gain, which):
            """x <- x + (sum over the ranks of the partial product `which`); h <- RMSNorm(x) * gain"""
            nonlocal x, x2, h_has_amax
            proj = self._proj[which]
            h_has_amax = False
            if self._peer is not None and self.fuse:
                # the all-reduce's summing stage adds the residual and normalises: one launch
                self._peer.all_reduce_region_add_rms_norm(which, x, gain, x2, self.h, cfg.eps,
                                                          amax_out=self.h_amax if self.use_packed else None)
                h_has_amax = self.use_packed
                self._count += 1
                x, x2 = x2, x
                return
            if self._peer is not None:
                self._peer.all_reduce_region(which, self.proj)
                self._count += 1
                proj = self.proj
            else:
                self._all_reduce(proj)
            if self.fuse and self.use_packed:
                L("AddRMSNormAmax", [x, proj, gain, x2, self.h, self.h_amax], norm_u)
                h_has_amax = True
                x, x2 = x2, x
            elif self.fuse:
                L("AddRMSNorm", [x, proj, gain, x2, self.h], norm_u)
                x, x2 = x2, x
            else:
                L("ElemAdd", [x, proj, x2])
                x, x2 = x2, x
                L("RMSNorm", [x, gain, self.h], norm_u)

        for li, lay in enumerate(self.model.layers):
            if li == 0:
                L("RMSNorm", [x, lay.g1, self.h], norm_u)
                h_has_amax = False
            else:
                add_norm(lay.g1, 1)              # the previous layer's second residual add

            def q_branch():
                self._linear(self.h, lay.wq, self.q)
                if not self.fuse:
                    L("RoPE", [self.pos_q, self.q], _u("<IIIf", B * self.hq, D, D, cfg.rope_base))

            def k_branch():
                self._linear(self.h, lay.wk, self.k)
                if self.fuse:
                    return
                L("RoPE", [self.pos_k, self.k], _u("<IIIf", B * self.hk, D, D, cfg.rope_base))
                krows = self.k
                if f16:
                    krows = self._k16
                    L("CastF32ToF16", [self.k, krows])
                L(scatter, [krows, self.slots, self.k_cache[li]], rp)

            def v_branch():
                self._linear(self.h, lay.wv, self.v)
                if self.fuse:
                    return
                vrows = self.v
                if f16:
                    vrows = self._v16
                    L("CastF32ToF16", [self.v, vrows])
                L(scatter, [vrows, self.slots, self.v_cache[li]], rp)

            if self.use_packed and self.fuse:
                # one product over q | k | v, each written to its own buffer
                w = lay.wqkv
                if h_has_amax:
                    L("QuantMatMulInt4PackedSplit3A", [self.h, self.h_amax, w.packed, self.q, self.k, self.v],
                      _u("<IIIIIIII", B, w.N, w.K, self.hq * D, self.hk * D, 0, 0, 0))
                else:
                    L("QuantMatMulInt4PackedSplit3", [self.h, w.packed, self.q, self.k, self.v],
                      _u("<IIIIIIII", B, w.N, w.K, self.hq * D, self.hk * D, 0, 0, 0))
            else:
                # q, k and v depend only on h: three branches that may run side by side
                self._parallel([q_branch, k_branch, v_branch])
            if self.fuse:
                L("RopeScatterQKVF16" if f16 else "RopeScatterQKV",
                  [self.pos_q, self.pos_k, self.slots, self.q, self.k, self.v, self.k_cache[li], self.v_cache[li]],
                  _u("<IIIIIIfI", B, self.hq, self.hk, D, D, self.capacity, cfg.rope_base, 0))
            attn_u = _u("<IIIIIIfI", B, self.hq, self.hk, D, cfg.block, self.max_pages, scale, 0)
            attn_b = [self.q, self.k_cache[li], self.v_cache[li], self.pages, self.lengths, self.attn]
            if maxima:
                # the kernel that writes a product's input also leaves its rows' largest magnitudes
                L("AttentionDecodeBatchedF16Max" if f16 else "AttentionDecodeBatchedMax", attn_b + [self.attn_max], attn_u)
                w = lay.wo_p
                L("QuantMatMulInt4PackedA", [self.attn, self.attn_max, w.packed, self._proj[0]],
                  _u("<IIII", B, w.N, w.K, self.attn_max.shape[1]))
            else:
                L("AttentionDecodeBatchedF16" if f16 else "AttentionDecodeBatched", attn_b, attn_u)
                self._linear(self.attn, lay.wo_p if self.use_packed else lay.wo, self._proj[0])
            add_norm(lay.g2, 0)
            act_has_max = False
            if self.use_packed and self.fuse:
                # gate and up as one product whose epilogue applies SwiGLU
                w = lay.wgu
                if h_has_amax and maxima:
                    L("QuantMatMulInt4PackedSwiGLUAMax", [self.h, self.h_amax, w.packed, self.act, self.act_max],
                      _u("<IIII", B, w.N, w.K, 0))
                    act_has_max = True
                elif h_has_amax:
                    L("QuantMatMulInt4PackedSwiGLUA", [self.h, self.h_amax, w.packed, self.act], _u("<IIII", B, w.N, w.K, 0))
                else:
                    L("QuantMatMulInt4PackedSwiGLU", [self.h, w.packed, self.act], _u("<IIII", B, w.N, w.K, 0))
            else:
                self._parallel([lambda: self._linear(self.h, lay.wg, self.gate),
                                lambda: self._linear(self.h, lay.wu, self.up)])
                L("SwiGLU", [self.gate, self.up, self.act])
            if act_has_max:
                w = lay.wd_p
                L("QuantMatMulInt4PackedA", [self.act, self.act_max, w.packed, self._proj[1]],
                  _u("<IIII", B, w.N, w.K, lay.wgu.N // 64))
            else:
                self._linear(self.act, lay.wd_p if self.use_packed else lay.wd, self._proj[1])
        add_norm(self.model.g_final, 1)
        if h_has_amax:
            w = self.model.lm_head_p
            L("QuantMatMulInt4PackedA", [self.h, self.h_amax, w.packed, self.logits_local], _u("<IIII", B, w.N, w.K, 0))
        else:
            self._linear(self.h, self.model.lm_head_p if self.use_packed else self.model.lm_head, self.logits_local)
        if self.shard.tp > 1:
            # each rank owns a column range of the vocabulary: it reduces its columns to one (largest
            # logit, index) pair per row, the ranks exchange the pairs (a sum over slots the others
            # left zero: 8 bytes per rank and row), and every rank merges them by SampleArgmax's rule
            tp, vr = self.shard.tp, self.shard.vocab
            L("ArgmaxShard", [self.logits_local, self._my_pairs],
              _u("<IIIIIIII", len(vr), B, tp, self.shard.rank, vr.start, 0, 0, 0))
            if self._peer is not None:
                self._peer.all_reduce_region(2, self.top_pairs)
                self._count += 1
            else:
                self.top_pairs.copy_(self._my_pairs)
                self._all_reduce(self.top_pairs)
            L("ArgmaxMerge", [self.top_pairs, self.next_tokens], _u("<IIII", B, tp, 0, 0))
        else:
            L("SampleArgmax", [self.logits, self.next_tokens], _u("<IIII", cfg.vocab, B, 0, 0))
        self.launches_per_step = self._count                      # dispatches by kernel name
        self.kernel_launches_per_step = count() - kernels0        # CUDA kernels they launched
        self._final_x = x

    def full_logits(self) -> torch.Tensor:
        """The last step's logits over the whole vocabulary [batch, vocab].  With the vocabulary
        split over ranks this is a collective (every rank calls it) outside the recorded step."""
        if self.shard.tp == 1:
            return self.logits_local
        import torch.distributed as dist
        # the shards are whole 128-column groups and may differ by one group: gather at the widest
        widths = [len(Shard.plan(self.cfg, self.shard.tp, r).vocab) for r in range(self.shard.tp)]
        wmax = max(widths)
        mine = torch.zeros((self.batch, wmax), dtype=torch.float32, device=self.dev)
        mine[:, :self.logits_local.shape[1]] = self.logits_local
        parts = [torch.empty_like(mine) for _ in range(self.shard.tp)]
        dist.all_gather(parts, mine, group=self.group)
        return torch.cat([parts[r][:, :widths[r]] for r in range(self.shard.tp)], dim=1)

    def prepare(self):
        if self.cfg.cache_dtype == torch.float16 and not hasattr(self, "_k16"):
            self._k16 = torch.zeros_like(self.k, dtype=torch.float16)
            self._v16 = torch.zeros_like(self.v, dtype=torch.float16)

    def capture(self, warmup: int = 2):
        """Runs the step eagerly (which also sizes the kernels' workspaces), then captures it."""
        self.prepare()
        s = torch.cuda.Stream(device=self.dev)
        s.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(s):
            for _ in range(warmup):
                self.record_step()
            s.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                self.record_step()
        torch.cuda.current_stream(self.dev).wait_stream(s)
        self.graph = g
        self._graph_stream = s

    def run_step(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self.prepare()
            self.record_step()

    # ------------------------------------------------------------------ the caller's loop
    def step(self, token_ids: np.ndarray) -> np.ndarray:
        """One end-to-end decode step as a caller makes it: host token ids in, host next-token ids
        out.  The per-step inputs are staged in pinned memory and copied to the device, the
        recorded step runs, and the argmax ids are read back."""
        packed = self.step_inputs_host(token_ids)
        if self._pin is None:
            self._pin = torch.empty(packed.size, dtype=I32).pin_memory()
            self._out_pin = torch.empty(self.batch, dtype=I32).pin_memory()
            self._err_pin = torch.zeros(1, dtype=I32).pin_memory()
        self._pin.numpy()[:] = packed
        self.inputs.copy_(self._pin, non_blocking=True)
        self.run_step()
        self._out_pin.copy_(self.next_tokens, non_blocking=True)
        if self._peer is not None:
            self._err_pin.copy_(self._peer.error_word, non_blocking=True)
        torch.cuda.current_stream(self.dev).synchronize()
        if self._peer is not None and int(self._err_pin[0]) != 0:
            # a bounded wait for a peer ran out: this step's sums are not the all-reduced ones.
            # The rank stops here; its peers' next all-reduce runs out the same way and they stop too.
            from . import _lib
            raise _lib.AccelError(_lib.AB_ERR_TIMEOUT,
                                  f"decode step: peer all-reduce call {int(self._err_pin[0])} gave up "
                                  "waiting for its peers; the sampled tokens of this step are invalid")
        self.lengths_host += 1
        return self._out_pin.numpy().copy()

    @property
    def h2d_bytes_per_step(self) -> int:
        return 4 * self.inputs.numel()

    @property
    def d2h_bytes_per_step(self) -> int:
        return 4 * self.batch

    def kv_bytes_read_per_step(self) -> int:
        """Algorithmic K/V bytes one step reads on this rank: every cached position of every
        sequence, K and V, once per KV head, in every layer."""
        e = 2 if self.cfg.cache_dtype == torch.float16 else 4
        return int(self.cfg.layers * 2 * self.hk * self.cfg.head_dim * e * (self.lengths_host + 1).sum())


class SeamStep:
    """The recorded decode step driven through the driver seam, as the reference's device layer drives
    a backend (internal/driver/plan.go:360-400): the step is recorded once as a plan - a host-write node
    for the per-step inputs, one dispatch node per kernel, a copy of the sampled ids into a
    host-visible block - compiled with ab_compile, and every step is set_payload + ab_exec_submit +
    ab_fence_wait + a read of the host-visible block.  The weights, caches and activations are the
    engine's own tensors, imported as blocks (the engine keeps them alive).  One GPU: the peer
    all-reduce of a sharded step is not a registered kernel."""

    def __init__(self, engine: "DecodeEngine", use_graphs: bool = True, max_in_flight: int = 0):
        from . import driver as drv
        if engine.shard.tp != 1:
            raise ValueError("SeamStep records the unsharded step")
        self.engine, self.drv = engine, drv
        self.dev = drv.Device(engine.dev.index or 0, use_graphs=use_graphs)
        self._blocks: dict = {}
        nodes: list = []

        def operand(t: torch.Tensor):
            key = (t.data_ptr(), t.numel() * t.element_size())
            blk = self._blocks.get(key)
            if blk is None:
                blk = self.dev.import_ptr(*key)
                self._blocks[key] = blk
            return drv.Operand(block=blk, offset=0, size=key[1])

        class Recorder:
            @staticmethod
            def launch(name, bindings, uniform=None):
                nodes.append(drv.Dispatch(name, [operand(t) for t in bindings], uniform))

            @staticmethod
            def launch_count():
                return 0

        engine.prepare()
        n_in = engine.inputs.numel() * 4
        nodes.append(drv.HostWrite(operand(engine.inputs), bytes(n_in)))
        ops, engine.ops = engine.ops, Recorder
        try:
            engine.record_step()
        finally:
            engine.ops = ops
        self.ids = self.dev.alloc(max(engine.batch * 4, 256), drv.MEMORY_HOST_VISIBLE, "sampled ids")
        nodes.append(drv.Copy(operand(engine.next_tokens), drv.Operand(block=self.ids, offset=0, size=engine.batch * 4)))
        self.nodes = len(nodes)
        self.exe = self.dev.compile(nodes, max_in_flight=max_in_flight)
        self._out = np.zeros(engine.batch, np.int32)

    def step(self, token_ids: np.ndarray) -> np.ndarray:
        """Host token ids in, host next-token ids out, through the compiled plan."""
        e = self.engine
        self.exe.set_payload(0, e.step_inputs_host(token_ids).astype(np.int32).tobytes())
        f = self.exe.submit()
        f.wait()
        f.free()
        e.lengths_host += 1
        return self.ids.read(0, self._out).copy()

    def close(self):
        self.exe.close()
        self.ids.free()
        for b in self._blocks.values():
            b.free()
        self._blocks = {}
        self.dev.close()

