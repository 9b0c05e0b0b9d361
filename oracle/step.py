"""One layer of the 7B-shape decode step on the CPU oracle: the bounded sample the benchmark times
as the CPU baseline.  TEST INFRASTRUCTURE ONLY (see accel_oracle.c); the product never imports it.

The layer is config 4's: batch 16 rows of activations, d_model 4096, 32 heads of 128, SwiGLU FFN
11008, RMSNorm, RoPE, an f32 paged KV cache (block 16) holding `context` positions per sequence,
every linear int4 with the reference's packing.  Weights and cache contents are seeded synthetic
values; the time does not depend on them."""
from __future__ import annotations

import time

import numpy as np

import oracle as orc


class LayerSample:
    def __init__(self, batch=16, d=4096, heads=32, kv_heads=32, head_dim=128, ffn=11008,
                 vocab=32000, context=2048, block=16, seed=1, with_head=True):
        self.B, self.d, self.H, self.KH, self.D, self.F, self.V = batch, d, heads, kv_heads, head_dim, ffn, vocab
        self.block, self.context = block, context
        rng = np.random.default_rng(seed)

        def qmat(k, n):
            w = rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.02)
            return orc.int4_quantize(w)

        self.wq, self.wk, self.wv = qmat(d, heads * head_dim), qmat(d, kv_heads * head_dim), qmat(d, kv_heads * head_dim)
        self.wo = qmat(heads * head_dim, d)
        self.wg, self.wu, self.wd = qmat(d, ffn), qmat(d, ffn), qmat(ffn, d)
        self.head = qmat(d, vocab) if with_head else None
        self.g1 = np.ones(d, np.float32)
        self.g2 = np.ones(d, np.float32)
        pages_per_seq = (context + 1 + block - 1) // block
        self.max_pages = pages_per_seq
        perm = rng.permutation(batch * pages_per_seq).astype(np.uint32)
        self.pages = perm.reshape(batch, pages_per_seq)
        cap = batch * pages_per_seq * block
        self.kc = rng.standard_normal((cap, kv_heads, head_dim), dtype=np.float32)
        self.vc = rng.standard_normal((cap, kv_heads, head_dim), dtype=np.float32)
        self.x = rng.standard_normal((batch, d), dtype=np.float32)
        self.lengths = np.full(batch, context + 1, np.uint32)
        pos = context
        self.slots = (self.pages[:, pos // block] * block + pos % block).astype(np.uint32)
        self.pos_q = np.full(batch * heads, pos, np.uint32)
        self.pos_k = np.full(batch * kv_heads, pos, np.uint32)

    def layer(self):
        B, d, H, KH, D, F = self.B, self.d, self.H, self.KH, self.D, self.F
        mm = lambda a, w, n, k: orc.quant_matmul_int4(a, *w, B, n, k)
        h = orc.rmsnorm(self.x, self.g1, 1e-5)
        q, k, v = mm(h, self.wq, H * D, d), mm(h, self.wk, KH * D, d), mm(h, self.wv, KH * D, d)
        q = orc.rope(q.reshape(B * H, D), self.pos_q, D, 10000.0)
        k = orc.rope(k.reshape(B * KH, D), self.pos_k, D, 10000.0)
        orc.scatter_rows(k.reshape(B, KH * D), self.slots, self.kc.reshape(-1, KH * D))
        orc.scatter_rows(v.reshape(B, KH * D), self.slots, self.vc.reshape(-1, KH * D))
        scale = float(np.float32(1) / np.float32(np.sqrt(D)))
        a = orc.attention_decode_batched(q, self.kc, self.vc, self.pages, self.lengths, B, H, KH, D,
                                         self.block, self.max_pages, scale)
        x = orc.elem_add(self.x, mm(a.reshape(B, H * D), self.wo, d, H * D))
        h = orc.rmsnorm(x, self.g2, 1e-5)
        act = orc.swiglu(mm(h, self.wg, F, d), mm(h, self.wu, F, d))
        return orc.elem_add(x, mm(act, self.wd, d, F))

    def head_and_argmax(self, x):
        h = orc.rmsnorm(x, self.g1, 1e-5)
        return orc.sample_argmax(orc.quant_matmul_int4(h, *self.head, self.B, self.V, self.d))

    def time_layer(self, repeats=1):
        best = float("inf")
        out = None
        for _ in range(repeats):
            t0 = time.perf_counter()
            out = self.layer()
            best = min(best, time.perf_counter() - t0)
        return best, out

    def time_head(self, x):
        t0 = time.perf_counter()
        self.head_and_argmax(x)
        return time.perf_counter() - t0
