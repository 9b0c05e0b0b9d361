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


def gpu_step_of(sample: "LayerSample", device="cuda:0"):
    """The same layer + lm_head + argmax run by the product on a GPU, from this sample's weights,
    cache contents, page table and activations: the thing the oracle checks.  Returns the hidden
    state after the layer [B, d], the logits [B, V] and the sampled ids [B] as numpy arrays."""
    import torch

    from accel_b200 import decode as dec
    s = sample
    cfg = dec.ModelConfig(layers=1, d_model=s.d, n_heads=s.H, n_kv_heads=s.KH, head_dim=s.D, ffn=s.F,
                          vocab=s.V, eps=1e-5, rope_base=10000.0, block=s.block,
                          cache_dtype=torch.float32)
    emb = np.zeros((s.V, s.d), np.float32)
    emb[:s.B] = s.x                                  # token i of the batch embeds to row i of x
    layer = {"g1": s.g1, "g2": s.g2, "wq": s.wq, "wk": s.wk, "wv": s.wv, "wo": s.wo, "wg": s.wg,
             "wu": s.wu, "wd": s.wd}
    model = dec.DecodeModel.from_host(cfg, device, [layer], s.g1, s.head, emb)
    eng = dec.DecodeEngine(model, s.B, max_context=s.max_pages * s.block)
    assert eng.max_pages == s.max_pages and eng.capacity == s.kc.shape[0]
    eng.k_cache[0].copy_(torch.from_numpy(s.kc))
    eng.v_cache[0].copy_(torch.from_numpy(s.vc))
    eng.page_rows = [list(map(int, row)) for row in s.pages]
    eng.upload_pages()
    eng.lengths_host[:] = s.context
    eng.set_inputs(np.arange(s.B))
    eng.prepare()
    eng.record_step()
    torch.cuda.synchronize()
    return (eng._final_x.cpu().numpy(), eng.full_logits().cpu().numpy(),
            eng.next_tokens.cpu().numpy().astype(np.int64))


def layer_parity(sample: "LayerSample", device="cuda:0") -> dict:
    """Runs the sample's layer + head on the CPU oracle and on the GPU and compares them: the
    hidden state's error relative to its largest magnitude, and whether the greedy ids agree on
    every row whose two best oracle logits are clearly apart.  The oracle leg mutates the sample's
    cache (it appends this step's K/V), so the GPU leg runs first on the pristine cache."""
    hidden, logits, ids = gpu_step_of(sample, device)
    want = sample.layer()
    h = orc.rmsnorm(want, sample.g1, 1e-5)
    want_logits = orc.quant_matmul_int4(h, *sample.head, sample.B, sample.V, sample.d)
    want_ids = orc.sample_argmax(want_logits).astype(np.int64)
    scale = float(np.max(np.abs(want)))
    top2 = np.sort(want_logits, axis=1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 2e-3 * float(np.max(np.abs(want_logits)))
    return {
        "hidden_rel_err": float(np.max(np.abs(hidden.astype(np.float64) - want)) / scale),
        "logits_rel_err": float(np.max(np.abs(logits.astype(np.float64) - want_logits))
                                / float(np.max(np.abs(want_logits)))),
        "rows_with_clear_argmax": int(clear.sum()), "rows": int(sample.B),
        "ids_equal_on_clear_rows": bool(np.array_equal(ids[clear], want_ids[clear])),
    }
