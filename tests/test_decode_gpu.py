"""The full decode step (config 4's wiring at a small shape) on a B200 against the same step run
on the CPU oracle: identical weights, identical cache contents, greedy tokens equal and logits
within the int4-product tolerance compounded over the layers."""
import numpy as np
import pytest
import torch

import oracle_ops
from accel_b200 import decode as dec
from util import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def small_cfg(cache_dtype=torch.float32):
    return dec.ModelConfig(layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512,
                           vocab=1024, block=16, cache_dtype=cache_dtype)


def clone_model_to_cpu(m: dec.DecodeModel) -> dec.DecodeModel:
    c = object.__new__(dec.DecodeModel)
    c.cfg, c.shard, c.device = m.cfg, m.shard, torch.device("cpu")
    cp = lambda w: dec.Int4Matrix(w.codes.cpu(), w.scales.cpu(), w.zeros.cpu(), w.K, w.N)
    c.layers = []
    for L in m.layers:
        n = dec.Layer()
        n.g1, n.g2 = L.g1.cpu(), L.g2.cpu()
        for k in ("wq", "wk", "wv", "wo", "wg", "wu", "wd"):
            setattr(n, k, cp(getattr(L, k)))
        c.layers.append(n)
    c.g_final, c.lm_head, c.embedding = m.g_final.cpu(), cp(m.lm_head), m.embedding.cpu()
    return c


@pytest.mark.parametrize("cache_dtype", [torch.float32, torch.float16])
def test_decode_steps_match_the_oracle(cache_dtype):
    cfg = small_cfg(cache_dtype)
    shard = dec.Shard.plan(cfg, 1, 0)
    model = dec.DecodeModel(cfg, shard, DEV, seed=3, std=0.08)
    batch, steps = 3, 40
    gpu = dec.DecodeEngine(model, batch, max_context=64)
    cpu = dec.DecodeEngine(clone_model_to_cpu(model), batch, max_context=64, ops=oracle_ops)
    for e in (gpu, cpu):
        for s in range(batch):
            e.reserve(s, steps + 1)
        e.upload_pages()
        e.prepare()
    assert gpu.page_rows == cpu.page_rows
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, cfg.vocab, (12, batch))
    tok = prompt[0]
    for t in range(steps):
        for e in (gpu, cpu):
            e.set_inputs(tok)
            e.run_step()
            e.lengths_host += 1
        g_logits, c_logits = gpu.full_logits().cpu().numpy(), cpu.full_logits().numpy()
        assert_close(g_logits, c_logits, 5e-3, f"logits at step {t}")
        g_next = gpu.next_tokens.cpu().numpy()
        c_next = cpu.next_tokens.numpy()
        # greedy tokens agree wherever the oracle's top two logits are not within the tolerance
        top2 = np.sort(c_logits, axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 1e-2 * np.abs(c_logits).max()
        assert np.array_equal(g_next[clear], c_next[clear]), t
        tok = prompt[t + 1] if t + 1 < len(prompt) else c_next      # teacher-forced, then greedy
    # the caches the two engines built are the same rows in the same slots
    for li in range(cfg.layers):
        assert_close(gpu.k_cache[li].float().cpu().numpy(), cpu.k_cache[li].float().numpy(), 5e-3, "K cache")


def test_graph_replay_and_device_advance_equal_the_host_loop():
    cfg = small_cfg()
    shard = dec.Shard.plan(cfg, 1, 0)
    model = dec.DecodeModel(cfg, shard, DEV, seed=5, std=0.08)
    batch, steps = 4, 20
    a = dec.DecodeEngine(model, batch, max_context=64)      # host loop: step()
    b = dec.DecodeEngine(model, batch, max_context=64)      # captured graph + device-side advance
    for e in (a, b):
        e.fill_context(17, seed=2)
        for s in range(batch):
            e.reserve(s, 17 + steps + 1)
        e.upload_pages()
    first = np.arange(batch) + 5
    b.set_inputs(first)
    b.capture(warmup=1)
    # the warm-up and capture runs appended their K/V at position 17 only, which the replay
    # rewrites with the same values; lengths are untouched
    out_a, out_b = [], []
    tok = first
    for t in range(steps):
        tok = a.step(tok)
        out_a.append(tok.copy())
    b.set_inputs(first)
    for t in range(steps):
        b.run_step()
        out_b.append(b.next_tokens.cpu().numpy().copy())
        b.advance_on_device()
    assert np.array_equal(np.array(out_a), np.array(out_b))
    assert a.launches_per_step == b.launches_per_step > 0


@pytest.mark.parametrize("cache", ["f32", "f16"])
def test_fused_support_kernels_equal_the_chain_of_reference_operators(cache):
    """AddRMSNorm and RopeScatterQKV against ElemAdd, RMSNorm, RoPE, (CastF32ToF16,) ScatterRows:
    the same step recorded both ways gives the same bits: tokens, logits and caches."""
    cfg = small_cfg(torch.float16 if cache == "f16" else torch.float32)
    shard = dec.Shard.plan(cfg, 1, 0)
    model = dec.DecodeModel(cfg, shard, DEV, seed=9, std=0.08)
    batch, steps = 3, 6
    # both on the reference-layout planes, so that the products are the same kernels in both
    fused = dec.DecodeEngine(model, batch, max_context=64, use_packed=False)
    chain = dec.DecodeEngine(model, batch, max_context=64, use_packed=False)
    assert fused.fuse
    chain.fuse = False
    for e in (fused, chain):
        e.fill_context(9, seed=4)
        for s in range(batch):
            e.reserve(s, 9 + steps + 1)
        e.upload_pages()
    tok_f = tok_c = np.arange(batch) + 3
    for t in range(steps):
        tok_f = fused.step(tok_f)
        tok_c = chain.step(tok_c)
        assert np.array_equal(tok_f, tok_c), t
        assert torch.equal(fused.full_logits(), chain.full_logits()), t
    assert fused.launches_per_step < chain.launches_per_step
    for li in range(cfg.layers):
        assert torch.equal(fused.k_cache[li], chain.k_cache[li])
        assert torch.equal(fused.v_cache[li], chain.v_cache[li])


def test_prepacked_products_give_the_step_of_the_reference_planes():
    """The same model stepped twice: on quant.Int4Quantize's planes (one product per matrix, SwiGLU as
    its own kernel) and on the load-time prepack (q | k | v as one product, gate | up as one product
    with SwiGLU in its epilogue).  Different kernels, same mathematics: logits within the int4
    tolerance compounded over the layers, greedy ids equal where the top two are clearly apart."""
    cfg = small_cfg()
    model = dec.DecodeModel(cfg, dec.Shard.plan(cfg, 1, 0), DEV, seed=21, std=0.08)
    assert model.packed
    batch, steps = 5, 8
    planes = dec.DecodeEngine(model, batch, max_context=64, use_packed=False)
    packed = dec.DecodeEngine(model, batch, max_context=64)
    assert packed.use_packed and not planes.use_packed
    for e in (planes, packed):
        e.fill_context(9, seed=4)
        for s in range(batch):
            e.reserve(s, 9 + steps + 1)
        e.upload_pages()
    tok = np.arange(batch) + 3
    for t in range(steps):
        a = planes.step(tok)
        b = packed.step(tok)
        la, lb = planes.full_logits().cpu().numpy(), packed.full_logits().cpu().numpy()
        assert_close(lb, la, 3e-3, f"logits at step {t}")
        top2 = np.sort(la, axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 1e-2 * np.abs(la).max()
        assert np.array_equal(a[clear], b[clear]), t
        tok = a
    assert packed.launches_per_step < planes.launches_per_step


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_tensor_parallel_step_on_the_gpus_matches_one_gpu():
    """Both collectives (NCCL; the peer all-reduce that also adds the residual and normalises),
    eager and from a replayed graph, against the unsharded step (child processes under torchrun)."""
    import os
    import subprocess
    import sys
    n = 4 if torch.cuda.device_count() >= 4 else 2
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                          "--master-addr", "127.0.0.1", "--master-port", "29617", os.path.join(here, "tp_check.py")],
                         env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, (out.stdout[-1500:], out.stderr[-3000:])
    assert "OK world=" in out.stdout


@pytest.mark.parametrize("graphs", [False, True])
def test_the_step_through_the_driver_seam_equals_the_direct_step(graphs):
    """The same step recorded as a plan and driven with ab_compile / set_payload / ab_exec_submit /
    ab_fence_wait (what the reference's device layer does with a backend) against the engine's own
    loop: same kernels, same order, so the sampled ids and the logits are equal bit for bit."""
    cfg = small_cfg()
    batch, steps = 3, 6
    engines = []
    for _ in range(2):
        model = dec.DecodeModel(cfg, dec.Shard.plan(cfg, 1, 0), DEV, seed=3, std=0.08)
        e = dec.DecodeEngine(model, batch, max_context=64)
        e.fill_context(9, seed=4)
        for s in range(batch):
            e.reserve(s, 9 + steps + 1)
        e.upload_pages()
        engines.append(e)
    direct, other = engines
    seam = dec.SeamStep(other, use_graphs=graphs)
    tok_a = tok_b = np.arange(batch) + 5
    for t in range(steps):
        tok_a = direct.step(tok_a)
        tok_b = seam.step(tok_b)
        assert np.array_equal(tok_a, tok_b), t
        assert torch.equal(direct.full_logits(), other.full_logits()), t
    assert seam.nodes > 10
    seam.close()


@pytest.mark.parametrize("cache_dtype", [torch.float32, torch.float16])
def test_prefill_leaves_the_cache_a_token_by_token_decode_leaves(cache_dtype):
    """DecodeEngine.prefill (batch kernels over batch x chunk rows, the paged causal prefill
    attention) against feeding the same prompt one token at a time through the decode step: the
    K/V the two leave in the pages agree, and so does the step that follows."""
    cfg = small_cfg(cache_dtype)
    batch, T = 3, 23
    rng = np.random.default_rng(2)
    prompt = rng.integers(0, cfg.vocab, (batch, T))
    engines = []
    for _ in range(2):
        model = dec.DecodeModel(cfg, dec.Shard.plan(cfg, 1, 0), DEV, seed=3, std=0.08)
        engines.append(dec.DecodeEngine(model, batch, max_context=72))     # 5 pages per row: rows of the table are not 16-byte aligned
    stepwise, bulk = engines
    for s in range(batch):
        stepwise.reserve(s, T + 2)
    stepwise.upload_pages()
    for t in range(T):
        stepwise.step(prompt[:, t])
    secs = bulk.prefill(prompt, chunk=5)                 # 4 chunks of 5 and one of 3
    assert secs > 0 and np.array_equal(bulk.lengths_host, stepwise.lengths_host)
    assert bulk.page_rows[0][:2] == stepwise.page_rows[0][:2]
    for li in range(cfg.layers):
        for a, b in ((stepwise.k_cache[li], bulk.k_cache[li]), (stepwise.v_cache[li], bulk.v_cache[li])):
            assert_close(b.float().cpu().numpy(), a.float().cpu().numpy(), 5e-3, f"layer {li} cache")
    for s in range(batch):
        bulk.reserve(s, T + 2)
    bulk.upload_pages()
    nxt = rng.integers(0, cfg.vocab, batch)
    ta, tb = stepwise.step(nxt), bulk.step(nxt)
    assert_close(bulk.full_logits().cpu().numpy(), stepwise.full_logits().cpu().numpy(), 5e-3, "the step after")
    la = stepwise.full_logits().cpu().numpy()
    top2 = np.sort(la, axis=1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 1e-2 * np.abs(la).max()
    assert np.array_equal(ta[clear], tb[clear])
