"""Seeded synthetic inputs and the tolerance rules the parity tests share."""
import math

import numpy as np

GEMM_TOL = 1e-3     # int4 GEMV / GEMM, relative, f32 accumulate
ATTN_TOL = 2e-3     # attention, relative


def normal(seed, shape, std=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * std).astype(np.float32)


def rel_err(got, want):
    """max |got - want| / max |want|: the error relative to the output's scale."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    denom = max(float(np.max(np.abs(want))), 1e-30)
    return float(np.max(np.abs(got - want))) / denom


def assert_close(got, want, tol, what=""):
    got = np.asarray(got)
    want = np.asarray(want)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert not np.any(np.isnan(got) != np.isnan(want)), f"{what}: NaN pattern differs"
    mask = ~np.isnan(want)
    e = rel_err(got[mask], want[mask]) if mask.any() else 0.0
    assert e <= tol, f"{what}: relative error {e:.3e} exceeds {tol:.1e}"
    return e


def paged_fixture(seed, batch, kv_heads, head_dim, block, lengths, max_pages=None, extra_blocks=3,
                  f16=False):
    """A shared pool, per-sequence disjoint page rows cut from one seeded permutation of it and
    padded with zeros, and K/V ~ N(0,1)."""
    rng = np.random.default_rng(seed)
    need = [(int(n) + block - 1) // block for n in lengths]
    if max_pages is None:
        max_pages = max(max(need), 1)
    pool_blocks = sum(need) + extra_blocks
    perm = rng.permutation(pool_blocks).astype(np.uint32)
    pages = np.zeros((batch, max_pages), np.uint32)
    at = 0
    for s in range(batch):
        pages[s, :need[s]] = perm[at:at + need[s]]
        at += need[s]
    cap = pool_blocks * block
    k = rng.standard_normal((cap, kv_heads, head_dim)).astype(np.float32)
    v = rng.standard_normal((cap, kv_heads, head_dim)).astype(np.float32)
    if f16:
        k = k.astype(np.float16)
        v = v.astype(np.float16)
    return k, v, pages, max_pages


def attn_scale(d):
    return float(np.float32(1) / np.float32(math.sqrt(d)))
