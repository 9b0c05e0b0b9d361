"""Causal prefill attention of one sequence (AttentionPrefill / AttentionPrefillPaged and their
f16-cache forms; internal/kernels/prefill.go:197,409, pagedprefillf16.go:31) on a B200 against the
oracle, through tensor.Attention's prefill branch.  Tolerance 2e-3 relative, as for every attention."""
import numpy as np
import pytest
import torch

import oracle as orc
from accel_b200 import tensor as T
from util import ATTN_TOL, assert_close, attn_scale, normal

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def u32(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.uint32).view(np.int32)).to(DEV)


@pytest.mark.parametrize("qH,kvH,D,block,q_seq,base,f16", [
    (4, 2, 16, 8, 300, 0, False),        # the reference's own fixture shape (prefill_test.go:1120)
    (8, 8, 128, 16, 64, 0, False),
    (8, 2, 64, 16, 130, 37, False),      # a prefill that extends a cache of 37 positions; GQA
    (8, 2, 64, 16, 130, 37, True),
    (32, 8, 128, 16, 40, 500, True),
    (32, 8, 128, 16, 70, 300, False),    # grouped heads of dimension 128: the tensor-core kernel, f32 cache
    (4, 2, 128, 8, 33, 90, False),       # two heads per KV head
])
def test_paged_prefill_matches_the_oracle(qH, kvH, D, block, q_seq, base, f16):
    rng = np.random.default_rng(q_seq + base)
    kv_len = base + q_seq
    n_pages = (kv_len + block - 1) // block
    pool = n_pages + 5
    q = normal(1, (q_seq, qH, D))
    dt = np.float16 if f16 else np.float32
    k = rng.standard_normal((pool * block, kvH, D)).astype(dt)
    v = rng.standard_normal((pool * block, kvH, D)).astype(dt)
    pages = rng.permutation(pool)[:n_pages].astype(np.uint32)
    lengths = np.array([kv_len], np.uint32)
    scale = attn_scale(D)
    ko, vo = (k.view(np.uint16), v.view(np.uint16)) if f16 else (k, v)     # the oracle takes f16 as bit patterns
    want = orc.attention_prefill_paged(q, ko, vo, pages, lengths, qH, kvH, D, q_seq, base, block, scale)
    got = T.attention(torch.from_numpy(q).to(DEV), torch.from_numpy(k).to(DEV), torch.from_numpy(v).to(DEV),
                      T.AttentionOptions(lengths=u32(lengths), pages=u32(pages), block=block, scale=scale, base=base))
    assert_close(got.cpu().numpy().ravel(), want, ATTN_TOL, "paged prefill")


def test_contiguous_prefill_and_a_length_shorter_than_the_mask():
    qH, kvH, D, q_seq, base = 4, 4, 32, 50, 10
    q = normal(2, (q_seq, qH, D))
    k, v = normal(3, (80, kvH, D)), normal(4, (80, kvH, D))
    scale = attn_scale(D)
    for kv_len in (base + q_seq, 25):                 # 25: rows past position 24 see only the first 25
        lengths = np.array([kv_len], np.uint32)
        want = orc.attention_prefill(q, k, v, lengths, qH, kvH, D, q_seq, base, scale)
        got = T.attention(torch.from_numpy(q).to(DEV), torch.from_numpy(k).to(DEV), torch.from_numpy(v).to(DEV),
                          T.AttentionOptions(lengths=u32(lengths), scale=scale, base=base))
        assert_close(got.cpu().numpy().ravel(), want, ATTN_TOL, f"contiguous prefill, length {kv_len}")


def test_prefill_then_decode_sees_what_the_prefill_saw():
    """The last row of a prefill is the decode step at that position: the two kernels agree."""
    qH, kvH, D, block, n = 8, 2, 64, 16, 77
    rng = np.random.default_rng(5)
    n_pages = (n + block - 1) // block
    q = normal(6, (n, qH, D))
    k = rng.standard_normal(((n_pages + 2) * block, kvH, D)).astype(np.float32)
    v = rng.standard_normal(((n_pages + 2) * block, kvH, D)).astype(np.float32)
    pages = rng.permutation(n_pages + 2)[:n_pages].astype(np.uint32)
    scale = attn_scale(D)
    kd, vd = torch.from_numpy(k).to(DEV), torch.from_numpy(v).to(DEV)
    pre = T.attention(torch.from_numpy(q).to(DEV), kd, vd,
                      T.AttentionOptions(lengths=u32([n]), pages=u32(pages), block=block, scale=scale, base=0))
    one = T.attention(torch.from_numpy(q[-1]).to(DEV), kd, vd,
                      T.AttentionOptions(lengths=u32([n]), pages=u32(pages), block=block, scale=scale))
    assert torch.equal(pre[-1], one)


def test_a_prefill_without_its_base_is_refused():
    q = torch.zeros(4, 2, 8, device=DEV)
    kv = torch.zeros(16, 2, 8, device=DEV)
    with pytest.raises(T.Refused, match="BaseName"):
        T.attention(q, kv, kv, T.AttentionOptions(lengths=u32([4]), scale=1.0))
