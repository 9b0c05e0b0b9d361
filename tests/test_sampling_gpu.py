"""The on-device sampling policy (Softmax, ScaleRows, TopKMaskRows, TopPMaskRows, SampleRows,
LogitBias, the penalty kernels and their uniform single-row forms) on a B200 against the oracle.
Masks, counts and sampled ids are index work: bit-exact.  Softmax is f32 arithmetic in the
reference's order of sums: compared bit for bit as well."""
import numpy as np
import pytest
import torch

import oracle as orc
from accel_b200 import runtime as rt
from accel_b200 import tensor as T

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint32:
        a = a.view(np.int32)
    return torch.from_numpy(a).to(DEV)


def host(t):
    a = t.cpu().numpy()
    return a.view(np.uint32) if a.dtype == np.int32 else a


@pytest.mark.parametrize("rows,vocab", [(16, 32000), (3, 1000), (1, 5), (4, 129)])
def test_softmax_and_the_masks_are_bit_identical_to_the_oracle(rows, vocab):
    rng = np.random.default_rng(vocab)
    logits = (rng.standard_normal((rows, vocab)) * 4).astype(np.float32)
    logits[0, : min(vocab, 7)] = logits[0, 0]                    # ties at the top
    want = orc.softmax(logits)
    got = T.softmax(dev(logits))
    assert np.array_equal(host(got), want)
    ks = rng.integers(0, 60, rows).astype(np.uint32)
    ks[0] = 0
    ps = rng.uniform(0.05, 0.95, rows).astype(np.float32)
    ps[-1] = 1.0
    d = rt.row_sample_dims(vocab, rows)
    out = torch.empty_like(got)
    rt.launch("TopKMaskRows", [got, dev(ks), out], d)
    want_k = orc.topk_mask(want, ks)
    assert np.array_equal(host(out), want_k)
    out2 = torch.empty_like(got)
    rt.launch("TopPMaskRows", [out, dev(ps), out2], d)
    assert np.array_equal(host(out2), orc.topp_mask(want_k, ps))
    # the uniform forms: one k, one p for every row
    rt.launch("TopKMask", [got, out], rt.top_dims(vocab, k=5))
    assert np.array_equal(host(out), orc.topk_mask(want, 5))
    rt.launch("TopPMask", [got, out], rt.top_dims(vocab, p=0.5))
    assert np.array_equal(host(out), orc.topp_mask(want, 0.5))


def test_reference_known_answers_on_the_device():
    # internal/kernels/sample_test.go:105-150, topk_test.go:67-105,152-180
    probs = np.array([[0.1, 0.2, 0.3, 0.4]], np.float32)
    out = torch.empty(1, dtype=torch.int32, device=DEV)
    for draw, want in [(0, 0), (0.05, 0), (0.1, 1), (0.3, 2), (0.6, 3), (0.999999, 3), (-0.5, 0), (1.5, 3), (1.0, 3)]:
        rt.launch("SampleCategorical", [dev(probs), dev(np.array([draw], np.float32)), out], rt.sample_dims(4, 1))
        assert int(out[0]) == want, draw
    for w, k, want in [([0.1, 0.5, 0.2, 0.4, 0.3], 2, [1, 3]), ([5, 5, 5, 5, 1], 2, [0, 1]), ([2, 2, 2, 2], 3, [0, 1, 2])]:
        o = torch.empty(len(w), device=DEV)
        rt.launch("TopKMask", [dev(np.array(w, np.float32)), o], rt.top_dims(len(w), k=k))
        assert [i for i, v in enumerate(host(o)) if v != 0] == want
    w = np.array([0.1, 0.2, 0.3, 0.4], np.float32)
    for p, want in [(0.3, [3]), (0.5, [2, 3]), (0.7, [2, 3]), (0.9, [1, 2, 3]), (1.0, [0, 1, 2, 3])]:
        o = torch.empty(4, device=DEV)
        rt.launch("TopPMask", [dev(w), o], rt.top_dims(4, p=p))
        assert [i for i, v in enumerate(host(o)) if v != 0] == want, p


@pytest.mark.parametrize("masked", [True, False])
def test_the_whole_policy_gives_the_oracle_s_tokens(masked):
    rows, vocab, cap = 16, 32000, 64
    rng = np.random.default_rng(7 + masked)
    logits = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    factor = (1.0 / rng.uniform(0.5, 1.5, rows)).astype(np.float32)
    factor[3] = 0.0                                                  # a greedy row beside stochastic ones
    draws = rng.random(rows).astype(np.float32)
    ks = rng.integers(1, 100, rows).astype(np.uint32) if masked else None
    ps = rng.uniform(0.3, 0.99, rows).astype(np.float32) if masked else None
    ids = rng.integers(0, vocab + 50, (rows, 4)).astype(np.uint32)   # ids past the vocabulary are empty slots
    vals = rng.standard_normal((rows, 4)).astype(np.float32)
    history = rng.integers(0, vocab + 10, (rows, cap)).astype(np.uint32)
    history[:, :8] = history[:, 8:9]                                 # repeats: what a frequency penalty counts
    filled = rng.integers(0, cap + 1, rows).astype(np.uint32)
    rep = rng.choice([0.0, 1.0, 1.3], rows).astype(np.float32)
    pres = rng.uniform(0, 0.5, rows).astype(np.float32)
    freq = rng.uniform(0, 0.2, rows).astype(np.float32)

    x = orc.logit_bias(logits, ids, vals)
    x, want_counts = orc.penalty_rows(x, history, filled, rep, pres, freq)
    x = orc.softmax(orc.scale_rows(x, factor))
    if masked:
        x = orc.topp_mask(orc.topk_mask(x, ks), ps)
    want = orc.sample_rows(x, draws, factor)

    counts = torch.full((rows, vocab), 77, dtype=torch.int32, device=DEV)   # left over from "the step before"
    pen = T.RowPenalties(dev(history), counts, dev(filled), dev(rep), dev(pres), dev(freq))
    got = T.sample_rows(dev(logits), dev(draws),
                        T.RowSampling(factor=dev(factor), top_k=dev(ks) if masked else None,
                                      top_p=dev(ps) if masked else None, bias=(dev(ids), dev(vals)), penalties=pen))
    assert np.array_equal(host(counts), want_counts)
    assert np.array_equal(host(got), want)
    assert int(got[3]) == int(np.argmax(x[3]))


def test_uniform_penalty_kernels():
    # internal/kernels/penalty_test.go:88-135: frequency scales with the count, presence does not;
    # only the filled part of the ring counts; an id past the vocabulary is dropped
    for logits, hist, count, r, p, f in [([0, 0, 0], [0, 1, 1, 2, 2, 2, 0, 0], 6, 0.0, 1.0, 0.5),
                                         ([0, 0, 0, 0], [1, 2, 3, 0, 0, 0, 0, 0], 3, 0.0, 1.0, 0.0),
                                         ([0, 0, 0, 0], [9, 4, 1, 4], 4, 0.0, 1.0, 0.0),
                                         ([2.0, -2.0], [0, 1], 2, 2.0, 0.0, 0.0)]:
        lg = np.array(logits, np.float32)
        h = np.array(hist, np.uint32)
        d = rt.penalty_dims(lg.size, h.size, count, r, p, f)
        counts = torch.full((lg.size,), 5, dtype=torch.int32, device=DEV)
        out = torch.empty(lg.size, device=DEV)
        rt.launch("PenaltyClear", [counts], d)
        rt.launch("PenaltyCount", [dev(h), counts], d)
        rt.launch("PenaltyApply", [dev(lg), counts, out], d)
        want, want_counts = orc.penalty_rows(lg, h, count, r, p, f)
        assert np.array_equal(host(counts), want_counts[0]) and np.array_equal(host(out), want[0])


def test_refusals():
    lg = torch.zeros(2, 8, device=DEV)
    with pytest.raises(T.Refused, match="Factor is nil"):
        T.sample_rows(lg, torch.zeros(2, device=DEV), T.RowSampling())
    with pytest.raises(T.Refused, match="exactly one per row"):
        T.sample_rows(lg, torch.zeros(2, device=DEV), T.RowSampling(factor=torch.zeros(3, device=DEV)))
