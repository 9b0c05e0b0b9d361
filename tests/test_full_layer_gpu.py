"""Parity at the configuration that is benchmarked: ONE full-size layer of the 7B-shape decode step
(batch 16, context 2048, d_model 4096, 32 heads of 128, SwiGLU 11008, f32 paged cache, every
linear int4) followed by the lm_head (vocab 32000) and the greedy argmax, run by this library on
the GPU and by the CPU oracle on identical seeded weights, cache contents and activations.

The small-shape step test (test_decode_gpu.py) covers many steps and both cache dtypes; this one
covers the shapes, split plans and kernel selections the benchmark actually times."""
import pytest

from oracle.step import LayerSample, layer_parity
from util import ATTN_TOL

pytestmark = pytest.mark.gpu


def test_one_full_size_layer_and_the_head_match_the_oracle():
    sample = LayerSample(batch=16, context=2048, seed=11)
    r = layer_parity(sample, "cuda:0")
    # the hidden state compounds seven int4 products (1e-3 each) and one attention (2e-3)
    assert r["hidden_rel_err"] <= ATTN_TOL, r
    assert r["logits_rel_err"] <= 5e-3, r
    assert r["rows_with_clear_argmax"] >= 1 and r["ids_equal_on_clear_rows"], r
