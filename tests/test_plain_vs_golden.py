"""The plain implementation against logits of the UNMODIFIED reference CPU engine.

tests/golden/ref_logits_*.npy were written by tests/golden/make_golden.py, which compiles
Cyxuan0311/Forge's CPU sources and runs `InferenceEngine::forward` (a prefill, then single
tokens) on the deterministic models of tests/golden/golden_model.py.
"""
import os

import numpy as np
import pytest
import torch

from golden.golden_model import GOLDEN_CONFIGS, GOLDEN_STEPS, golden_tensors
from plain.llama import PlainLlama

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("name", sorted(GOLDEN_CONFIGS))
def test_plain_equals_reference_engine(name):
    ref = np.load(os.path.join(HERE, "golden", f"ref_logits_{name}.npy"))
    cfg = GOLDEN_CONFIGS[name]
    plain = PlainLlama.from_tensors(cfg, golden_tensors(cfg, seed=7))
    ids = [t for _, toks in GOLDEN_STEPS[name] for t in toks]
    mine = plain.logits(ids).to(torch.float32).numpy()
    assert mine.shape == ref.shape
    scale = np.abs(ref).max()
    # the reference computes in float32; 1e-5 of the logit scale is a few of its ulps
    assert np.abs(mine - ref).max() <= 1e-5 * scale


def test_golden_models_differ_in_every_option():
    a, b = GOLDEN_CONFIGS["mha_untied"], GOLDEN_CONFIGS["mqa_tied_bias"]
    for key in a:
        assert a[key] != b[key], key


def test_a_golden_model_pins_the_kv_head_of_a_query_head():
    """One of the models has 1 < kv heads < heads, and a plain implementation with the other mapping
    (h % kv heads) would not pass against the reference's logits."""
    import plain.llama as L
    cfg = GOLDEN_CONFIGS["gqa_6_2_bias"]
    assert 1 < cfg["num_key_value_heads"] < cfg["num_attention_heads"]
    ref = np.load(os.path.join(HERE, "golden", "ref_logits_gqa_6_2_bias.npy"))
    plain = PlainLlama.from_tensors(cfg, golden_tensors(cfg, seed=7))
    ids = [t for _, toks in GOLDEN_STEPS["gqa_6_2_bias"] for t in toks]
    real = L.attention

    def other_mapping(q, k, v, window=None):
        nh, nkv = q.shape[1], k.shape[1]
        place = [(h % nkv) * (nh // nkv) + h // nkv for h in range(nh)]      # where head h must stand to read kv head h % nkv
        head_at = [place.index(i) for i in range(nh)]
        return real(q[:, head_at], k, v, window)[:, place]

    L.attention = other_mapping
    try:
        wrong = plain.logits(ids).to(torch.float32).numpy()
    finally:
        L.attention = real
    assert np.abs(wrong - ref).max() > 1e-2 * np.abs(ref).max()
