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
    a, b = GOLDEN_CONFIGS["gqa_untied"], GOLDEN_CONFIGS["mqa_tied_bias"]
    for key in a:
        assert a[key] != b[key], key
