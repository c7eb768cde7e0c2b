"""The plain implementation itself: properties that hold whatever the weights are."""
import torch

from helpers import TINY, make_model_dir, random_tokens
from plain.llama import PlainLlama, attention, rms_norm, rope


def test_causal_and_deterministic(tmp_path_factory):
    d = make_model_dir(tmp_path_factory, "A")
    m = PlainLlama(d)
    ids = random_tokens(12, TINY["A"]["vocab_size"], 3)
    full = m.logits(ids)
    assert torch.equal(full, m.logits(ids))
    assert torch.allclose(full[:7], m.logits(ids[:7]), atol=1e-12)          # later tokens do not matter
    assert not torch.allclose(full[3], m.logits(ids[:2] + [ids[2] ^ 1] + ids[3:])[3])


def test_rope_is_a_rotation_that_depends_on_relative_position():
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, 32, generator=g, dtype=torch.float64), torch.randn(1, 1, 32, generator=g, dtype=torch.float64)
    def dot(pq, pk):
        return float((rope(q, torch.tensor([pq]), 1e4) * rope(k, torch.tensor([pk]), 1e4)).sum())
    assert abs(dot(5, 3) - dot(105, 103)) < 1e-9 and abs(dot(5, 3) - dot(5, 4)) > 1e-6
    assert abs(float(rope(q, torch.tensor([77]), 5e5).norm()) - float(q.norm())) < 1e-12


def test_attention_window_and_groups():
    g = torch.Generator().manual_seed(1)
    q = torch.randn(9, 4, 8, generator=g, dtype=torch.float64)
    k = torch.randn(9, 2, 8, generator=g, dtype=torch.float64)
    v = torch.randn(9, 2, 8, generator=g, dtype=torch.float64)
    full = attention(q, k, v)
    assert torch.allclose(full[0, 0], v[0, 0]) and torch.allclose(full[0, 3], v[0, 1])   # heads 2,3 read kv head 1
    win = attention(q, k, v, window=3)
    assert torch.allclose(win[:3], full[:3]) and not torch.allclose(win[8], full[8])
    assert torch.allclose(attention(q, k, v, window=1)[5, 1], v[5, 0])


def test_rms_norm_scale():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(rms_norm(x, torch.ones(2, dtype=torch.float64), 0.0), x / (12.5 ** 0.5))
