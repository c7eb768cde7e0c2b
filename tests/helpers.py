"""Shared pieces of the tests: the two tiny configurations, model folders made in temporary
directories, schedules, and the tolerances (fixed here once, for every test)."""
import os

import torch

from forge_b200.config import config_from_dict
from forge_b200.weights import write_random_model

# Two tiny LLaMA configurations that differ in every size and option: layers, width, heads and groups
# (GQA 4:2 vs MQA 3:1, the latter a group of 3), head size, a feed-forward width and a vocabulary that are
# no powers of two, rotary base, norm eps, q/k/v bias, tied or untied head, position limit.
TINY = {
    "A": dict(architectures=["LlamaForCausalLM"], vocab_size=250, hidden_size=64, intermediate_size=176,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16, rope_theta=10000.0,
              rms_norm_eps=1e-5, attention_bias=False, tie_word_embeddings=False, max_position_embeddings=768),
    "B": dict(architectures=["LlamaForCausalLM"], vocab_size=387, hidden_size=96, intermediate_size=264,
              num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1, head_dim=32, rope_theta=500000.0,
              rms_norm_eps=1e-6, attention_bias=True, tie_word_embeddings=True, max_position_embeddings=1024),
    # head size 64 and widths at which the bfloat16 path takes the kernels that serving takes at real sizes:
    # the tcgen05 prompt attention (requests of 128 rows and more), wide GEMM tiles, the few-rows GEMM with
    # its reduction cut across a cluster.  eps is large enough that losing it on the way from config.json to
    # a norm would show in every logit.
    "C": dict(architectures=["LlamaForCausalLM"], vocab_size=1000, hidden_size=512, intermediate_size=1408,
              num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=64, rope_theta=20000.0,
              rms_norm_eps=1e-2, attention_bias=False, tie_word_embeddings=False, max_position_embeddings=1536),
    # head size 128 with 7 query heads on one kv head and q/k/v bias (the Qwen2.5-7B kind of layer): the tcgen05 prompt
    # attention with two blocks per head and tiles of 18 tokens = 126 rows, the projection whose epilogue rotates heads
    # of 128, a q width (896) that is not the hidden width (448)
    "D": dict(architectures=["Qwen2ForCausalLM"], vocab_size=777, hidden_size=448, intermediate_size=1216,
              num_hidden_layers=2, num_attention_heads=7, num_key_value_heads=1, head_dim=128, rope_theta=1000000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=1280),
}
SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3}
# weights are drawn so that attention is far from uniform and the logits are of order 10 at every width
STDS = {"A": dict(std=0.12, embed_std=0.6, norm_std=0.15, bias_std=0.2),
        "B": dict(std=0.12, embed_std=0.6, norm_std=0.15, bias_std=0.2),
        "C": dict(std=0.07, embed_std=0.6, norm_std=0.15, bias_std=0.2),
        "D": dict(std=0.07, embed_std=0.6, norm_std=0.15, bias_std=0.3)}

# max |engine - plain| allowed, as a fraction of max |plain logits| of the compared rows.
# float32: the engine rounds every product and sum to fp32 (the oracle is float64) and takes rotary
# angles in fp32.  bfloat16: activations, cache and matrices are rounded to 8 bits of mantissa.
TOL = {"float32": 2e-4, "bfloat16": 4e-2}


def tiny_config(name):
    return config_from_dict(TINY[name])


def make_model_dir(tmp_path_factory, name):
    """A model folder with weights large enough that attention is far from uniform and every norm
    weight and bias matters."""
    d = str(tmp_path_factory.mktemp(f"tiny{name}"))
    write_random_model(tiny_config(name), d, seed=SEEDS[name], **STDS[name])
    return d


def random_tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def assert_greedy_follows_plain(logits_fn, prompt, got, tol, what=""):
    """Every generated token must be the plain implementation's best next token given the tokens before it,
    or lie within 2*tol (of the logit scale) of the best: only a near-tie may be decided differently.  Unlike
    a comparison of two texts this does not stop meaning anything after the first near-tie."""
    ids = list(prompt)
    for i, t in enumerate(got):
        lg = logits_fn(ids)[-1]
        gap = float((lg.max() - lg[t]) / lg.abs().max())
        assert gap <= 2 * tol, f"{what} token {i}: engine chose {t}, plain prefers {int(lg.argmax())} by {gap:.3g} of the scale"
        ids.append(int(t))


def max_rel_err(got, want):
    want = want.to(torch.float32).cpu()
    got = got.to(torch.float32).cpu()
    return float((got - want).abs().max() / want.abs().max())
