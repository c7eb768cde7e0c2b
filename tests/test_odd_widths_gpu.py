"""Widths that no fast path takes: a hidden width of 102 (not a multiple of 4: the norm goes element by element, the
products that add into the residual write without vectors or TMA) and an intermediate width of 150; with them the
reduction dimension of the q/k/v, gate/up and output-head products is no multiple of 8, so in bfloat16 those go to the
FMA kernel on bfloat16 operands while the o-projection (reduction over 6 x 16 = 96) stays on the tensor cores.
The whole model against the plain implementation, in every way of cutting, both precisions."""
import pytest
import torch

import schedules
from helpers import TOL, random_tokens
from plain.llama import PlainLlama
from test_engine_gpu import first_bad, make_runner, run_schedule

pytestmark = pytest.mark.gpu

ODD = dict(architectures=["LlamaForCausalLM"], vocab_size=333, hidden_size=102, intermediate_size=150,
           num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=3, head_dim=16, rope_theta=7000.0,
           rms_norm_eps=1e-4, attention_bias=False, tie_word_embeddings=False, max_position_embeddings=512)
LENGTHS = [150, 31, 77, 200]


@pytest.fixture(scope="module")
def odd(tmp_path_factory):
    from forge_b200.config import config_from_dict
    from forge_b200.weights import write_random_model
    d = str(tmp_path_factory.mktemp("odd"))
    write_random_model(config_from_dict(ODD), d, seed=21, std=0.12, embed_std=0.6, norm_std=0.15, bias_std=0.2)
    plain = PlainLlama(d)
    reqs = {f"r{i}": random_tokens(n, ODD["vocab_size"], seed=5 * i + 1) for i, n in enumerate(LENGTHS)}
    want = {rid: plain.logits(toks).float() for rid, toks in reqs.items()}
    return d, reqs, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("schedule", ["whole", "last_one_by_one", "changing_portions", "mixed"])
def test_schedules_equal_plain(odd, dtype, schedule):
    d, reqs, want = odd
    steps = getattr(schedules, schedule)(reqs)
    runner = make_runner(d, dtype, schedules.peak_tokens(reqs, steps, round_to=16))
    if dtype == "bfloat16":
        mixer = runner.model.blocks[0].mixer
        assert not mixer.qkv.tensor_core and mixer.o.tensor_core
    got = run_schedule(runner, reqs, steps)
    assert first_bad(got, want, TOL[dtype]) is None, first_bad(got, want, TOL[dtype])
    assert runner.manager.num_free_pages() == {g: runner.num_pages for g in runner.manager.groups}


def test_greedy_generation_through_the_entry_point(odd):
    import forge_b200 as forge
    from test_generate_gpu import assert_greedy_follows_plain
    d, reqs, want = odd
    plain = PlainLlama(d)
    model = forge.Model(d, dtype="bfloat16", max_num_seqs=4, cache_tokens=1024)
    for p in (reqs["r1"], reqs["r2"][:9]):
        out = model.generate(p, max_new_tokens=24, do_sample=False)["token_ids"]
        assert len(out) == 24
        assert_greedy_follows_plain(plain.logits, p, out, TOL["bfloat16"], f"prompt of {len(p)} tokens")
