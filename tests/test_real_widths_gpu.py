"""The engine at the layer widths that the benchmark times (TinyLlama-1.1B: hidden 2048, 32 query heads on 4
kv heads of 64, feed-forward 5632, vocabulary 32000), with 2 of its 22 layers so that the plain float64
implementation stays a matter of seconds.  At these widths the bfloat16 path runs the kernels that the small
test configurations never reach as a whole model: the tcgen05 prompt attention, the CTA-pair matrix product,
the few-rows product with its reduction cut across a cluster, and the evenly dealt output head.  Same four
ways of cutting and batching as for the tiny models, every position compared."""
import pytest
import torch

import schedules
from helpers import TOL, max_rel_err, random_tokens
from plain.llama import PlainLlama
from test_engine_gpu import first_bad, run_schedule

pytestmark = pytest.mark.gpu

WIDTHS = dict(architectures=["LlamaForCausalLM"], vocab_size=32000, hidden_size=2048, intermediate_size=5632,
              num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=4, head_dim=64, rope_theta=10000.0,
              rms_norm_eps=1e-5, attention_bias=False, tie_word_embeddings=False, max_position_embeddings=2048)
LENGTHS = [300, 40, 150, 90, 200, 64]


@pytest.fixture(scope="module")
def real_widths(tmp_path_factory):
    from forge_b200.config import config_from_dict
    from forge_b200.weights import write_random_model
    d = str(tmp_path_factory.mktemp("widths"))
    write_random_model(config_from_dict(WIDTHS), d, seed=5, std=0.03, embed_std=0.5, norm_std=0.1)
    plain = PlainLlama(d)
    reqs = {f"w{i}": random_tokens(n, WIDTHS["vocab_size"], seed=100 + i) for i, n in enumerate(LENGTHS)}
    want = {rid: plain.logits(toks).float() for rid, toks in reqs.items()}
    del plain
    return d, reqs, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [16, 64])
def test_every_schedule_at_benchmark_widths(real_widths, dtype, page_size):
    from forge_b200.engine import ModelRunner
    d, reqs, want = real_widths
    plans = {name: getattr(schedules, name)(reqs) for name in ("whole", "last_one_by_one", "changing_portions", "mixed")}
    # one runner for all four (loading is the slow part); the pool is the largest peak, so within the mixed
    # schedule pages that one request gave back are taken by the next at once
    peak = max(schedules.peak_tokens(reqs, steps, round_to=page_size) for steps in plans.values())
    runner = ModelRunner(d, dtype=dtype, page_size=page_size, cache_tokens=peak, max_requests=4)
    results = {}
    for name, steps in plans.items():
        got = results[name] = run_schedule(runner, reqs, steps)
        msg = first_bad(got, want, TOL[dtype])
        assert msg is None, f"{name}, pages of {page_size}: {msg}"
        assert runner.manager.num_free_pages() == {g: runner.num_pages for g in runner.manager.groups}
    if dtype == "float32":      # in 32-bit the four must agree to the bit
        for name, got in results.items():
            for rid in reqs:
                assert torch.equal(got[rid], results["whole"][rid]), f"{name}: request {rid} differs from the whole-prompt run"


def test_greedy_generation_at_benchmark_widths(real_widths):
    """Through the Python entry point, bfloat16, eight requests at once (decode steps replay the graph)."""
    import forge_b200 as forge
    from helpers import assert_greedy_follows_plain
    d, reqs, want = real_widths
    plain = PlainLlama(d)
    model = forge.Model(d, dtype="bfloat16", block_size=64, max_num_seqs=4, cache_tokens=1024)
    sched = forge.RequestScheduler(model, max_num_seqs=4)
    prompts = [reqs["w1"][:37], reqs["w3"][:70], reqs["w5"][:5]]
    ids = [sched.submit(p, max_new_tokens=6, sampler_config=forge.SamplerConfig(do_sample=False)) for p in prompts]
    done = {r.request_id: r for r in sched.run()}
    for rid, p in zip(ids, prompts):
        assert_greedy_follows_plain(plain.logits, p, done[rid].output_tokens, TOL["bfloat16"], f"request {rid}")
