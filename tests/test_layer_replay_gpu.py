"""The launches of one layer, noted and repeated for the layers after it (engine/model.py, kernels.LayerReplay):
models deep enough for it, against the plain implementation and, bit for bit, against the same engine with every layer
run by its parts."""
import pytest
import torch

from helpers import STDS, TINY, TOL, random_tokens
from plain.llama import PlainLlama
import schedules
from test_engine_gpu import first_bad, run_schedule

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]

# the tiny configurations A (small heads, every kernel's general form), C (the serving kernels of head size 64) and D
# (heads of 128, bias) with six layers: one run by the parts and noted, five repeated
DEEP = {name: dict(TINY[name], num_hidden_layers=6) for name in ("A", "C", "D")}
LENGTHS = {"A": [70, 129, 33, 200], "C": [300, 20, 131, 260], "D": [210, 9, 95, 150]}


@pytest.fixture(scope="module", params=["A", "C", "D"])
def deep(request, tmp_path_factory):
    from forge_b200.config import config_from_dict
    from forge_b200.weights import write_random_model
    name = request.param
    d = str(tmp_path_factory.mktemp(f"deep{name}"))
    # smaller weights than the shallow models': six layers of them keep the logits at order 10
    std = dict(STDS[name], std=STDS[name]["std"] * 0.7)
    write_random_model(config_from_dict(DEEP[name]), d, seed=40 + len(name), **std)
    plain = PlainLlama(d)
    reqs = {f"r{i}": random_tokens(n, DEEP[name]["vocab_size"], seed=7 * i + 3) for i, n in enumerate(LENGTHS[name])}
    want = {rid: plain.logits(toks).float() for rid, toks in reqs.items()}
    return name, d, reqs, want


def make_runner(model_dir, dtype, cache_tokens, page_size=16):
    from forge_b200.engine import ModelRunner
    return ModelRunner(model_dir, dtype=dtype, page_size=page_size, cache_tokens=cache_tokens, max_requests=4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("schedule", ["whole", "last_one_by_one", "changing_portions", "mixed"])
def test_deep_models_equal_plain_and_themselves_without_replay(deep, dtype, schedule, monkeypatch):
    name, d, reqs, want = deep
    steps = getattr(schedules, schedule)(reqs)
    tokens = schedules.peak_tokens(reqs, steps, round_to=16)
    runner = make_runner(d, dtype, tokens)
    assert runner.model._replay_ok, "the stock layers declare that their launches may be repeated"
    got = run_schedule(runner, reqs, steps)
    assert first_bad(got, want, TOL[dtype]) is None, first_bad(got, want, TOL[dtype])
    # the same schedule with every layer run by its parts: the same launches, so the same bits
    monkeypatch.setenv("FORGE_LAYER_REPLAY", "0")
    plain_runner = make_runner(d, dtype, tokens)
    again = run_schedule(plain_runner, reqs, steps)
    for rid in reqs:
        assert torch.equal(got[rid], again[rid]), f"request {rid}: repeated launches gave other bits than the parts' own"


@pytest.mark.parametrize("dtype", DTYPES)
def test_launches_are_counted_and_really_repeated(deep, dtype, monkeypatch):
    """A prompt step makes the same number of launches with and without repetition, and with it only one of the six
    layers goes through the parts (seen by counting the calls of one part)."""
    from forge_b200 import kernels
    from forge_b200.engine import StepEntry
    from forge_b200.parts.norm import RMSNorm
    name, d, reqs, want = deep
    toks = reqs["r0"]
    calls = [0]
    orig = RMSNorm.forward

    def counted(self, *a, **k):
        calls[0] += 1
        return orig(self, *a, **k)
    monkeypatch.setattr(RMSNorm, "forward", counted)
    runner = make_runner(d, dtype, 512)
    runner.admit("a"); runner.step([StepEntry("a", toks, [len(toks) - 1])]); runner.release("a")      # sizes the workspace
    counts = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("FORGE_LAYER_REPLAY", mode)
        calls[0] = 0
        before = kernels.launch_count()
        runner.admit("a")
        logits = runner.step([StepEntry("a", toks, [len(toks) - 1])])
        runner.release("a")
        counts[mode] = (kernels.launch_count() - before, calls[0], logits.clone())
    assert counts["1"][0] == counts["0"][0]
    assert counts["0"][1] == 2 * 6 + 1 and counts["1"][1] == 2 * 1 + 1      # two norms a layer, and the final one
    assert torch.equal(counts["1"][2], counts["0"][2])


def test_a_step_that_outgrows_the_workspace_is_not_repeated(deep):
    """The first step of a fresh runner gets some of its outputs from the allocator (the workspace is sized by the
    steps seen so far): their addresses mean nothing in the next layer, so that step's layers all run by their parts."""
    from forge_b200.engine import StepEntry
    name, d, reqs, want = deep
    toks = reqs["r1"] if len(reqs["r1"]) > 100 else reqs["r0"]
    rid = "r1" if len(reqs["r1"]) > 100 else "r0"
    runner = make_runner(d, "bfloat16", 512)
    runner.admit("a")
    first = runner.step([StepEntry("a", toks, list(range(len(toks))))]).cpu()
    runner.release("a")
    runner.admit("a")
    second = runner.step([StepEntry("a", toks, list(range(len(toks))))]).cpu()
    runner.release("a")
    assert torch.equal(first, second)
    assert float((first - want[rid]).abs().max() / want[rid].abs().max()) <= TOL["bfloat16"]


def test_layers_with_parts_that_do_not_declare_it_are_run_by_their_parts(tmp_path):
    """A norm defined here, without the declaration: the model built from it never repeats launches."""
    from forge_b200.config import config_from_dict
    from forge_b200.config.base import PartSpec
    from forge_b200.engine import ModelRunner, StepEntry
    from forge_b200.parts import register_part, unregister_part
    from forge_b200.parts.norm import RMSNorm
    from forge_b200.weights import write_random_model

    class CountingNorm(RMSNorm):               # keeps host state per call: must not be skipped
        seen = 0

        def forward(self, x, out_dtype=None, rows=None):
            CountingNorm.seen += 1
            return super().forward(x, out_dtype, rows)

    register_part("norm", "counting_rmsnorm", CountingNorm)
    try:
        cfg = config_from_dict(DEEP["A"])
        d = str(tmp_path / "m")
        write_random_model(cfg, d, seed=5, **STDS["A"])
        orig_plan = type(cfg).plan

        def plan(self):
            p = orig_plan(self)
            for layer in p.layers:
                for key, spec in list(layer.norms.items()):
                    layer.norms[key] = PartSpec("counting_rmsnorm", spec.params)
            return p
        type(cfg).plan = plan
        try:
            runner = ModelRunner(d, dtype="bfloat16", page_size=16, cache_tokens=256, max_requests=2)
        finally:
            type(cfg).plan = orig_plan
        assert not runner.model._replay_ok
        toks = random_tokens(90, DEEP["A"]["vocab_size"], seed=1)
        for _ in range(2):
            CountingNorm.seen = 0
            runner.admit("a"); runner.step([StepEntry("a", toks, [89])]); runner.release("a")
            assert CountingNorm.seen == 2 * 6
    finally:
        unregister_part("norm", "counting_rmsnorm")


def test_a_first_layer_of_another_kind_is_run_by_its_parts_and_the_second_is_noted(tmp_path, monkeypatch):
    """Only the first layer has the norm that does not declare it: that layer always runs by its parts, the second is
    noted and the four after it repeat its launches; the same bits as with every layer run by its parts."""
    from forge_b200.config import config_from_dict
    from forge_b200.config.base import PartSpec
    from forge_b200.engine import ModelRunner, StepEntry
    from forge_b200.parts import register_part, unregister_part
    from forge_b200.parts.norm import RMSNorm
    from forge_b200.weights import write_random_model

    class FirstNorm(RMSNorm):
        seen = 0

        def forward(self, x, out_dtype=None, rows=None):
            FirstNorm.seen += 1
            return super().forward(x, out_dtype, rows)

    register_part("norm", "first_rmsnorm", FirstNorm)
    try:
        cfg = config_from_dict(DEEP["C"])
        d = str(tmp_path / "m")
        write_random_model(cfg, d, seed=6, **STDS["C"])
        orig_plan = type(cfg).plan

        def plan(self):
            p = orig_plan(self)
            for key, spec in list(p.layers[0].norms.items()):
                p.layers[0].norms[key] = PartSpec("first_rmsnorm", spec.params)
            return p
        toks = random_tokens(150, DEEP["C"]["vocab_size"], seed=2)
        outs = {}
        for mode in ("1", "0"):
            monkeypatch.setenv("FORGE_LAYER_REPLAY", mode)
            type(cfg).plan = plan
            try:
                runner = ModelRunner(d, dtype="bfloat16", page_size=16, cache_tokens=256, max_requests=2)
            finally:
                type(cfg).plan = orig_plan
            assert runner.model._replay_ok and runner.model._replay_from == 1
            for _ in range(2):              # the second step finds its workspace sized
                FirstNorm.seen = 0
                runner.admit("a")
                outs[mode] = runner.step([StepEntry("a", toks, list(range(150)))]).clone()
                runner.release("a")
                assert FirstNorm.seen == 2
        assert torch.equal(outs["1"], outs["0"])
    finally:
        unregister_part("norm", "first_rmsnorm")
