"""The engine (model, step function, cache, kernels) against the plain implementation, in 32-bit and in
bfloat16, under every way of cutting and batching the same requests."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import schedules
from helpers import TINY, TOL, make_model_dir, max_rel_err, random_tokens
from plain.llama import PlainLlama

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]
# C: with 4 query heads per kv head a request brings 128 rows from 32 tokens on; its lengths lie on both sides
LENGTHS = {"A": [70, 129, 33, 200, 64, 97], "B": [150, 47, 16, 240, 81], "C": [300, 20, 131, 700, 45, 257],
           "D": [210, 9, 95, 400, 37]}


@pytest.fixture(scope="module", params=["A", "B", "C", "D"])
def tiny(request, tmp_path_factory):
    name = request.param
    d = make_model_dir(tmp_path_factory, name)
    plain = PlainLlama(d)
    reqs = {f"r{i}": random_tokens(n, TINY[name]["vocab_size"], seed=10 * i + len(name))
            for i, n in enumerate(LENGTHS[name])}
    want = {rid: plain.logits(toks).float() for rid, toks in reqs.items()}
    return name, d, plain, reqs, want


def run_schedule(runner, reqs, steps):
    """Feeds the schedule through ModelRunner.step asking for every position's logits; returns
    {request: [len, V] tensor}."""
    from forge_b200.engine import StepEntry
    V = runner.plan.vocab_size
    got = {rid: torch.full((len(t), V), float("nan")) for rid, t in reqs.items()}
    for entries, end in steps:
        for rid, p, n in entries:
            if not runner.is_live(rid):
                runner.admit(rid)
        logits = runner.step([StepEntry(rid, reqs[rid][p:p + n], list(range(n))) for rid, p, n in entries]).cpu()
        o = 0
        for rid, p, n in entries:
            got[rid][p:p + n] = logits[o:o + n]
            o += n
        for rid in end:
            runner.release(rid)
        runner.manager.check()
    runner.check_status()
    return got


def first_bad(got, want, tol):
    """(request, position) of the first row beyond tolerance, for the failure message."""
    for rid in want:
        scale = want[rid].abs().max()
        err = (got[rid] - want[rid]).abs().amax(dim=1) / scale
        bad = torch.nonzero(~(err <= tol))
        if len(bad):
            p = int(bad[0])
            return f"first wrong row: request {rid} position {p} (of {len(want[rid])}), rel err {float(err[p]):.3g}"
    return None


def make_runner(model_dir, dtype, cache_tokens, page_size=16):
    from forge_b200.engine import ModelRunner
    return ModelRunner(model_dir, dtype=dtype, page_size=page_size, cache_tokens=cache_tokens, max_requests=4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("schedule", ["whole", "last_one_by_one", "changing_portions", "mixed"])
def test_schedules_equal_plain(tiny, dtype, schedule):
    name, d, plain, reqs, want = tiny
    steps = getattr(schedules, schedule)(reqs)
    # exactly as many pages as the schedule's peak needs: freed pages are taken again at once
    runner = make_runner(d, dtype, schedules.peak_tokens(reqs, steps, round_to=16))
    got = run_schedule(runner, reqs, steps)
    assert first_bad(got, want, TOL[dtype]) is None, first_bad(got, want, TOL[dtype])
    assert runner.manager.num_free_pages() == {g: runner.num_pages for g in runner.manager.groups}


@pytest.mark.parametrize("dtype", DTYPES)
def test_page_size_does_not_matter(tiny, dtype):
    name, d, plain, reqs, want = tiny
    small = {k: reqs[k] for k in list(reqs)[:3]}
    for ps in (8, 16, 64):
        steps = schedules.mixed(small, max_live=3)
        runner = make_runner(d, dtype, schedules.peak_tokens(small, steps, round_to=ps), page_size=ps)
        got = run_schedule(runner, small, steps)
        msg = first_bad(got, {k: want[k] for k in small}, TOL[dtype])
        assert msg is None, f"page size {ps}: {msg}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(tiny, dtype):
    """A 3-token prompt, then hundreds of tokens one by one."""
    name, d, plain, reqs, want = tiny
    n = {"A": 400, "B": 520, "C": 330, "D": 300}[name]
    toks = random_tokens(n, TINY[name]["vocab_size"], seed=77)
    ref = plain.logits(toks).float()
    runner = make_runner(d, dtype, -(-n // 16) * 16)
    steps = [([("x", 0, 3)], [])] + [([("x", p, 1)], []) for p in range(3, n)]
    got = run_schedule(runner, {"x": toks}, steps)
    msg = first_bad(got, {"x": ref}, TOL[dtype])
    assert msg is None, msg


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens(tiny, dtype):
    """A sequence's first tokens, each in a step of its own, from an empty cache."""
    name, d, plain, reqs, want = tiny
    toks = reqs["r0"][:5]
    runner = make_runner(d, dtype, 64)
    got = run_schedule(runner, {"r0": toks}, [([("r0", p, 1)], []) for p in range(5)])
    assert max_rel_err(got["r0"], want["r0"][:5]) <= TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_wanted_rows_only(tiny, dtype):
    """Asking for some rows gives the same numbers as asking for all; asking for none returns nothing."""
    from forge_b200.engine import StepEntry
    name, d, plain, reqs, want = tiny
    runner = make_runner(d, dtype, 512)
    runner.admit("a"), runner.admit("b")
    other = next(k for k in reqs if k != "r0" and len(reqs[k]) >= 30)
    ta, tb = reqs["r0"][:40], reqs[other][:30]
    assert runner.step([StepEntry("a", ta[:20], [])]) is None
    lg = runner.step([StepEntry("a", ta[20:], [19, 0]), StepEntry("b", tb, [29])]).cpu()
    assert lg.shape == (3, runner.plan.vocab_size)
    tol = TOL[dtype]
    assert max_rel_err(lg[0:1], want["r0"][39:40]) <= tol
    assert max_rel_err(lg[1:2], want["r0"][20:21]) <= tol
    assert max_rel_err(lg[2:3], want[other][29:30]) <= tol


def test_step_refuses_bad_input(tiny):
    from forge_b200.cache import OutOfPages
    from forge_b200.engine import StepEntry, StepError
    name, d, plain, reqs, want = tiny
    runner = make_runner(d, "float32", 32)
    runner.admit("a")
    V = runner.plan.vocab_size
    with pytest.raises(StepError):
        runner.step([StepEntry("a", [V], [0])])
    with pytest.raises(StepError):
        runner.step([StepEntry("zz", [1], [0])])
    with pytest.raises(OutOfPages):
        runner.step([StepEntry("a", [1] * 33, [0])])
    # nothing was held back by the refused steps
    assert runner.manager.num_tokens("a") == 0
    assert runner.step([StepEntry("a", [1] * 32, [31])]) is not None
    runner.manager.check()


def test_fp32_schedules_are_bitwise_equal(tiny):
    """In 32-bit every sum runs in a fixed order (matrix products over k, attention over a token's keys, the
    norms' reduction tree) whatever the step looks like, so the logits at a position must be the SAME BITS
    however the tokens were cut into steps, whatever else was in the batch and wherever the pages lie."""
    name, d, plain, reqs, want = tiny
    results = {}
    for schedule in ("whole", "last_one_by_one", "changing_portions", "mixed"):
        steps = getattr(schedules, schedule)(reqs)
        for ps in ((16, 64) if schedule == "mixed" else (16,)):
            runner = make_runner(d, "float32", schedules.peak_tokens(reqs, steps, round_to=ps), page_size=ps)
            results[(schedule, ps)] = run_schedule(runner, reqs, steps)
            del runner
    base = results[("whole", 16)]
    for key, got in results.items():
        for rid in reqs:
            same = (got[rid] == base[rid]).all(dim=1)
            assert bool(same.all()), (f"{key}: request {rid} position {int(torch.nonzero(~same)[0])} differs from the "
                                      f"whole-prompt run by {float((got[rid] - base[rid]).abs().max()):.3g}")


def _trace_lines(reqs, steps):
    lines = []
    for s, (entries, end) in enumerate(steps):
        lines.append(json.dumps({"step": s, "end": end, "entries": [
            {"id": rid, "tokens": reqs[rid][p:p + n], "want": list(range(n))} for rid, p, n in entries]}))
    return "\n".join(lines) + "\n"


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program(tiny, dtype, tmp_path):
    """bin/trace_run as a user runs it: steps on stdin, <step>.f32 files and `done <step>` lines out."""
    name, d, plain, reqs, want = tiny
    small = {k: reqs[k] for k in list(reqs)[:4]}
    steps = schedules.mixed(small, max_live=3)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype,
                           "--out", str(out), "--max-tokens", str(schedules.peak_tokens(small, steps, 64))],
                          input=_trace_lines(small, steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s}" for s in range(len(steps))]
    V = TINY[name]["vocab_size"]
    for s, (entries, end) in enumerate(steps):
        arr = torch.from_numpy(np.fromfile(out / f"{s}.f32", dtype="<f4").reshape(-1, V))
        o = 0
        for rid, p, n in entries:
            assert max_rel_err(arr[o:o + n], want[rid][p:p + n]) <= TOL[dtype], (s, rid, p)
            o += n
        assert o == arr.shape[0]


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_steps_do_not_go_through_the_allocator(tiny, dtype):
    """The outputs of a step's kernels are views into the runner's workspace: after a first step of some size, a
    step of that size asks the allocator for the logits it hands out and for nothing else, and a step beyond
    max_tokens_per_step is refused before anything is touched."""
    from forge_b200.engine import ModelRunner, StepEntry, StepError
    name, d, plain, reqs, want = tiny
    runner = ModelRunner(d, dtype=dtype, page_size=16, cache_tokens=512, max_requests=4, max_tokens_per_step=96)
    toks = reqs["r0"][:64]
    got = []
    for rep in range(3):
        runner.admit("a"), runner.admit("b")
        torch.cuda.synchronize()
        before, misses = torch.cuda.memory_stats()["allocation.all.allocated"], runner.workspace.allocations
        lg = runner.step([StepEntry("a", toks[:40], [39]), StepEntry("b", toks[:24], [0, 23])])
        torch.cuda.synchronize()
        if rep > 0:
            assert runner.workspace.allocations == misses, "a kernel output did not fit the workspace"
            assert torch.cuda.memory_stats()["allocation.all.allocated"] - before <= 1, "more than the logits was allocated"
        got.append(lg.cpu())
        runner.release("a"), runner.release("b")
    assert torch.equal(got[0], got[1]) and torch.equal(got[1], got[2])
    assert max_rel_err(got[2][0:1], want["r0"][39:40]) <= TOL[dtype]
    assert runner.workspace.capacity > 0 and runner.workspace.high <= runner.workspace.capacity
    runner.admit("c")
    with pytest.raises(StepError, match="96"):
        runner.step([StepEntry("c", toks + toks[:33], [])])
    assert runner.manager.num_tokens("c") == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_schedules_under_the_checks_build(tiny, dtype, monkeypatch):
    """FORGE_CHECKS=1: the kernels are built with a test of every page id, slot and token index before it is used.
    The four schedules (valid tables only) must run as before and leave the status word at zero."""
    from forge_b200 import kernels
    name, d, plain, reqs, want = tiny
    monkeypatch.setenv("FORGE_CHECKS", "1")
    for schedule in ("whole", "last_one_by_one", "changing_portions", "mixed"):
        steps = getattr(schedules, schedule)(reqs)
        runner = make_runner(d, dtype, schedules.peak_tokens(reqs, steps, round_to=16))
        assert runner.first_bad is not None
        got = run_schedule(runner, reqs, steps)             # ends with check_status(): raises if a check fired
        assert int(runner.status.item()) == 0 and runner.first_bad.tolist() == [0, 0, 0]
        assert first_bad(got, want, TOL[dtype]) is None, (schedule, first_bad(got, want, TOL[dtype]))
    built = [n for (n, defines) in kernels._libs if ("FORGE_CHECKS", 1) in defines]
    assert "core" in built and (dtype == "float32" or "attention_mma" in built), built
