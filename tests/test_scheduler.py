"""The scheduler's decisions with a fake step function: a real CacheManager, no model, no GPU."""
from types import SimpleNamespace

import pytest

from forge_b200.cache import CacheManager, GroupSpec
from forge_b200.engine.scheduler import RequestScheduler, RequestStatus
from forge_b200.sampling import SamplerConfig, XorShift64


class FakeRunner:
    """Stands in for ModelRunner: appends tokens to the real cache manager and returns 'logits' that are
    just the (request, position) of each wanted row."""

    def __init__(self, pages=8, page_size=4, max_requests=4, vocab=100, max_positions=64):
        self.manager = CacheManager([GroupSpec("g", pages)], page_size, max_requests)
        self.plan = SimpleNamespace(vocab_size=vocab, max_positions=max_positions)
        self.steps = []

    def admit(self, rid):
        return self.manager.admit(rid)

    def release(self, rid):
        self.manager.free(rid)

    def step(self, entries):
        self.steps.append([(e.req_id, len(e.tokens), list(e.want)) for e in entries])
        rows = []
        for e in entries:
            start = self.manager.num_tokens(e.req_id)
            self.manager.append(e.req_id, len(e.tokens))
            rows += [(e.req_id, start + w, e.tokens[w]) for w in e.want]
        self.manager.check()
        return rows


def next_token(rows, samplers):
    """'Samples' token = (last input token + 1) % 100: generation is a counter, easy to check."""
    return [(tok + 1) % 100 for _, _, tok in rows]


def make(pages=8, max_num_seqs=4, budget=16, **kw):
    r = FakeRunner(pages=pages, **kw)
    return r, RequestScheduler(r, max_num_seqs=max_num_seqs, max_tokens_per_step=budget, sample_fn=next_token)


def test_prompt_is_cut_under_the_token_budget_and_decodes_follow():
    r, s = make(pages=16, budget=5)
    rid = s.submit(list(range(10, 22)), max_new_tokens=3)          # 12 prompt tokens
    assert s.step() and r.steps[-1] == [(rid, 5, [])]
    assert s.step() and r.steps[-1] == [(rid, 5, [])]
    assert s.step() and r.steps[-1] == [(rid, 2, [1])]              # last portion: logits wanted at its end
    assert s.requests[rid].status == RequestStatus.Decoding and s.requests[rid].output_tokens == [22]
    assert s.step() and r.steps[-1] == [(rid, 1, [0])]
    assert s.step()
    (done,) = s.get_finished()
    assert done.output_tokens == [22, 23, 24] and done.finish_reason == "length" and done.num_generated == 3
    assert not s.has_pending() and not s.step()
    assert r.manager.num_free_pages("g") == 16


def test_decodes_go_first_and_prompts_fill_the_rest():
    r, s = make(pages=32, budget=8)
    a = s.submit([1, 2, 3], max_new_tokens=10)
    s.step()                                                        # a prefilled, now decoding
    b = s.submit(list(range(20)), max_new_tokens=2)
    s.step()
    assert r.steps[-1] == [(a, 1, [0]), (b, 7, [])]                 # 1 decode + 7 of b's prompt = budget 8
    s.step()
    assert r.steps[-1] == [(a, 1, [0]), (b, 7, [])]
    s.step()
    assert r.steps[-1] == [(a, 1, [0]), (b, 6, [5])]


def test_admission_is_fifo_and_bounded_by_max_num_seqs():
    r, s = make(pages=32, max_num_seqs=2, budget=64)
    ids = [s.submit([5, 6, 7], max_new_tokens=2) for _ in range(4)]
    s.step()
    assert [e[0] for e in r.steps[-1]] == ids[:2] and s.num_waiting() == 2 and s.num_active() == 2
    s.step()                                                        # both finish (2 tokens each)
    assert sorted(x.request_id for x in s.get_finished()) == ids[:2]
    s.step()
    assert [e[0] for e in r.steps[-1]] == ids[2:]
    s.run()
    assert r.manager.num_free_pages("g") == 32


def test_finish_reasons():
    r, s = make(pages=16)
    a = s.submit([10], max_new_tokens=50, eos_token_id=13)
    b = s.submit([20], max_new_tokens=50, stop_token_ids=[24])
    c = s.submit([30], max_new_tokens=2)
    done = {x.request_id: x for x in s.run()}
    assert (done[a].finish_reason, done[a].output_tokens) == ("eos", [11, 12, 13])
    assert (done[b].finish_reason, done[b].output_tokens) == ("stop", [21, 22, 23, 24])
    assert (done[c].finish_reason, done[c].output_tokens) == ("length", [31, 32])
    assert all(x.status == RequestStatus.Finished for x in done.values())


def test_abort_frees_pages():
    r, s = make(pages=8)
    a = s.submit([1] * 9, max_new_tokens=20)
    s.step()
    assert r.manager.num_free_pages("g") == 5
    s.abort(a)
    (x,) = s.get_finished()
    assert x.status == RequestStatus.Failed and x.finish_reason == "aborted"
    assert r.manager.num_free_pages("g") == 8 and not s.has_pending()


def test_pages_run_out_youngest_is_preempted_and_recomputed():
    # 6 pages of 4 tokens.  a and b each take 2 pages for their 8-token prompts, then decode: each needs a
    # 3rd page after 1 token (fine: 6 pages), and a 4th after 5 tokens: not both.
    r, s = make(pages=6, budget=64)
    a = s.submit(list(range(8)), max_new_tokens=12)
    b = s.submit(list(range(50, 58)), max_new_tokens=12)
    done = {x.request_id: x for x in s.run()}
    assert s.num_preemptions >= 1 and done[b].num_preemptions >= 1 and done[a].num_preemptions == 0
    # preemption does not change what is generated
    assert done[a].output_tokens == list(range(8, 20)) and done[b].output_tokens == list(range(58, 70))
    assert done[a].finish_reason == done[b].finish_reason == "length"
    # b's recompute step fed prompt + generated tokens as one prompt
    assert any(e[0] == b and e[1] > 8 for step in r.steps for e in step)
    assert r.manager.num_free_pages("g") == 6
    r.manager.check()


def test_a_request_that_cannot_fit_alone_fails_cleanly():
    r, s = make(pages=3, budget=64, max_positions=64)
    a = s.submit(list(range(10)), max_new_tokens=20)               # needs 8 pages in the end, pool has 3
    (x,) = s.run()
    assert x.status == RequestStatus.Failed and x.finish_reason == "error:out_of_pages"
    assert x.output_tokens == [10, 11, 12]                          # what fit was generated
    assert r.manager.num_free_pages("g") == 3
    with pytest.raises(ValueError, match="never fit"):
        s.submit(list(range(13)), max_new_tokens=1)


def test_submit_refuses_bad_requests():
    r, s = make()
    with pytest.raises(ValueError, match="empty"):
        s.submit([])
    with pytest.raises(ValueError, match="outside"):
        s.submit([100])
    with pytest.raises(ValueError, match="positions"):
        s.submit([1] * 10, max_new_tokens=56)
    with pytest.raises(ValueError, match="positive"):
        s.submit([1], max_new_tokens=0)


def test_prompt_portion_shrinks_to_the_free_pages():
    r, s = make(pages=4, budget=64)
    a = s.submit(list(range(8)), max_new_tokens=4)                  # 2 pages, then a 3rd while decoding
    s.step()
    b = s.submit(list(range(20, 31)), max_new_tokens=1)             # 11 tokens = 3 pages; only 2 free after a's decode
    s.step()
    assert r.steps[-1] == [(a, 1, [0]), (b, 4, [])]                  # a's decode took a page; one page for b
    r.manager.check()
    done = {x.request_id: x for x in s.run()}
    assert done[a].output_tokens == [8, 9, 10, 11] and done[b].output_tokens == [31]


def test_xorshift_matches_the_reference_recurrence():
    g = XorShift64(0)
    assert g.state == 12345
    x = 12345
    for _ in range(5):
        x ^= (x << 13) & (2**64 - 1)
        x ^= x >> 7
        x ^= (x << 17) & (2**64 - 1)
        assert g.uniform() == float(x & 0x7FFFFFFF) / float(0x7FFFFFFF)
    assert XorShift64(7).state == 7
    assert SamplerConfig(temperature=0.0).greedy and SamplerConfig(do_sample=False).greedy
    assert not SamplerConfig(temperature=0.8).greedy


# ------------------------------------------------------------------ decoding one step ahead of the host
class FakeAheadRunner(FakeRunner):
    """A runner whose decode steps hand back a handle instead of tokens, and that can take a step's input
    tokens from the previous step's outputs 'on the device'."""
    cuda_graphs = True

    def __init__(self, **kw):
        super().__init__(**kw)
        self.device_tokens = None
        self.from_previous = 0
        self.sampling = []

    def validate(self, entries):
        assert len({e.req_id for e in entries}) == len(entries)

    def decode_step_async(self, entries, from_previous=False, sampling=None):
        self.sampling.append(sampling)
        toks = [e.tokens[0] for e in entries]
        if from_previous:
            assert self.device_tokens is not None and len(self.device_tokens) == len(entries)
            toks = self.device_tokens
            self.from_previous += 1
        self.steps.append([(e.req_id, 1, [0]) for e in entries])
        for e in entries:
            self.manager.append(e.req_id, 1)
        self.manager.check()
        out = self.device_tokens = [(t + 1) % 100 for t in toks]
        return SimpleNamespace(tokens=lambda: list(out))

    def decode_step(self, entries):
        # one-token prompts look like decode steps to the runner; requests that are decoding never come here
        assert all(self.manager.num_tokens(e.req_id) == 0 for e in entries)
        return self.step(entries), None


GREEDY = SamplerConfig(do_sample=False)


def run_both(submissions, late=(), **kw):
    """The same requests through the plain and the run-ahead scheduler; ``late``: (after step, submission)."""
    results = []
    for cls in (FakeRunner, FakeAheadRunner):
        r = cls(**{k: v for k, v in kw.items() if k in ("pages", "page_size", "max_requests", "max_positions")})
        s = RequestScheduler(r, max_num_seqs=kw.get("max_num_seqs", 4), max_tokens_per_step=kw.get("budget", 64),
                             sample_fn=next_token)
        for sub in submissions:
            s.submit(sampler_config=GREEDY, **sub)
        n = 0
        while s.has_pending():
            assert s.step()
            n += 1
            for after, sub in late:
                if after == n:
                    s.submit(sampler_config=GREEDY, **sub)
        done = {x.request_id: (x.output_tokens, x.finish_reason, x.status) for x in s.get_finished()}
        assert r.manager.num_free_pages("g") == kw.get("pages", 8)
        r.manager.check()
        results.append((done, r, s))
    return results


def test_running_ahead_gives_the_same_tokens_and_reasons():
    subs = [dict(prompt_tokens=[10], max_new_tokens=30, eos_token_id=17),
            dict(prompt_tokens=[20, 21], max_new_tokens=9),
            dict(prompt_tokens=[40], max_new_tokens=30, stop_token_ids=[52]),
            dict(prompt_tokens=[60, 61, 62], max_new_tokens=25)]
    (plain, _, _), (ahead, r, s) = run_both(subs, pages=32)
    assert ahead == plain and len(ahead) == 4
    assert r.from_previous >= 10                      # most decode steps took their tokens from the device
    # an eos costs one dropped token: request 0 (a one-token prompt, so every step it is in brings one token)
    # was in one more step than it has tokens
    in_steps = sum(1 for step in r.steps for e in step if e[0] == 0)
    assert in_steps == len(ahead[0][0]) + 1


def test_sampling_requests_run_ahead_too_with_their_own_uniform_numbers():
    """Temperature / top-k / top-p need nothing from the host but a uniform number, which the request's generator
    gives when the step is launched: such requests run ahead like greedy ones, each row with its own parameters (a
    greedy row beside them keeps its argmax); a repeat penalty needs the history on the host and waits for its tokens."""
    r = FakeAheadRunner(pages=32)
    s = RequestScheduler(r, max_num_seqs=4, max_tokens_per_step=64, sample_fn=next_token)
    a = s.submit(prompt_tokens=[10], max_new_tokens=8, sampler_config=SamplerConfig(temperature=0.8, top_k=40, top_p=0.9, seed=3))
    b = s.submit(prompt_tokens=[20], max_new_tokens=8, sampler_config=GREEDY)
    c = s.submit(prompt_tokens=[30], max_new_tokens=8, sampler_config=SamplerConfig(temperature=0.5, seed=4))
    done = {x.request_id: x for x in s.run()}
    assert all(len(done[i].output_tokens) == 8 for i in (a, b, c))
    assert r.from_previous >= 4
    given = [x for x in r.sampling if x is not None]
    assert len(given) >= 5
    want_a, want_c = XorShift64(3), XorShift64(4)
    for step in given:
        (ta, ka, pa, ua, ga, na), (tb, kb, pb, ub, gb, nb), (tc, kc, pc, uc, gc, nc) = step
        assert (ta, ka, pa, ga, na) == (0.8, 40, 0.9, False, 1.0) and ua == want_a.uniform()
        assert gb and kb == 1
        assert (tc, kc, pc, gc, nc) == (0.5, 0, 1.0, False, 1.0) and uc == want_c.uniform()
    # with a repeat penalty in the batch nothing runs ahead on a runner that keeps no history on the device
    r2 = FakeAheadRunner(pages=32)
    s2 = RequestScheduler(r2, max_num_seqs=4, max_tokens_per_step=64, sample_fn=next_token)
    s2.submit(prompt_tokens=[10], max_new_tokens=6, sampler_config=SamplerConfig(temperature=0.8, repeat_penalty=1.1))
    r2.decode_step = lambda entries: (r2.step(entries), None)
    s2.run()
    assert r2.sampling == [] and r2.from_previous == 0
    # and on one that does, it runs ahead: the histories go along with the first step of a run, and only then
    r3 = FakeAheadRunner(pages=32)
    r3.device_history = True
    r3.histories = []
    plain_async = r3.decode_step_async

    def with_history(entries, from_previous=False, sampling=None, history=None):
        r3.histories.append(None if history is None else [None if h is None else dict(h) for h in history])
        return plain_async(entries, from_previous=from_previous, sampling=sampling)
    r3.decode_step_async = with_history
    s3 = RequestScheduler(r3, max_num_seqs=4, max_tokens_per_step=64, sample_fn=next_token)
    s3.submit(prompt_tokens=[10], max_new_tokens=7, sampler_config=SamplerConfig(temperature=0.8, repeat_penalty=1.1))
    s3.submit(prompt_tokens=[50], max_new_tokens=7, sampler_config=GREEDY)
    done3 = s3.run()
    assert all(len(x.output_tokens) == 7 for x in done3) and r3.from_previous >= 3
    given3 = [h for h in r3.histories if h is not None]
    assert len(given3) >= 1 and given3[0][1] is None and isinstance(given3[0][0], dict)      # the penalised row's history only
    assert r3.histories[1] is None                                                              # the run's later steps bring none
    assert all(step[0][5] == 1.1 and step[1][5] == 1.0 for step in r3.sampling if step is not None)


def test_running_ahead_waits_before_admissions_and_when_pages_run_short():
    subs = [dict(prompt_tokens=list(range(8)), max_new_tokens=12),
            dict(prompt_tokens=list(range(50, 58)), max_new_tokens=12)]
    late = [(4, dict(prompt_tokens=[90, 91], max_new_tokens=5))]
    (plain, _, sp), (ahead, r, sa) = run_both(subs, late=late, pages=6, budget=64)
    assert ahead == plain and len(ahead) == 3
    assert sa.num_preemptions >= 1 and sa.num_preemptions == sp.num_preemptions


def test_abort_while_a_step_is_in_flight():
    r = FakeAheadRunner(pages=16)
    s = RequestScheduler(r, max_num_seqs=4, max_tokens_per_step=64, sample_fn=next_token)
    a = s.submit([10], max_new_tokens=20, sampler_config=GREEDY)
    b = s.submit([30], max_new_tokens=6, sampler_config=GREEDY)
    for _ in range(3):
        s.step()
    s.abort(a)
    done = {x.request_id: x for x in s.run()}
    assert done[a].finish_reason == "aborted" and done[b].output_tokens == [31, 32, 33, 34, 35, 36]
    assert r.manager.num_free_pages("g") == 16


def test_logger_gets_a_line_per_step_at_debug_level():
    """forge.Logger in the reference's manner: levels 0..5, a Python sink; at debug the scheduler reports each step."""
    import forge_b200 as forge
    lines = []
    forge.Logger.set_python_sink(lambda level, msg: lines.append((level, msg)))
    forge.Logger.set_level(4)
    try:
        runner, sched = make(pages=64, budget=16)
        sched.submit([1] * 20, max_new_tokens=3)
        sched.run()
    finally:
        forge.Logger.set_level(2)
        forge.Logger.reset_sink()
    steps = [m for lv, m in lines if lv == 4 and m.startswith("step ")]
    assert len(steps) == sched.num_steps and "16 tokens (0 decodes, 1 portions)" in steps[0] and "free pages" in steps[0]
    assert forge.Logger.level() == 2
    with pytest.raises(ValueError):
        forge.Logger.set_level(9)
