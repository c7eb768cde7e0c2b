"""Continuous batching above the step function: admits requests, cuts prompts into portions under a token
budget, decodes one token per running request per step, finishes and frees.

Names and meanings follow the reference's RequestScheduler (include/forge/request_scheduler.h:17-53,
src/inference/request_scheduler.cpp:157-416): submit / step / get_finished / has_pending / abort / reset,
requests Waiting -> Prefilling -> Decoding -> Finished | Failed with finish_reason "eos" | "stop" | "length"
| "aborted" | "error:...".  What differs, on purpose:
  * a prompt is cut into portions so that no step exceeds ``max_tokens_per_step`` (the reference hands the
    whole prompt to one step, :238-244); portions of prompts run beside single decoded tokens;
  * admission needs a free request slot AND free pages for the portion (the reference looks only at how
    full layer 0 is, :386-416);
  * when pages run out, the most recently admitted running request is PREEMPTED: its pages go back, its
    prompt plus the tokens it has generated become the prompt to recompute, and it returns to the front of
    the queue; a request that cannot make progress even alone fails with "error:out_of_pages" (the
    reference logs "cache overflow" and carries on, src/inference/kv_cache.cpp:629-633);
  * every request has its own sampler state;
  * decoding runs one step AHEAD of the host: while the same requests keep decoding, step k is launched with its
    input tokens taken on the device from step k-1's tokens (the argmax of the graph, or the draw of the sampling
    kernel with the uniform number that the request's generator gave at launch), and only then are step k-1's
    tokens read and handed to their requests.  A repeat penalty is applied from a history of generated tokens
    that the runner keeps on the device (uploaded from the host's at the first of a run of such steps).  A request that turns out to have ended (eos, a stop token) has then computed
    one token too many, which is dropped; anything else that would change the batch (a request about to reach
    its length, an admission, pages running short) first waits for the step in flight.
"""
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, List, Optional

from .. import log
from ..cache import OutOfPages
from ..sampling import RequestSampler, SamplerConfig
from .batch import StepEntry


class RequestStatus(Enum):
    Waiting = 0
    Prefilling = 1
    Decoding = 2
    Finished = 3
    Failed = 4


@dataclass
class GenerateRequest:
    request_id: int
    prompt_tokens: List[int]
    max_new_tokens: int = 256
    eos_token_id: int = -1
    sampler_config: SamplerConfig = field(default_factory=SamplerConfig)
    stop_token_ids: List[int] = field(default_factory=list)
    status: RequestStatus = RequestStatus.Waiting
    output_tokens: List[int] = field(default_factory=list)
    num_generated: int = 0
    current_pos: int = 0                 # tokens of this request that are in the cache
    finish_reason: str = ""
    num_preemptions: int = 0
    callback: Optional[Callable] = None  # callback(request_id, token_id, step, status)
    sampler: Optional[RequestSampler] = None

    def tokens_to_compute(self):
        """Everything that must be in the cache before the next token can be sampled: the prompt and all
        generated tokens (after a preemption those are recomputed like a prompt)."""
        return self.prompt_tokens + self.output_tokens


class RequestScheduler:
    def __init__(self, runner, max_num_seqs=4, max_tokens_per_step=2048, sample_fn=None):
        """runner: a ModelRunner (or anything with .manager, .plan, .admit, .release, .step).
        sample_fn(logits, samplers) -> token list; defaults to the device sampler."""
        self.runner = runner
        self.manager = runner.manager
        self.max_num_seqs = min(int(max_num_seqs), self.manager.max_requests)
        self.max_tokens_per_step = int(max_tokens_per_step)
        if self.max_num_seqs <= 0 or self.max_tokens_per_step <= 0:
            raise ValueError("max_num_seqs and max_tokens_per_step must be positive")
        if sample_fn is None:
            from ..sampling import sample_batch
            sample_fn = sample_batch
        self.sample_fn = sample_fn
        self.requests = {}
        self.waiting = deque()
        self.active = []                 # admission order
        self.finished = []
        self.next_request_id = 0
        self.num_steps = 0
        self.num_preemptions = 0
        self.last_step = None            # what the last step ran, for tests and logs
        self._inflight = None            # (requests, handle) of a decode step whose tokens have not been read yet

    # ------------------------------------------------------------------------------- public API
    def submit(self, prompt_tokens, max_new_tokens=256, eos_token_id=-1, sampler_config=None, callback=None,
               stop_token_ids=()):
        prompt = [int(t) for t in prompt_tokens]
        V, limit = self.runner.plan.vocab_size, self.runner.plan.max_positions
        if not prompt:
            raise ValueError("empty prompt")
        if max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be positive")
        bad = [t for t in prompt if not 0 <= t < V]
        if bad:
            raise ValueError(f"prompt token id {bad[0]} is outside [0, {V})")
        if len(prompt) + max_new_tokens - 1 > limit:
            raise ValueError(f"prompt of {len(prompt)} tokens plus {max_new_tokens} new ones exceeds the model's "
                             f"{limit} positions")
        total_pages = min(p.num_pages for p in self.manager.pools.values()) if self.manager.pools else None
        if total_pages is not None and -(-len(prompt) // self.manager.page_size) > total_pages:
            raise ValueError(f"prompt of {len(prompt)} tokens can never fit the cache "
                             f"({total_pages} pages of {self.manager.page_size})")
        cfg = sampler_config or SamplerConfig()
        rid = self.next_request_id
        self.next_request_id += 1
        self.requests[rid] = GenerateRequest(rid, prompt, int(max_new_tokens), int(eos_token_id), cfg,
                                             [int(t) for t in stop_token_ids], callback=callback,
                                             sampler=RequestSampler(cfg))
        self.waiting.append(rid)
        return rid

    def has_pending(self):
        return bool(self.waiting or self.active)

    def num_active(self):
        return len(self.active)

    def num_waiting(self):
        return len(self.waiting)

    def get_finished(self):
        out, self.finished = self.finished, []
        for r in out:
            self.requests.pop(r.request_id, None)
        return out

    def get_all_requests(self):
        return list(self.requests.values())

    def abort(self, request_id):
        r = self.requests.get(request_id)
        if r is None or r.status in (RequestStatus.Finished, RequestStatus.Failed):
            return
        self._finish(r, RequestStatus.Failed, "aborted")

    def reset(self):
        for rid in list(self.active):
            self.runner.release(rid)
        self.requests.clear()
        self.waiting.clear()
        self.active.clear()
        self.finished.clear()
        self._inflight = None

    # ------------------------------------------------------------------------------- one step
    def plan_step(self):
        """Decides what the next step runs.  Returns a list of (request, first token index, n tokens,
        wants_logits).  Frees and re-queues requests when pages run out; admits waiting requests."""
        mgr, budget = self.manager, self.max_tokens_per_step
        plan, reserve = [], {g: 0 for g in mgr.groups}

        def reserve_for(rid, n):
            need = mgr.pages_needed(rid, n)
            for g, k in need.items():
                reserve[g] += k

        # 1. one token for every decoding request, oldest first; preempt the youngest when pages run out
        for rid in list(self.active):
            if rid not in self.active:
                continue                                     # preempted below while serving an older one
            r = self.requests[rid]
            if r.status != RequestStatus.Decoding or budget <= 0:
                continue
            while not mgr.can_append(rid, 1, reserve):
                victim = self._youngest_other_than(rid, {p[0].request_id for p in plan})
                if victim is None:
                    break
                self._preempt(victim)
            if not mgr.can_append(rid, 1, reserve):
                if len(self.active) == 1 and not plan:
                    self._finish(r, RequestStatus.Failed, "error:out_of_pages")
                else:
                    self._preempt(rid)
                continue
            reserve_for(rid, 1)
            plan.append((r, r.current_pos, 1, True))
            budget -= 1

        # 2. portions of prompts: requests already admitted first, then the queue, in order
        def portion(r):
            nonlocal budget
            todo = r.tokens_to_compute()
            left = len(todo) - r.current_pos
            n = min(left, budget)
            # shrink to what the free pages hold
            while n > 0 and not mgr.can_append(r.request_id, n, reserve):
                room = min(mgr.num_free_pages(g) - reserve[g] for g in mgr.groups) if mgr.groups else n
                fit = max(0, room) * mgr.page_size + (-mgr.num_tokens(r.request_id)) % mgr.page_size
                n = min(n - 1, fit)
            if n <= 0:
                return False
            reserve_for(r.request_id, n)
            plan.append((r, r.current_pos, n, r.current_pos + n == len(todo)))
            budget -= n
            return True

        for rid in self.active:
            r = self.requests[rid]
            if r.status == RequestStatus.Prefilling and budget > 0:
                portion(r)
        while self.waiting and budget > 0 and len(self.active) < self.max_num_seqs and mgr.has_free_slot():
            rid = self.waiting[0]
            r = self.requests[rid]
            self.runner.admit(rid)
            r.status, r.current_pos = RequestStatus.Prefilling, 0
            if not portion(r):
                self.runner.release(rid)            # no page for even one token: stays waiting
                r.status = RequestStatus.Waiting
                break
            self.waiting.popleft()
            self.active.append(rid)

        if not plan and self.active:
            # nobody can move: every page is held by requests that all need more.  Give the youngest's back.
            victim = self.active[-1]
            if len(self.active) == 1:
                self._finish(self.requests[victim], RequestStatus.Failed, "error:out_of_pages")
            else:
                self._preempt(victim)
                return self.plan_step()
        return plan

    def step(self):
        """Runs one step.  Returns False when there was nothing to do."""
        handed_out = False
        if self._inflight is not None and not self._can_run_ahead():
            self._resolve_inflight()
            handed_out = True
        plan = self.plan_step()
        if not plan:
            if self._inflight is not None:
                self._resolve_inflight()
                return True
            return handed_out                             # reading the last step's tokens was work too
        ahead = self._plan_runs_ahead(plan)
        if self._inflight is not None and not (ahead and [p[0] for p in plan] == self._inflight[0]):
            self._resolve_inflight()                      # the plan is not the one the check above foresaw
            return self.step()
        entries, rows = [], []
        for r, start, n, wants in plan:
            if self._inflight is not None:
                toks = [0]                                # placeholder: the token is on the device
            elif r.status == RequestStatus.Decoding and n == 1:
                toks = [r.output_tokens[-1]]              # no need to rebuild prompt + outputs for one token
            else:
                toks = r.tokens_to_compute()[start:start + n]
            entries.append(StepEntry(r.request_id, toks, [n - 1] if wants else []))
            if wants:
                rows.append(r)
        self.last_step = [(r.request_id, start, n, wants) for r, start, n, wants in plan]
        decode_only = all(n == 1 and wants for _, _, n, wants in plan) and getattr(self.runner, "cuda_graphs", False)
        greedy = handle = None
        try:
            if ahead:
                self.runner.validate(entries)
                sampling = history = None
                if not all(self._greedy_only(r) for r in rows):
                    # the uniform number of a row that samples comes from the request's own generator, now, in the
                    # order in which the request's tokens are drawn; the draw itself happens on the device
                    sampling = [(1.0, 1, 1.0, 0.5, True, float(r.sampler.config.repeat_penalty)) if r.sampler.config.greedy else
                                (float(r.sampler.config.temperature), int(r.sampler.config.top_k), float(r.sampler.config.top_p),
                                 r.sampler.rng.uniform(), False, float(r.sampler.config.repeat_penalty)) for r in rows]
                    if self._inflight is None and any(r.sampler.config.repeat_penalty != 1.0 for r in rows):
                        # the first of a run of steps: the host's histories are complete and go to the device, which
                        # keeps them up to date itself from here on
                        history = [r.sampler.history if r.sampler.config.repeat_penalty != 1.0 else None for r in rows]
                if history is not None:
                    handle = self.runner.decode_step_async(entries, from_previous=False, sampling=sampling, history=history)
                else:
                    handle = self.runner.decode_step_async(entries, from_previous=self._inflight is not None, sampling=sampling)
            elif decode_only:
                self.runner.validate(entries)
                logits, greedy = self.runner.decode_step(entries)
            else:
                logits = self.runner.step(entries)
        except OutOfPages:
            raise                                         # plan_step reserved pages; this is a bug
        except Exception as e:                            # a failed step fails the requests that were in it
            self._inflight = None
            for r, _, _, _ in plan:
                self._finish(r, RequestStatus.Failed, f"error:{type(e).__name__}")
            raise
        self.num_steps += 1
        if log.Logger.enabled(log.DEBUG):
            decodes = sum(1 for _, _, n, w in plan if n == 1 and w)
            log.debug(f"step {self.num_steps}: {sum(n for _, _, n, _ in plan)} tokens ({decodes} decodes, {len(plan) - decodes} portions), "
                      f"{len(self.active)} running, {len(self.waiting)} waiting, free pages {self.manager.num_free_pages()}, "
                      f"{self.num_preemptions} preemptions, {'graph' if (ahead or decode_only) else 'eager'}")
        if self.num_steps % 256 == 0 and hasattr(self.runner, "check_status"):
            self.runner.check_status()                    # device error words, read now and then
        for r, start, n, wants in plan:
            r.current_pos = start + n
        if ahead:
            previous, self._inflight = self._inflight, (rows, handle)
            if previous is not None:
                self._hand_out(previous)
        elif rows:
            if greedy is not None and all(self._greedy_only(r) for r in rows):
                tokens = greedy.tolist()                  # argmax ran inside the decode graph
                for r, tok in zip(rows, tokens):
                    r.sampler.record(tok)
            else:
                tokens = self.sample_fn(logits, [r.sampler for r in rows])
            for r, tok in zip(rows, tokens):
                self._accept(r, int(tok))
        return True

    # ---------------------------------------------------------------------- running ahead of the host
    @staticmethod
    def _greedy_only(r):
        return r.sampler.config.greedy and r.sampler.config.repeat_penalty == 1.0

    def _drawn_on_device(self, r):
        """Greedy, or temperature / top-k / top-p sampling: the token can be chosen on the device from the logits and a
        uniform number known beforehand.  A repeat penalty needs the request's history: only a runner that keeps
        one on the device (``device_history``) can apply it without the host."""
        return r.sampler.config.repeat_penalty == 1.0 or getattr(self.runner, "device_history", False)

    def _plan_runs_ahead(self, plan):
        """A step of single decoded tokens whose choice needs nothing from the host but numbers known beforehand, on a
        runner that can leave the tokens on the device."""
        return (getattr(self.runner, "cuda_graphs", False) and hasattr(self.runner, "decode_step_async")
                and all(n == 1 and wants and r.status == RequestStatus.Decoding and self._drawn_on_device(r)
                        for r, _, n, wants in plan))

    def _can_run_ahead(self):
        """True if the next step is certainly the same requests as the one in flight, one more token each,
        whatever tokens that one produces (short of eos / stop, which cost one dropped token)."""
        rows = self._inflight[0]
        if self.active != [r.request_id for r in rows]:
            return False
        if self.waiting and len(self.active) < self.max_num_seqs and self.manager.has_free_slot():
            return False                                  # somebody could be admitted
        reserve = {g: 0 for g in self.manager.groups}
        for r in rows:
            if r.status != RequestStatus.Decoding or r.num_generated + 1 >= r.max_new_tokens:
                return False                              # gone, or its token in flight is its last
            if not self.manager.can_append(r.request_id, 1, reserve):
                return False                              # pages run short: plan_step must see final states
            for g, k in self.manager.pages_needed(r.request_id, 1).items():
                reserve[g] += k
        return True

    def _hand_out(self, inflight):
        rows, handle = inflight
        for r, tok in zip(rows, handle.tokens()):
            if r.status == RequestStatus.Decoding:        # not ended or aborted since the step was launched
                r.sampler.record(int(tok))
                self._accept(r, int(tok))

    def _resolve_inflight(self):
        inflight, self._inflight = self._inflight, None
        self._hand_out(inflight)

    def run(self):
        """Steps until no request is pending; returns the finished requests."""
        while self.has_pending():
            if not self.step():
                break
        self._inflight = None                             # what is left in flight belongs to ended requests
        if hasattr(self.runner, "check_status"):
            self.runner.check_status()
        return self.get_finished()

    # ------------------------------------------------------------------------------- internals
    def _accept(self, r, tok):
        r.output_tokens.append(tok)
        r.num_generated += 1
        r.status = RequestStatus.Decoding
        if r.callback:
            r.callback(r.request_id, tok, r.num_generated - 1, r.status)
        if r.eos_token_id >= 0 and tok == r.eos_token_id:
            self._finish(r, RequestStatus.Finished, "eos")
        elif tok in r.stop_token_ids:
            self._finish(r, RequestStatus.Finished, "stop")
        elif r.num_generated >= r.max_new_tokens:
            self._finish(r, RequestStatus.Finished, "length")

    def _finish(self, r, status, reason):
        rid = r.request_id
        if rid in self.active:
            self.active.remove(rid)
            self.runner.release(rid)
        elif rid in self.waiting:
            self.waiting.remove(rid)
        r.status, r.finish_reason = status, reason
        self.finished.append(r)
        if r.callback and status == RequestStatus.Failed:
            r.callback(rid, -1, r.num_generated, status)

    def _youngest_other_than(self, rid, planned):
        for cand in reversed(self.active):
            if cand != rid and cand not in planned:
                return cand
        return None

    def _preempt(self, rid):
        r = self.requests[rid]
        self.active.remove(rid)
        self.runner.release(rid)
        r.status, r.current_pos = RequestStatus.Waiting, 0
        r.num_preemptions += 1
        self.num_preemptions += 1
        log.info(f"request {rid} preempted ({len(r.output_tokens)} tokens generated so far): pages ran out")
        self.waiting.appendleft(rid)
