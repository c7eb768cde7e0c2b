"""The step function: one call runs one batch of (request, its next tokens) through the model, from the
cache that earlier steps left, and returns the logits at the wanted places.

``ModelRunner`` owns the model, the cache storage and the cache manager.  Callers (the scheduler, the
replay tool, tests) admit a request, feed it tokens over any number of steps, cut anywhere, and release
it; the runner makes no scheduling decision of its own.  (Reference counterparts:
InferenceEngine::forward / forward_batch, include/forge/engine.h:65-90.)
"""
import os

import torch

from ..cache import CacheStorage, OutOfPages, bytes_per_page
from ..config import load_config
from ..parts import Runtime
from ..parts.base import is_graph_safe
from ..weights.loader import load_tensors
from .batch import StepEntry, build_step_batch, layout_step
from .decode_graph import DecodeGraph
from .model import Model

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


class StepError(ValueError):
    """The step was refused before anything ran (bad token id, position limit, unknown request)."""


def resolve_dtype(dtype):
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype}")
        return dtype
    try:
        return DTYPES[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {dtype!r}") from None


class ModelRunner:
    def __init__(self, model_dir=None, *, config=None, tensors=None, dtype="bfloat16", device="cuda:0",
                 page_size=64, cache_tokens=None, max_requests=8, memory_fraction=0.6, cuda_graphs=True,
                 max_tokens_per_step=None, max_decode_graphs=16, fused_decode=None):
        """Either ``model_dir`` (config.json + safetensors) or ``config`` + ``tensors`` ({file name: tensor}).
        ``cache_tokens``: capacity of every cache group in tokens (default: what ``memory_fraction`` of the
        free device memory holds, capped by max_requests * max positions).  ``cuda_graphs``: replay decode
        steps as CUDA graphs where every part of the model allows it (``Part.graph_safe``); a model with a part
        that does not takes the ordinary step, whatever this says.  ``max_tokens_per_step``: a step with more
        tokens is refused (None: no limit); the step's activations live in a workspace of that many rows.
        ``fused_decode``: run all layers of a decode step of up to 16 requests in one persistent kernel where the
        model allows it (None: only if FORGE_FUSED_DECODE=1; it is the slower path at the sizes measured).
        ``max_decode_graphs``: how many captured graphs (one per batch size and context bucket) are kept; the
        one used longest ago goes first."""
        if not torch.cuda.is_available():
            raise RuntimeError("forge_b200 runs on a CUDA device (B200, sm_100a) only; no device is visible")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.dtype = resolve_dtype(dtype)
        self.rt = Runtime(self.device, self.dtype)
        if config is None:
            if model_dir is None:
                raise ValueError("give a model folder, or a config and tensors")
            config = load_config(model_dir)
        self.config = config
        self.plan = config.plan()
        self.model = Model(self.plan, self.rt)
        if tensors is None:
            tensors = load_tensors(model_dir, self.model.tensor_specs())
        else:
            from ..weights.loader import check_tensors
            check_tensors("tensors", self.model.tensor_specs(), {n: (tuple(t.shape), t.dtype) for n, t in tensors.items()})
        self.model.load(tensors, where=str(model_dir or "tensors"))
        del tensors
        from .. import log
        log.info(f"model loaded: {type(config).__name__}, {len(self.plan.layers)} layers, hidden {self.plan.hidden_size}, "
                 f"vocabulary {self.plan.vocab_size}, {self.dtype}")

        self.page_size, self.max_requests = int(page_size), int(max_requests)
        specs, cfrom = self.model.cache_specs(), self.model.cache_from()
        if cache_tokens is None:
            per_page = max(bytes_per_page(specs, cfrom, self.page_size, self.dtype).values(), default=0)
            free, _ = torch.cuda.mem_get_info(self.device)
            cap = self.max_requests * self.plan.max_positions
            cache_tokens = cap if per_page == 0 else min(cap, int(free * memory_fraction) // per_page * self.page_size)
        self.num_pages = max(1, -(-int(cache_tokens) // self.page_size))
        self.storage = CacheStorage(specs, cfrom, self.page_size, self.num_pages, self.max_requests, self.dtype,
                                    self.device)
        self.manager = self.storage.manager
        # width of a request's block table.  A group that keeps every key can never give a request more
        # pages than its pool has; a windowed group hands old pages back but its table keeps its logical
        # length (-1 where a page went), so it must reach the model's last position.
        self.max_pages_per_request = -(-self.plan.max_positions // self.page_size)
        if all(g.window is None for g in self.manager.groups.values()):
            self.max_pages_per_request = min(self.num_pages, self.max_pages_per_request)
        self.max_tokens_per_step = None if max_tokens_per_step is None else int(max_tokens_per_step)
        # Decode steps of up to 16 requests can run all their layers in ONE persistent kernel (csrc/decode_layers.cu).
        # Measured on B200 at TinyLlama widths it is correct but slower than one kernel per operation (1.07 ms
        # against 0.79 ms for the 22 layers at batch 8: five grid barriers a layer and the per-CTA conversion of
        # the token operand cost more than the seven kernel hand-overs they replace), so it is off unless asked
        # for (fused_decode=True or FORGE_FUSED_DECODE=1).
        want = fused_decode if fused_decode is not None else os.environ.get("FORGE_FUSED_DECODE", "0") == "1"
        self.fused_decode = bool(want) and self.model.enable_fused_decode(self.storage.layers, self.max_requests)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        # Outputs of a step's kernels are views into one buffer that is as large as the largest step so far needed
        # (one layer's intermediates at max_tokens_per_step, if that is given, plus the step's integers): after the
        # first step of the largest size no step asks the allocator for anything but the logits it hands out.
        from .. import kernels
        self.workspace = kernels.StepWorkspace(self.device)
        # FORGE_CHECKS=1: kernels test every page id, slot and token index before use (csrc/checks.cuh)
        self.first_bad = torch.zeros(3, dtype=torch.int32, device=self.device) if kernels.checks_enabled() else None
        # decode steps replay a captured graph only if every part of the model says that it may be captured
        self.graph_safe = self.model.graph_safe()
        self._cuda_graphs = bool(cuda_graphs) and self.graph_safe
        self.max_decode_graphs = max(1, int(max_decode_graphs))
        self._decode_graphs = {}
        self._last_greedy = None
        self._token_rings = {}

    @property
    def cuda_graphs(self):
        """Whether decode steps replay a captured graph now: the runner was made so, the model allows it, and the
        per-kernel timing (kernels.profiler_enable) is off."""
        from .. import kernels
        return self._cuda_graphs and not kernels.profiler_enabled()

    @cuda_graphs.setter
    def cuda_graphs(self, on):
        self._cuda_graphs = bool(on) and self.graph_safe

    # ---------------------------------------------------------------------------------- requests
    def admit(self, req_id):
        return self.manager.admit(req_id)

    def release(self, req_id):
        self.manager.free(req_id)

    def is_live(self, req_id):
        return req_id in self.manager.live_requests()

    # ---------------------------------------------------------------------------------- the step
    def validate(self, entries):
        V, limit = self.plan.vocab_size, self.plan.max_positions
        live = set(self.manager.live_requests())
        seen = set()
        total = sum(len(e.tokens) for e in entries)
        if self.max_tokens_per_step is not None and total > self.max_tokens_per_step:
            raise StepError(f"the step brings {total} tokens, the runner was made for {self.max_tokens_per_step} a step")
        for e in entries:
            if e.req_id not in live:
                raise StepError(f"request {e.req_id!r} was not admitted")
            if e.req_id in seen:
                raise StepError(f"request {e.req_id!r} appears twice in one step")
            seen.add(e.req_id)
            if not e.tokens:
                raise StepError(f"request {e.req_id!r} brings no tokens")
            if not set(map(type, e.tokens)) <= {int} or min(e.tokens) < 0 or max(e.tokens) >= V:
                bad = next((t for t in e.tokens if type(t) is not int or not 0 <= t < V), e.tokens[0])
                raise StepError(f"request {e.req_id!r}: token id {bad!r} is outside [0, {V})")
            after = self.manager.num_tokens(e.req_id) + len(e.tokens)
            if after > limit:
                raise StepError(f"request {e.req_id!r} would exceed the model's {limit} positions")
            if -(-after // self.page_size) > self.max_pages_per_request:
                raise OutOfPages(f"request {e.req_id!r} would hold {-(-after // self.page_size)} pages; block tables "
                                 f"have room for {self.max_pages_per_request}")

    def step(self, entries):
        """entries: list of StepEntry.  Runs exactly the tokens given, as one batch; returns fp32 logits
        [number of wanted places, vocab] on the device in the order of the entries and of their ``want``
        (None if nothing is wanted).  The tensor is the caller's: no later step writes into it.  Raises
        StepError / OutOfPages before anything has run."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        self.validate(entries)
        if self.cuda_graphs and all(len(e.tokens) == 1 and e.want == [0] for e in entries):
            # the graph's own logits buffer is rewritten by the next replay: hand out a copy
            return self.decode_step(entries)[0].clone()
        if self.first_bad is not None:
            from .. import kernels
            kernels.configure_checks(self.num_pages, self.page_size, sum(len(e.tokens) for e in entries), self.status, self.first_bad)
        from .. import kernels as _k
        _k.profiler_step_begin()
        with self.workspace.step() as ws:
            batch = build_step_batch(entries, self.manager, self.device, self.max_pages_per_request, status=self.status)
            self.storage.zero_state_slots(self.manager.take_fresh_slots())
            logits = self.model.forward(batch, self.storage.layers, workspace=ws)
        for e in entries:
            self.manager.release_out_of_window(e.req_id)
        return logits

    def decode_step(self, entries, tokens_on_device=False):
        """One token for each entry, logits wanted for all: replays the CUDA graph captured for this number
        of requests.  Returns (logits [S,V], greedy tokens int32 [S]); both are overwritten by the next
        decode step of the same size.  Entries must have been validated.  ``tokens_on_device``: the
        entries' token ids are placeholders; the step consumes the previous decode step's greedy tokens
        straight from device memory."""
        S = len(entries)
        # graphs are kept per (batch size, context bucket): the key slicing of the decode attention is part of
        # the graph, and slicing for 32k tokens when the longest request holds 500 wastes CTAs and merge work
        longest = max(self.manager.num_tokens(e.req_id) for e in entries) + 1
        bucket = 256
        while bucket < longest:
            bucket *= 2
        bucket = min(bucket, self.plan.max_positions)
        if not self.graph_safe:
            raise StepError("this model has a part that may not be captured in a CUDA graph; use step()")
        g = self._decode_graphs.pop((S, bucket), None)
        if g is None:
            while len(self._decode_graphs) >= self.max_decode_graphs:      # the one used longest ago goes
                self._decode_graphs.pop(next(iter(self._decode_graphs)))
                self._last_greedy = None
            g = DecodeGraph(self, S, max_context=bucket)
        self._decode_graphs[(S, bucket)] = g                               # most recently used last
        if self.first_bad is not None:
            from .. import kernels
            kernels.configure_checks(self.num_pages, self.page_size, S, self.status, self.first_bad)
        hs = layout_step(entries, self.manager)
        self.storage.zero_state_slots(self.manager.take_fresh_slots())
        prev = self._last_greedy if tokens_on_device else None
        if prev is not None and prev.numel() != S:
            raise StepError("tokens_on_device needs a previous decode step of the same batch size")
        out = g.run(hs, tokens_from=prev)
        self._last_greedy = out[1]
        for e in entries:
            self.manager.release_out_of_window(e.req_id)
        return out

    device_history = True      # repeat penalties can be applied from a history kept on the device (decode_step_async)

    def decode_step_async(self, entries, from_previous=False, sampling=None, history=None):
        """decode_step whose tokens are not waited for: returns a handle whose ``tokens()`` blocks until the step has
        run and gives them as a list.  ``from_previous``: take the input tokens from the previous decode step's
        tokens on the device (the entries' token ids are placeholders).  ``sampling``: None, the tokens are the
        greedy ones of the graph; or one (temperature, top_k, top_p, u, greedy, repeat_penalty) per entry: rows that
        are not greedy draw their token on the device with the uniform number u that the request's generator gave (the
        sampling kernel of ``forge_b200.sampling``, so a request draws what it would draw with its logits on the host).
        Rows with a repeat penalty are penalised from a history of generated tokens that is kept on the device, one row
        of counts per request slot, and the step adds its token to it; ``history`` (one Counter or None per entry)
        replaces the slots' rows first: the caller gives it when the host's histories are complete, i.e. at the first
        of a run of such steps."""
        logits, greedy = self.decode_step(entries, tokens_on_device=from_previous)
        S = greedy.numel()
        ring = self._token_rings.get(S)
        if ring is None:
            # a handle is read at the latest after the NEXT step has been launched: four buffers are plenty
            ring = self._token_rings[S] = {"bufs": [torch.empty(S, dtype=torch.int32, pin_memory=True) for _ in range(4)],
                                           "events": [torch.cuda.Event() for _ in range(4)], "pos": 0,
                                           "params": [torch.empty(6, S, dtype=torch.float32, pin_memory=True) for _ in range(4)],
                                           "params_dev": torch.empty(6, S, dtype=torch.float32, device=self.device),
                                           "drawn": [torch.empty(S, dtype=torch.int32, device=self.device) for _ in range(2)]}
        i = ring["pos"]
        ring["pos"] = (i + 1) % len(ring["bufs"])
        chosen = greedy
        penalised = sampling is not None and any(pen != 1.0 for *_, pen in sampling)
        if sampling is not None and (penalised or not all(g for _, _, _, _, g, _ in sampling)):
            from .. import kernels
            host = ring["params"][i]                    # free: its handle was read before this slot came round again
            host[0] = torch.tensor([t for t, *_ in sampling])
            host[1] = torch.tensor([p for _, _, p, *_ in sampling])
            host[2] = torch.tensor([u for _, _, _, u, *_ in sampling])
            host[3].view(torch.int32).copy_(torch.tensor([k for _, k, *_ in sampling], dtype=torch.int32))
            host[4] = torch.tensor([pen for *_, pen in sampling])
            host[5].view(torch.int32).copy_(torch.tensor([self.manager.slot(e.req_id) for e in entries], dtype=torch.int32))
            dev = ring["params_dev"]
            dev.copy_(host, non_blocking=True)
            slots_dev = dev[5].view(torch.int32)
            if penalised:
                counts = self._history_counts(logits.shape[1])
                if history is not None:
                    for e, h in zip(entries, history):
                        if h is not None:
                            row = counts[self.manager.slot(e.req_id)]
                            row.zero_()
                            if h:
                                row[torch.tensor(list(h.keys()), device=self.device)] = \
                                    torch.tensor(list(h.values()), dtype=torch.int32, device=self.device)
                kernels.history_penalty(logits, counts, slots_dev, dev[4])
                greedy = kernels.argmax(logits)         # of the penalised logits
            all_greedy = all(g for _, _, _, _, g, _ in sampling)
            chosen = ring["drawn"][i % 2]
            if all_greedy:
                chosen.copy_(greedy)
            else:
                kernels.sample(logits, dev[0], dev[3].view(torch.int32), dev[1], dev[2], out=chosen)
                if any(g for _, _, _, _, g, _ in sampling):      # greedy rows keep the argmax (lowest index wins a tie)
                    mask = torch.tensor([bool(g) for _, _, _, _, g, _ in sampling]).to(self.device, non_blocking=True)
                    torch.where(mask, greedy, chosen, out=chosen)
            if penalised:
                kernels.history_add(counts, slots_dev, chosen, dev[4])
            self._last_greedy = chosen                  # what the next step takes its input tokens from
        ring["bufs"][i].copy_(chosen, non_blocking=True)
        ring["events"][i].record()
        return PendingTokens(ring["bufs"][i], ring["events"][i])

    def _history_counts(self, vocab):
        """int32 [request slots, vocabulary]: how often each request has generated each token (made at first use)."""
        if getattr(self, "_history", None) is None:
            self._history = torch.zeros(self.manager.max_requests, vocab, dtype=torch.int32, device=self.device)
        return self._history

    def check_status(self):
        """Reads the device error word (synchronises); raises if a kernel flagged a problem."""
        from .. import kernels
        try:
            kernels.check_kernel_status(self.device)      # tensor-core kernels: a bounded wait that ran out
        except kernels.KernelError:
            if self.model._fused is not None:
                self.model._fused[0].reset_after_error()
            raise
        overrun = self.storage.check_canaries() + ([] if self.workspace.canary_intact() else ["the step workspace (behind it)"])
        if overrun:
            raise RuntimeError("canary words were overwritten, a kernel wrote outside its tensor: " + "; ".join(overrun))
        s = int(self.status.item())
        if s:
            self.status.zero_()
            raise RuntimeError(f"a kernel reported an error (status word {s:#x}): "
                               + ("token id outside the vocabulary; " if s & 1 else "")
                               + ("a bounded wait ran out; " if s & 2 else "")
                               + (self._bad_index() if s & 16 else ""))

    def _bad_index(self):
        kind, value, limit = self.first_bad.tolist() if self.first_bad is not None else (0, 0, 0)
        self.first_bad.zero_() if self.first_bad is not None else None
        what = {1: "page id", 2: "cache slot", 3: "token index"}.get(kind, "index")
        return f"a kernel was given a {what} outside its range: {value} (limit {limit}); "


class PendingTokens:
    """The tokens of a decode step on their way to pinned host memory."""

    def __init__(self, host, event):
        self.host, self.event = host, event

    def tokens(self):
        self.event.synchronize()
        return self.host.tolist()


__all__ = ["ModelRunner", "PendingTokens", "StepEntry", "StepError", "OutOfPages", "resolve_dtype"]
