"""The decode step as a CUDA graph: one token for each of S requests, captured once per S and replayed.

A decode step is ~180 small kernel launches; launched one by one from Python they cost more than they
run.  The graph fixes every launch, so a step is: fill one pinned host buffer with the step's integers
(tokens, positions, slots, block tables), one host-to-device copy, one graph launch.  Greedy selection
(argmax) is part of the graph; the logits stay available for samplers that need them.
"""
import gc

import torch

from .. import kernels
from .batch import GroupBatch, StepBatch


class _OnDeviceOnly:
    """Stands where a batch keeps host copies of per-step numbers.  A graph is captured once and replayed for
    later steps, so a part that planned from host numbers would replay the captured step's; every use raises."""

    def __init__(self, what):
        self._what = what

    def _refuse(self, *a, **k):
        raise RuntimeError(f"StepBatch.{self._what} does not exist in a decode step that a CUDA graph replays: "
                           "read the batch's device tensor instead, or leave graph_safe off for this part")

    __getitem__ = __iter__ = __len__ = __bool__ = __contains__ = _refuse


class DecodeGraph:
    def __init__(self, runner, num_requests, max_context=None):
        """max_context: the longest context (tokens cached + 1) any replay of this graph will see; the attention
        kernel's slicing of the keys is fixed at capture and sized for it."""
        S, dev = int(num_requests), runner.device
        self.runner, self.S = runner, S
        self.max_pages = mp = runner.max_pages_per_request
        self.group_names = list(runner.manager.groups)
        # one packed int32 buffer: token_ids, positions, context_before, slots, then per group
        # slot_mapping [S] and block_table [S*mp]
        n = 4 * S + len(self.group_names) * (S + S * mp)
        # a small ring of pinned staging buffers: the host may run several steps ahead of the device, and a
        # buffer is rewritten only after the copy that read it has happened (its event has passed)
        self.ring = [torch.empty(n, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self.ring_np = [b.numpy() for b in self.ring]
        self.ring_events = [None] * len(self.ring)
        self.ring_pos = 0
        self.host = self.ring[0]
        self.dev = torch.zeros(n, dtype=torch.int32, device=dev)
        v = lambda i, m: self.dev[i:i + m]
        ar = torch.arange(S + 1, dtype=torch.int32, device=dev)
        groups, off = {}, 4 * S
        for g in self.group_names:
            groups[g] = GroupBatch(self.dev[off + S:off + S + S * mp].view(S, mp), v(off, S))
            off += S + S * mp
        self.batch = StepBatch(
            num_tokens=S, num_requests=S, num_logits=S, token_ids=v(0, S), positions=v(S, S),
            tok_req=ar[:S].contiguous(), q_start=ar, context_before=v(2 * S, S), slots=v(3 * S, S),
            logits_rows=ar[:S].contiguous(), groups=groups, status=runner.status,
            host_q_start=list(range(S + 1)), host_context_before=_OnDeviceOnly("host_context_before"),
            host_slots=_OnDeviceOnly("host_slots"))
        self.batch.decode_only = True
        self.batch.max_context = int(max_context or runner.plan.max_positions)
        self.graph = None
        self.logits = self.tokens = None
        self.kernels_per_replay = 0

    def _fill(self, hs, tokens_from=None):
        i = self.ring_pos
        self.ring_pos = (i + 1) % len(self.ring)
        if self.ring_events[i] is not None:
            self.ring_events[i].synchronize()
        S, mp, h = self.S, self.max_pages, self.ring_np[i]
        h[0:S] = hs.token_ids
        h[S:2 * S] = hs.positions
        h[2 * S:3 * S] = hs.context_before
        h[3 * S:4 * S] = hs.slots
        off = 4 * S
        for g in self.group_names:
            h[off:off + S] = hs.slot_maps[g]
            tab = h[off + S:off + S + S * mp].reshape(S, mp)
            for s, t in enumerate(hs.tables[g]):
                tab[s, :len(t)] = t
            off += S + S * mp
        if tokens_from is not None:     # the token ids are on the device already (the previous step's argmax)
            self.dev[S:].copy_(self.ring[i][S:], non_blocking=True)
            self.dev[0:S].copy_(tokens_from, non_blocking=True)
        else:
            self.dev.copy_(self.ring[i], non_blocking=True)
        ev = self.ring_events[i] or torch.cuda.Event()
        ev.record()
        self.ring_events[i] = ev

    def _forward(self):
        logits = self.runner.model.forward(self.batch, self.runner.storage.layers)
        return logits, kernels.argmax(logits)

    def run(self, hs, tokens_from=None):
        """hs: HostStep of S single-token entries.  Returns (logits [S,V], greedy tokens int32 [S]), both
        device tensors that the next replay overwrites.  ``tokens_from``: an int32 [S] device tensor to take
        the token ids from instead of hs.token_ids (the previous step's greedy tokens, which never left the
        device)."""
        self._fill(hs, tokens_from)
        if self.graph is None:
            # first use: once eagerly (sets kernel attributes, warms allocator), then capture
            n0 = kernels.launch_count()
            self._forward()
            self.kernels_per_replay = kernels.launch_count() - n0
            torch.cuda.current_stream().synchronize()
            g = torch.cuda.CUDAGraph()
            # objects that die during a capture (an older runner's graph, say) would free device memory in
            # the middle of it, which CUDA refuses: collect them first and keep the collector off meanwhile
            gc.collect()
            was_enabled = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(g):
                    self.logits, self.tokens = self._forward()
            finally:
                if was_enabled:
                    gc.enable()
            self.graph = g
        self.graph.replay()
        kernels.count_launches(self.kernels_per_replay)
        return self.logits, self.tokens
