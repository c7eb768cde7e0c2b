"""The batch of one step: for each request its next tokens (a portion of its prompt, cut anywhere, or one
decoded token), flattened into one list of tokens that every kernel runs over once.

The reference's InferenceBatch (include/forge/inference_batch.h:10-76) carries the same information per
item; its engine then loops over sequences (transformer_engine.cpp:201-254).  Here the arrays are flat and
on the device: attention is the only kernel that looks at request boundaries.
"""
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch


@dataclass
class StepEntry:
    """One request's share of a step.  ``want``: indices into ``tokens`` whose logits are asked for."""
    req_id: object
    tokens: List[int]
    want: List[int] = field(default_factory=list)


@dataclass
class GroupBatch:
    block_table: torch.Tensor          # int32 [S, max_pages]; -1 where a page was released
    slot_mapping: torch.Tensor         # int32 [T]: page * page_size + offset of each new token


@dataclass
class StepBatch:
    num_tokens: int
    num_requests: int
    num_logits: int
    token_ids: torch.Tensor            # int32 [T]
    positions: torch.Tensor            # int32 [T]   position of each token in its request
    tok_req: torch.Tensor              # int32 [T]   row (0..S-1) of each token's request in this step
    q_start: torch.Tensor              # int32 [S+1] first token of each request in the flat list
    context_before: torch.Tensor       # int32 [S]   tokens the request already had in the cache
    slots: torch.Tensor                # int32 [S]   request slot (row of fixed-size state tensors)
    logits_rows: Optional[torch.Tensor]  # int32 [R] flat token indices whose logits are wanted
    groups: Dict[str, GroupBatch]
    status: Optional[torch.Tensor] = None    # int32 [1] device error flags raised by kernels
    # host copies for parts and kernels that plan their work on the host
    host_q_start: List[int] = field(default_factory=list)
    host_context_before: List[int] = field(default_factory=list)
    host_slots: List[int] = field(default_factory=list)
    attention_plan: dict = field(default_factory=dict)


@dataclass
class HostStep:
    """A step laid out on the host, before it is copied to the device."""
    token_ids: List[int]
    positions: List[int]
    tok_req: List[int]
    q_start: List[int]
    context_before: List[int]
    slots: List[int]
    rows: List[int]
    slot_maps: Dict[str, List[int]]
    tables: Dict[str, List[List[int]]]


def layout_step(entries, manager):
    """Appends every entry's tokens to its request in the cache manager (allocating pages) and lays the
    step out as flat host lists.  Raises OutOfPages before touching anything if the step cannot grow."""
    reserve = {g: 0 for g in manager.groups}
    for e in entries:
        for g, n in manager.pages_needed(e.req_id, len(e.tokens)).items():
            reserve[g] += n
    for g, n in reserve.items():
        if n > manager.num_free_pages(g):
            from ..cache import OutOfPages
            raise OutOfPages(f"step needs {n} pages of group {g!r}, {manager.num_free_pages(g)} free")
    hs = HostStep([], [], [], [0], [], [], [], {g: [] for g in manager.groups}, {g: [] for g in manager.groups})
    for s, e in enumerate(entries):
        n0, n = manager.num_tokens(e.req_id), len(e.tokens)
        new_slots = manager.append(e.req_id, n)
        for g in hs.slot_maps:
            hs.slot_maps[g].extend(new_slots[g])
            hs.tables[g].append(manager.block_table(e.req_id, g))
        base = len(hs.token_ids)
        hs.token_ids.extend(e.tokens)
        hs.positions.extend(range(n0, n0 + n))
        hs.tok_req.extend([s] * n)
        hs.q_start.append(base + n)
        hs.context_before.append(n0)
        hs.slots.append(manager.slot(e.req_id))
        for w in e.want:
            if not 0 <= w < n:
                raise ValueError(f"request {e.req_id!r}: wanted index {w} outside its {n} tokens")
            hs.rows.append(base + w)
    return hs


def build_step_batch(entries, manager, device, max_pages, status=None):
    """Lays the step out (see ``layout_step``) and copies it to the device as one StepBatch: all integer
    arrays travel in one buffer and one copy, the batch's tensors are views into it."""
    hs = layout_step(entries, manager)
    T, S, R = len(hs.token_ids), len(entries), len(hs.rows)
    for s, e in enumerate(entries):
        for g in manager.groups:
            if len(hs.tables[g][s]) > max_pages:
                raise ValueError(f"request {e.req_id!r} holds {len(hs.tables[g][s])} pages, tables have room for {max_pages}")
    parts = [hs.token_ids, hs.positions, hs.tok_req, hs.q_start, hs.context_before, hs.slots, hs.rows]
    total = sum(len(p) for p in parts) + len(manager.groups) * (T + S * max_pages)
    buf = np.empty(total, dtype=np.int32)
    spans, off = [], 0
    for p in parts:
        buf[off:off + len(p)] = p
        spans.append((off, len(p)))
        off += len(p)
    group_spans = {}
    for g in manager.groups:
        buf[off:off + T] = hs.slot_maps[g]
        table = buf[off + T:off + T + S * max_pages].reshape(S, max_pages)
        table.fill(-1)
        for s, t in enumerate(hs.tables[g]):
            table[s, :len(t)] = t
        group_spans[g] = (off, off + T)
        off += T + S * max_pages
    from .. import kernels
    dev = kernels.new_tensor((total,), torch.int32, device)      # from the step's workspace, if one is open
    dev.copy_(torch.from_numpy(buf))

    def view(i):
        o, n = spans[i]
        return dev[o:o + n]

    groups = {g: GroupBatch(dev[t0:t0 + S * max_pages].view(S, max_pages), dev[s0:s0 + T]) for g, (s0, t0) in group_spans.items()}
    return StepBatch(
        num_tokens=T, num_requests=S, num_logits=R, token_ids=view(0), positions=view(1), tok_req=view(2), q_start=view(3),
        context_before=view(4), slots=view(5), logits_rows=view(6) if R else None, groups=groups, status=status,
        host_q_start=hs.q_start, host_context_before=hs.context_before, host_slots=hs.slots)
