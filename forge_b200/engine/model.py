"""A model assembled from a ``ModelPlan``: embedding, layers (blocks of parts), final norm, output head.

The model knows nothing about any architecture: it builds the parts the plan names, collects the tensors
they expect under the plan's prefixes, hands each part its tensors, and runs the layers in the order of
``plan.schedule``.  (The reference's counterpart is TransformerEngine + GenericEngine,
src/inference/engines/transformer_engine.cpp:445-522, with the layer body at generic_engine.cpp:916-1085.)
"""
import os

import torch

from .. import kernels
from ..config.base import ConfigError, ModelPlan
from ..parts import Runtime, build_block, build_part
from ..parts.base import is_graph_safe, replay_of
from ..weights.loader import WeightError


class Model:
    def __init__(self, plan: ModelPlan, rt: Runtime):
        self.plan, self.rt = plan, rt
        self.embedding = build_part("embedding", plan.embedding, rt)
        self.blocks = [build_block(spec, rt) for spec in plan.layers]
        self.final_norm = build_part("norm", plan.final_norm, rt)
        self.lm_head = build_part("lm_head", plan.lm_head, rt)
        n = len(plan.layers)
        for i in plan.schedule:
            if not 0 <= i < n:
                raise ConfigError(f"schedule names layer {i}, the plan has {n} layers")
        for i, spec in enumerate(plan.layers):
            if spec.cache_from is not None and not 0 <= spec.cache_from < n:
                raise ConfigError(f"layer {i}: cache_from {spec.cache_from} is not a layer")
        self.loaded = False
        self._fused = None
        self._replay_ok, self._replay_from, self._replay_tensors = False, 0, []

    # ---------------------------------------------------------------------------------- tensors
    def _children(self):
        p = self.plan
        out = [(p.embedding_prefix, self.embedding), (p.final_norm_prefix, self.final_norm),
               (p.lm_head_prefix, self.lm_head)]
        out += [(spec.weight_prefix, blk) for spec, blk in zip(p.layers, self.blocks)]
        return out

    def tensor_specs(self):
        """{tensor name in the file: TensorSpec}, in a fixed order."""
        specs = {}
        for prefix, part in self._children():
            for name, s in part.tensor_specs().items():
                specs[prefix + name] = s
        return specs

    def load(self, tensors, where="weights"):
        """tensors: {file name: tensor}; every expected tensor present (checked by the loader before)."""
        for prefix, part in self._children():
            mine = {name: tensors[prefix + name] for name in part.tensor_specs() if prefix + name in tensors}
            if part is self.lm_head:
                head_name = next(iter(part.tensor_specs()))
                if part.tied and head_name in mine:
                    emb_name = self.plan.embedding_prefix + next(iter(self.embedding.tensor_specs()))
                    if not torch.equal(mine[head_name].cpu(), tensors[emb_name].cpu()):
                        raise WeightError(where, wrong=[f"{prefix + head_name}: embeddings are tied but the file's "
                                                        "output head differs from the embedding table"])
                    mine = {}
                part.bind(mine, shared_table=self.embedding.output_table())
            else:
                part.bind(mine)
        self.loaded = True
        # layers whose launches may be repeated from one noted layer: all runs of the schedule from the first on, or
        # (a model whose first layer is of another kind) from the second on, declare it with one key
        runs = [replay_of(self.blocks[i]) for i in self.plan.schedule]
        self._replay_ok = False
        for first in (0, 1):
            rest = runs[first:]
            if len(rest) >= 2 and all(r is not None for r in rest) and len({r[0] for r in rest}) == 1:
                self._replay_ok, self._replay_from = True, first
                break
        self._replay_tensors = [r[1] if r is not None else None for r in runs]

    def graph_safe(self):
        """True if every part that a step runs declares that a CUDA graph may capture it."""
        parts = [self.embedding, self.final_norm, self.lm_head] + [self.blocks[i] for i in set(self.plan.schedule)]
        return all(is_graph_safe(p) for p in parts)

    # ---------------------------------------------------------------------------------- cache needs
    # Caches belong to positions of the schedule, not to layers: a layer that runs twice shares its weights
    # between the two runs but each run keeps keys/values (or state) of its own.
    def cache_specs(self):
        """Per schedule position: what that run of its layer's mixer keeps."""
        return [self.blocks[i].mixer.cache_spec() for i in self.plan.schedule]

    def cache_from(self):
        """Per schedule position: the earlier position whose cache it reads instead of keeping one (None:
        its own).  A LayerSpec names a LAYER in ``cache_from``; that resolves to the latest earlier run of
        that layer."""
        out = []
        for pos, i in enumerate(self.plan.schedule):
            src_layer = self.plan.layers[i].cache_from
            if src_layer is None:
                out.append(None)
                continue
            earlier = [q for q in range(pos) if self.plan.schedule[q] == src_layer]
            if not earlier:
                raise ConfigError(f"layer {i} reads the cache of layer {src_layer}, which has not run before it")
            out.append(earlier[-1])
        return out

    # ---------------------------------------------------------------------------------- all layers in one kernel
    def enable_fused_decode(self, position_caches, max_requests):
        """Prepares the kernel that runs every layer of a decode step in one launch, if this model is one it
        can run: every layer the stock arrangement of stock parts with equal sizes, each run once, in order, on
        a cache of its own, all in one cache group.  Returns whether it is on."""
        from .. import kernels
        self._fused = None
        sched = self.plan.schedule
        if self.rt.full_precision or not sched or sched != list(range(len(self.blocks))):
            return False
        descs = [b.fused_decode() if hasattr(b, "fused_decode") else None for b in self.blocks]
        if any(d is None for d in descs):
            return False
        keys = ("hidden", "intermediate", "num_heads", "num_kv_heads", "head_dim", "theta", "rotary", "eps", "window", "scale")
        first = descs[0]
        if any(d[k] != first[k] for d in descs for k in keys):
            return False
        caches = list(position_caches)
        if any(c is None or c.kv is None or not c.writable or c.group != caches[0].group for c in caches):
            return False
        if not kernels.DecodeLayers.supports(first["hidden"], first["intermediate"], first["num_heads"], first["num_kv_heads"],
                                             first["head_dim"]):
            return False
        layers = [dict(d["tensors"], kv=c.kv) for d, c in zip(descs, caches)]
        self._fused = (kernels.DecodeLayers(layers, first["hidden"], first["intermediate"], first["num_heads"],
                                            first["num_kv_heads"], first["head_dim"], caches[0].page_size, first["theta"],
                                            first["rotary"], first["eps"], window=first["window"], scale=first["scale"],
                                            max_tokens=min(max_requests, kernels.DecodeLayers.MAX_TOKENS)), caches[0].group)
        return True

    def _fused_decode_applies(self, batch):
        fused = getattr(self, "_fused", None)
        if fused is None or batch.num_tokens != batch.num_requests or batch.num_tokens > fused[0].max_tokens:
            return False
        return True

    def _replay_applies(self, position_caches, ws):
        """Whether the layers after the noted one may repeat its launches: every layer from the noted one on declares
        it and has the same key (``parts.base.replay_of``), their caches are of one kind, the outputs come from the
        step's workspace (so a layer's intermediates have the same addresses in every layer), and no timing table is
        being taken (it wants an event per launch)."""
        if ws is None or not self._replay_ok or kernels.profiler_enabled() or os.environ.get("FORGE_LAYER_REPLAY", "1") == "0":
            return False
        c1 = position_caches[self._replay_from]
        kind = (getattr(c1, "group", None), getattr(c1, "writable", None), getattr(c1, "page_size", None))
        for c in position_caches[self._replay_from:]:
            kv = getattr(c, "kv", None)
            if kv is None or (getattr(c, "group", None), getattr(c, "writable", None), getattr(c, "page_size", None)) != kind \
                    or kv.shape != c1.kv.shape or kv.dtype != c1.kv.dtype:
                return False
        return True

    # ---------------------------------------------------------------------------------- forward
    def forward(self, batch, position_caches, workspace=None):
        """Runs the step's tokens through the schedule; ``position_caches[p]`` is the cache of the p-th run.
        Returns fp32 logits [R,V] at ``batch.logits_rows`` (None if no row is wanted).  ``workspace``: the open
        StepWorkspace that the kernels' outputs are cut from; a layer's share of it is given back after the layer."""
        residual = self.embedding.forward(batch.token_ids, status=batch.status)
        if self._fused_decode_applies(batch):
            fused, group = self._fused
            g = batch.groups[group]
            fused.run(residual, g.block_table, batch.positions, g.slot_mapping)
        else:
            ws = workspace
            replay = None
            for pos, i in enumerate(self.plan.schedule):
                if replay is not None:
                    replay.run(self._replay_tensors[pos] + [position_caches[pos].kv])
                    continue
                # one layer's launches are noted and repeated for the layers after it (what the whole step shares,
                # tile lists and the table of angles, is made inside the first layer: those launches are marked
                # and stay out of the notes)
                note = pos == self._replay_from and self._replay_applies(position_caches, ws)
                m = ws.mark() if ws is not None else 0
                if note:
                    overflow = ws.allocations
                    with kernels.record_launches() as rec:
                        self.blocks[i].forward(residual, batch, position_caches[pos])
                    if ws.allocations == overflow:      # every output came from the workspace: the addresses repeat
                        replay = kernels.LayerReplay(rec, self._replay_tensors[pos] + [position_caches[pos].kv])
                else:
                    self.blocks[i].forward(residual, batch, position_caches[pos])
                if ws is not None:
                    ws.release(m)              # a layer's intermediates are dead: the residual stream carries on
        if batch.num_logits == 0:
            return None
        x = self.final_norm.forward(residual, rows=batch.logits_rows)
        if workspace is None:
            return self.lm_head.forward(x)
        with workspace.paused():               # the logits are the caller's to keep
            return self.lm_head.forward(x)
