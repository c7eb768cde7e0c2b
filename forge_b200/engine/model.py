"""A model assembled from a ``ModelPlan``: embedding, layers (blocks of parts), final norm, output head.

The model knows nothing about any architecture: it builds the parts the plan names, collects the tensors
they expect under the plan's prefixes, hands each part its tensors, and runs the layers in the order of
``plan.schedule``.  (The reference's counterpart is TransformerEngine + GenericEngine,
src/inference/engines/transformer_engine.cpp:445-522, with the layer body at generic_engine.cpp:916-1085.)
"""
import torch

from ..config.base import ConfigError, ModelPlan
from ..parts import Runtime, build_block, build_part
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
                part.bind(mine, shared_table=self.embedding.table)
            else:
                part.bind(mine)
        self.loaded = True

    # ---------------------------------------------------------------------------------- cache needs
    def cache_specs(self):
        return [blk.mixer.cache_spec() for blk in self.blocks]

    def cache_from(self):
        return [spec.cache_from for spec in self.plan.layers]

    # ---------------------------------------------------------------------------------- forward
    def forward(self, batch, layer_caches):
        """Runs the step's tokens through all layers; returns fp32 logits [R,V] at ``batch.logits_rows``
        (None if no row is wanted)."""
        residual = self.embedding.forward(batch.token_ids, status=batch.status)
        for i in self.plan.schedule:
            self.blocks[i].forward(residual, batch, layer_caches[i])
        if batch.num_logits == 0:
            return None
        x = self.final_norm.forward(residual, rows=batch.logits_rows)
        return self.lm_head.forward(x)
