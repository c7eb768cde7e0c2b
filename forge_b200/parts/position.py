"""Position encodings applied to q and k on their way into attention and the cache.

"rope": half-split rotary embedding of the whole head (reference: src/operators/cuda/cuda_rope.cu:8-34,
generic_engine.cpp:428-433).  "none": no encoding (keys are stored as projected).  Both are one fused
kernel that also writes k and v into the paged cache.
"""
from .. import kernels
from .base import Part, register_part


class RotaryEmbedding(Part):
    rotary = True

    def __init__(self, rt, head_dim, theta=10000.0):
        self.rt, self.head_dim, self.theta = rt, int(head_dim), float(theta)

    def encode_and_store(self, qkv, positions, slot_mapping, kv_cache, num_heads, num_kv_heads, page_size, batch=None):
        """``batch`` (optional): the step's batch; its ``attention_plan`` dict keeps the step's cos/sin table so
        that it is computed once per step, not once per layer."""
        table = None
        if self.rotary and batch is not None and qkv.shape[0] >= 64:
            key = ("rope", self.head_dim, self.theta)
            table = batch.attention_plan.get(key)
            if table is None:
                table = batch.attention_plan[key] = kernels.rope_table(positions, self.head_dim, self.theta)
        return kernels.rope_kv_write(qkv, positions, slot_mapping, kv_cache, num_heads, num_kv_heads, self.head_dim,
                                     page_size, self.theta, self.rt.dtype, rotary=self.rotary, table=table)


class NoPosition(RotaryEmbedding):
    rotary = False

    def __init__(self, rt, head_dim):
        super().__init__(rt, head_dim, 1.0)


register_part("position", "rope", RotaryEmbedding, replace=True)
register_part("position", "none", NoPosition, replace=True)
