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

    def encode_and_store(self, qkv, positions, slot_mapping, kv_cache, num_heads, num_kv_heads, page_size):
        return kernels.rope_kv_write(qkv, positions, slot_mapping, kv_cache, num_heads, num_kv_heads, self.head_dim,
                                     page_size, self.theta, self.rt.dtype, rotary=self.rotary)


class NoPosition(RotaryEmbedding):
    rotary = False

    def __init__(self, rt, head_dim):
        super().__init__(rt, head_dim, 1.0)


register_part("position", "rope", RotaryEmbedding, replace=True)
register_part("position", "none", NoPosition, replace=True)
