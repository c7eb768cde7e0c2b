"""Position encodings applied to q and k on their way into attention and the cache.

"rope": half-split rotary embedding of the whole head (reference: src/operators/cuda/cuda_rope.cu:8-34,
generic_engine.cpp:428-433).  "none": no encoding (keys are stored as projected).  Both are one fused
kernel that also writes k and v into the paged cache.

A position part may also offer its encoding to the decode step's one-launch attention kernel, which rotates
q and k itself: ``fused_decode()`` returns the kernel's parameters, or None.  Only a part whose
``encode_and_store`` computes exactly what that kernel computes may return them; a subclass with other
arithmetic inherits None and keeps one path for prompt and decode steps.
"""
from .. import kernels
from .base import Part, register_part


class RotaryEmbedding(Part):
    rotary = True
    graph_safe = True       # angles come from ``positions`` on the device

    def __init__(self, rt, head_dim, theta=10000.0):
        self.rt, self.head_dim, self.theta = rt, int(head_dim), float(theta)

    def fused_decode(self):
        """{"theta", "rotary"} for the decode attention kernel that encodes by itself, or None.  The kernel
        hard-wires the half-split rotation of the whole head, so only the two stock classes offer it."""
        if type(self) not in (RotaryEmbedding, NoPosition):
            return None
        return {"theta": self.theta, "rotary": self.rotary}

    def replay_tensors(self):
        return [] if type(self) in (RotaryEmbedding, NoPosition) else None      # no tensors: the angles come from positions

    def replay_key(self):
        return (type(self).__name__, self.head_dim, self.theta, self.rotary)

    def _table(self, positions, batch, by_pair=False):
        """The step's cos/sin table, computed once per step (kept in the batch's ``attention_plan``), not once per
        layer.  A batch that a CUDA graph replays keeps no table: the table of the captured step would be replayed
        with every later step's positions.  ``by_pair``: the layout [head_dim/2, tokens, 2] that the fused projection
        reads."""
        if not self.rotary or batch is None or getattr(batch, "decode_only", False):
            return None
        key = ("rope", self.head_dim, self.theta, positions.data_ptr(), by_pair)
        table = batch.attention_plan.get(key)
        if table is None:
            table = batch.attention_plan[key] = kernels.rope_table(positions, self.head_dim, self.theta, by_pair=by_pair)
        return table

    def fused_projection(self, positions, batch):
        """For the q/k/v product whose epilogue encodes and stores by itself (prompt portions): {"table": the step's
        (cos, sin) table by pair, or None for no rotation}, or None if this part does not offer it.  As with
        ``fused_decode`` only the stock classes do: that epilogue computes the half-split rotation of the whole head."""
        if type(self) not in (RotaryEmbedding, NoPosition) or batch is None or getattr(batch, "decode_only", False):
            return None
        return {"table": self._table(positions, batch, by_pair=True)}

    def encode_and_store(self, qkv, positions, slot_mapping, kv_cache, num_heads, num_kv_heads, page_size, batch=None):
        """``batch`` (optional): the step's batch, which keeps the step's table of angles."""
        table = self._table(positions, batch) if qkv.shape[0] >= 64 else None
        return kernels.rope_kv_write(qkv, positions, slot_mapping, kv_cache, num_heads, num_kv_heads, self.head_dim,
                                     page_size, self.theta, self.rt.dtype, rotary=self.rotary, table=table)


class NoPosition(RotaryEmbedding):
    rotary = False

    def __init__(self, rt, head_dim):
        super().__init__(rt, head_dim, 1.0)


register_part("position", "rope", RotaryEmbedding, replace=True)
register_part("position", "none", NoPosition, replace=True)
