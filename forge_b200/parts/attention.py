"""Grouped-query causal self-attention over the paged cache.

  qkv = x . [Wq;Wk;Wv]^T (+b);  q, k <- position(q, k);  cache <- k, v;  o = softmax(q k^T / sqrt(HD)) v;
  residual += o . Wo^T
(reference: src/inference/engines/generic_engine.cpp:940-1002; kv head of q head h is h // (NH/NKV)).
The three projections are one matrix product (rows of Wq, Wk, Wv concatenated at load time).
"""
import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import KVCacheSpec, Part, build_part, register_part
from .linear import Linear

DEFAULT_NAMES = {"q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj", "o": "self_attn.o_proj"}


class GQAAttention(Part):
    graph_safe = True       # request boundaries, positions and tables are read from the batch's device tensors

    def sub_parts(self):
        return [self.position]

    def __init__(self, rt, hidden_size, num_heads, num_kv_heads, head_dim, position, qkv_bias=False, out_bias=False,
                 window=None, names=None):
        self.rt = rt
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.qkv_bias, self.out_bias, self.window = bool(qkv_bias), bool(out_bias), window
        self.names = {**DEFAULT_NAMES, **(names or {})}
        self.position = build_part("position", position, rt)
        self.scale = head_dim ** -0.5
        self.qkv = self.o = None

    def tensor_specs(self):
        n, H = self.names, self.hidden_size
        q_out, kv_out = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        specs = {n["q"] + ".weight": TensorSpec((q_out, H)), n["k"] + ".weight": TensorSpec((kv_out, H)),
                 n["v"] + ".weight": TensorSpec((kv_out, H)), n["o"] + ".weight": TensorSpec((H, q_out))}
        if self.qkv_bias:
            specs.update({n["q"] + ".bias": TensorSpec((q_out,), role="bias"),
                          n["k"] + ".bias": TensorSpec((kv_out,), role="bias"),
                          n["v"] + ".bias": TensorSpec((kv_out,), role="bias")})
        if self.out_bias:
            specs[n["o"] + ".bias"] = TensorSpec((H,), role="bias")
        return specs

    def bind(self, tensors):
        n = self.names
        w = torch.cat([tensors[n[k] + ".weight"] for k in "qkv"], dim=0)
        b = torch.cat([tensors[n[k] + ".bias"] for k in "qkv"], dim=0) if self.qkv_bias else None
        self.qkv = Linear(self._matrix(w), None if b is None else self._vector_f32(b), self.rt)
        ob = self._vector_f32(tensors[n["o"] + ".bias"]) if self.out_bias else None
        self.o = Linear(self._matrix(tensors[n["o"] + ".weight"]), ob, self.rt)

    def cache_spec(self):
        return KVCacheSpec(self.num_kv_heads, self.head_dim, self.window)

    def replay_tensors(self):
        from .base import replay_of
        pos = replay_of(self.position)
        if type(self) is not GQAAttention or pos is None:
            return None
        return self.qkv.replay_tensors() + self.o.replay_tensors() + pos[1]

    def replay_key(self):
        from .base import replay_of
        pos = replay_of(self.position)
        return None if pos is None else ("gqa", self.num_heads, self.num_kv_heads, self.head_dim, self.window, self.scale,
                                         self.qkv.replay_key(), self.o.replay_key(), pos[0])

    def _decode_in_one_kernel(self, batch, cache):
        """A step of one new token per request, with a position part that offers its encoding to the decode
        kernel (``fused_decode``): encoding, cache write and attention run as one launch.  Returns the
        position part's parameters for that kernel, or None."""
        if batch.num_tokens != batch.num_requests or not cache.writable or self.rt.full_precision:
            return None
        offer = getattr(self.position, "fused_decode", None)
        params = offer() if offer is not None else None
        if params is None:
            return None
        max_ctx = getattr(batch, "max_context", None) or (max(batch.host_context_before) + 1)
        ok = kernels.decode_attention_fused_supports(self.rt.dtype, self.head_dim, self.num_heads // self.num_kv_heads,
                                                     batch.num_requests, self.num_kv_heads, max_ctx,
                                                     page_size=cache.page_size)
        return params if ok else None

    def forward(self, x, batch, cache, residual):
        """x [T,H] normed input; cache: the layer's KV cache view; adds the output projection into residual."""
        g = batch.groups[cache.group]
        offer = getattr(self.position, "fused_projection", None)
        if offer is not None and self.qkv.tensor_core and kernels.gemm_sm100_qkv_rope_supports(x.shape[0], self.head_dim, self.hidden_size):
            fused = offer(batch.positions, batch)
            if fused is not None:
                # prompt portions: the projection's epilogue rotates q and k and writes k and v into the pages
                q = kernels.gemm_sm100_qkv_rope(x, self.qkv.weight, self.qkv.bias, fused["table"],
                                                g.slot_mapping if cache.writable else None, cache.kv if cache.writable else None,
                                                self.num_heads, self.num_kv_heads, self.head_dim, cache.page_size)
                o = kernels.paged_attention(q, cache.kv, g, batch, self.num_heads, self.num_kv_heads, self.head_dim,
                                            cache.page_size, window=self.window, scale=self.scale)
                self.o.forward(o, accumulate_into=residual)
                return
        qkv = self.qkv.forward(x)                                           # fp32 [T,(NH+2NKV)*HD]
        fused = self._decode_in_one_kernel(batch, cache)
        if fused is not None:
            o = kernels.decode_attention_fused(qkv, cache.kv, g.block_table, batch.positions, g.slot_mapping,
                                               self.num_heads, self.num_kv_heads, self.head_dim, cache.page_size,
                                               fused["theta"], rotary=fused["rotary"], window=self.window,
                                               scale=self.scale,
                                               max_context=getattr(batch, "max_context", None) or max(batch.host_context_before) + 1)
            self.o.forward(o, accumulate_into=residual)
            return
        slots = g.slot_mapping if cache.writable else None
        q = self.position.encode_and_store(qkv, batch.positions, slots, cache.kv if cache.writable else None,
                                           self.num_heads, self.num_kv_heads, cache.page_size, batch=batch)
        o = kernels.paged_attention(q, cache.kv, g, batch, self.num_heads, self.num_kv_heads, self.head_dim,
                                    cache.page_size, window=self.window, scale=self.scale)
        self.o.forward(o, accumulate_into=residual)


register_part("mixer", "attention", GQAAttention, replace=True)
