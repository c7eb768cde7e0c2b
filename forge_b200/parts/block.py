"""Arrangements of a layer's parts around the fp32 residual stream.

"pre_norm":  r += mixer(norm_in(r));  r += feed_forward(norm_post(r))
(reference: src/inference/engines/generic_engine.cpp:931-938, 1045-1052, 1080).  The additions happen in
the epilogue of each part's last matrix product, in fp32.
"""
from ..weights.loader import TensorSpec  # noqa: F401  (re-exported for part authors)
from .base import Part, build_part, register_part


class PreNormBlock(Part):
    graph_safe = True       # the arrangement itself looks at nothing of the step; its parts answer for themselves

    def sub_parts(self):
        return [self.mixer, self.feed_forward, self.norm_in, self.norm_post]
    NORM_NAMES = {"input": "input_layernorm.", "post_mixer": "post_attention_layernorm."}

    def __init__(self, rt, layer_spec):
        self.rt = rt
        self.mixer = build_part("mixer", layer_spec.mixer, rt)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, rt)
        self.norm_in = build_part("norm", layer_spec.norms["input"], rt)
        self.norm_post = build_part("norm", layer_spec.norms["post_mixer"], rt)

    def _children(self):
        return [("", self.mixer), ("", self.feed_forward), (self.NORM_NAMES["input"], self.norm_in),
                (self.NORM_NAMES["post_mixer"], self.norm_post)]

    def tensor_specs(self):
        specs = {}
        for prefix, part in self._children():
            for name, s in part.tensor_specs().items():
                specs[prefix + name] = s
        return specs

    def bind(self, tensors):
        for prefix, part in self._children():
            part.bind({name: tensors[prefix + name] for name in part.tensor_specs() if prefix + name in tensors})

    def fused_decode(self):
        """What the kernel that runs all layers of a decode step at once needs of this layer, or None: the layer
        must be exactly the stock arrangement of the stock parts (that kernel computes RMSNorm, rotary attention
        over the paged cache and SwiGLU, and nothing else), in bfloat16 on the tensor-core products."""
        from .attention import GQAAttention
        from .feedforward import SwiGLU
        from .norm import RMSNorm
        m, f, n1, n2 = self.mixer, self.feed_forward, self.norm_in, self.norm_post
        if type(self) is not PreNormBlock or type(m) is not GQAAttention or type(f) is not SwiGLU \
                or type(n1) is not RMSNorm or type(n2) is not RMSNorm or self.rt.full_precision:
            return None
        pos = m.position.fused_decode() if hasattr(m.position, "fused_decode") else None
        if pos is None or m.out_bias or n1.eps != n2.eps or m.qkv is None:
            return None
        if not all(lin.tensor_core for lin in (m.qkv, m.o, f.gate_up, f.down)):
            return None
        return {"hidden": m.hidden_size, "intermediate": f.intermediate_size, "num_heads": m.num_heads,
                "num_kv_heads": m.num_kv_heads, "head_dim": m.head_dim, "theta": pos["theta"], "rotary": pos["rotary"],
                "eps": n1.eps, "window": m.window or 0, "scale": m.scale,
                "tensors": {"wqkv": m.qkv.weight, "wo": m.o.weight, "wgu": f.gate_up.weight, "wdown": f.down.weight,
                            "norm1": n1.weight, "norm2": n2.weight, "bias": m.qkv.bias}}

    def _replay_parts(self):
        from .base import replay_of
        parts = [replay_of(p) for p in (self.norm_in, self.mixer, self.norm_post, self.feed_forward)]
        return None if type(self) is not PreNormBlock or any(p is None for p in parts) else parts

    def replay_tensors(self):
        parts = self._replay_parts()
        return None if parts is None else [t for _, tensors in parts for t in tensors]

    def replay_key(self):
        parts = self._replay_parts()
        return None if parts is None else ("pre_norm",) + tuple(k for k, _ in parts)

    def forward(self, residual, batch, cache):
        x = self.norm_in.forward(residual)
        self.mixer.forward(x, batch, cache, residual)
        x = self.norm_post.forward(residual)
        self.feed_forward.forward(x, residual)


def build_block(layer_spec, rt):
    from .base import _REGISTRY
    from ..config.base import ConfigError
    try:
        cls = _REGISTRY["block"][layer_spec.block]
    except KeyError:
        raise ConfigError(f"no block arrangement named {layer_spec.block!r}") from None
    return cls(rt, layer_spec)


register_part("block", "pre_norm", PreNormBlock, replace=True)
