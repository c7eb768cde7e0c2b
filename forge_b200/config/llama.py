"""Typed configuration of the dense LLaMA decoder (GQA attention, RMSNorm, rotary positions, SwiGLU),
read from the keys of the architecture's own config.json.

The same numbers the reference keeps in its flat ModelConfig (include/forge/model.h:21-41) and fills from
GGUF / NINF metadata (src/model/arch_config_parser.cpp:42-89, src/model/model.cpp:184-204); here the key
names are those of a Hugging Face style config.json.  No size or constant of the model lives anywhere else.
"""
from dataclasses import asdict, dataclass
from typing import Optional

from .base import ConfigError, LayerSpec, ModelPlan, PartSpec, optional, require


@dataclass(frozen=True)
class LlamaConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 4096
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    # default of attention_bias when the key is absent, per registered architecture name
    BIAS_DEFAULT = {"LlamaForCausalLM": False, "Qwen2ForCausalLM": True}

    @classmethod
    def from_dict(cls, d, architecture="LlamaForCausalLM"):
        nh = require(d, "num_attention_heads", int)
        hidden = require(d, "hidden_size", int)
        if nh <= 0:
            raise ConfigError("config.json: 'num_attention_heads' must be positive")
        if "head_dim" not in d or d["head_dim"] is None:
            if hidden % nh != 0:
                raise ConfigError(f"config.json: 'head_dim' is absent and hidden_size {hidden} is not a multiple "
                                  f"of num_attention_heads {nh}")
        eos = d.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        cfg = cls(
            architecture=architecture,
            vocab_size=require(d, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=require(d, "intermediate_size", int),
            num_hidden_layers=require(d, "num_hidden_layers", int),
            num_attention_heads=nh,
            num_key_value_heads=optional(d, "num_key_value_heads", int, nh),
            head_dim=optional(d, "head_dim", int, hidden // nh),
            rope_theta=optional(d, "rope_theta", float, 10000.0),
            rms_norm_eps=optional(d, "rms_norm_eps", float, 1e-6),
            max_position_embeddings=optional(d, "max_position_embeddings", int, 4096),
            tie_word_embeddings=optional(d, "tie_word_embeddings", bool, False),
            attention_bias=optional(d, "attention_bias", bool, cls.BIAS_DEFAULT.get(architecture, False)),
            bos_token_id=optional(d, "bos_token_id", int, None),
            eos_token_id=None if eos is None else int(eos),
            torch_dtype=optional(d, "torch_dtype", str, "bfloat16"),
        )
        # options of the file format that this engine does not compute: refuse rather than ignore
        if d.get("rope_scaling") not in (None, {}):
            raise ConfigError("config.json: 'rope_scaling' is set; scaled rotary variants are not implemented "
                              "(the reference's LLaMA path has none either, generic_engine.cpp:428-433)")
        if optional(d, "hidden_act", str, "silu") != "silu":
            raise ConfigError(f"config.json: hidden_act {d['hidden_act']!r} is not supported (only 'silu')")
        if optional(d, "mlp_bias", bool, False):
            raise ConfigError("config.json: 'mlp_bias' true is not supported")
        cfg.validate()
        return cfg

    def validate(self):
        for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, k) <= 0:
                raise ConfigError(f"config.json: '{k}' must be positive, got {getattr(self, k)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(f"config.json: num_attention_heads {self.num_attention_heads} is not a multiple of "
                              f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even for rotary embedding")
        if not (self.rms_norm_eps > 0.0) or not (self.rope_theta > 0.0):
            raise ConfigError("config.json: rms_norm_eps and rope_theta must be positive")

    def to_dict(self):
        d = asdict(self)
        d["architectures"] = [d.pop("architecture")]
        d["model_type"] = "llama"
        d["hidden_act"] = "silu"
        return {k: v for k, v in d.items() if v is not None}

    def plan(self) -> ModelPlan:
        """Every layer: pre-norm block of [rmsnorm -> attention] and [rmsnorm -> swiglu] around a residual
        stream (src/inference/engines/generic_engine.cpp:916-1085)."""
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        mixer = PartSpec("attention", {
            "hidden_size": self.hidden_size, "num_heads": self.num_attention_heads,
            "num_kv_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "qkv_bias": self.attention_bias, "out_bias": False, "window": None,
            "position": PartSpec("rope", {"head_dim": self.head_dim, "theta": self.rope_theta}),
        })
        ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size})
        layers = [LayerSpec(block="pre_norm", mixer=mixer, feed_forward=ffn,
                            norms={"input": norm, "post_mixer": norm},
                            weight_prefix=f"model.layers.{i}.") for i in range(self.num_hidden_layers)]
        return ModelPlan(
            hidden_size=self.hidden_size, vocab_size=self.vocab_size, max_positions=self.max_position_embeddings,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}),
            final_norm=norm,
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                                         "tied": self.tie_word_embeddings}),
            layers=layers, schedule=list(range(self.num_hidden_layers)))
