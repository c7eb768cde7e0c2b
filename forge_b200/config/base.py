"""Architecture-neutral description of a model: which parts make up each layer and in what order
layers run.  A configuration class (one per architecture) turns its config.json keys into a
``ModelPlan``; everything downstream (weights, cache, step function) reads only the plan.
"""
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """A config.json key is missing, has a bad value, or names something this engine does not run."""


@dataclass(frozen=True)
class PartSpec:
    """A part of a layer: its kind (a name in the part registry) and its sizes and constants."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: how its parts are arranged (``block``), the parts, and where its tensors live.

    ``cache_from``: index (into ``ModelPlan.layers``) of another layer whose cache this layer's mixer
    reads instead of keeping one of its own.
    """
    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Dict[str, PartSpec]
    weight_prefix: str
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    final_norm: PartSpec
    lm_head: PartSpec
    layers: List[LayerSpec]
    # order in which layers run; an index may appear twice (the layer's weights are reused)
    schedule: List[int]
    embedding_prefix: str = "model.embed_tokens."
    final_norm_prefix: str = "model.norm."
    lm_head_prefix: str = "lm_head."


def require(d, key, typ):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    return coerce(key, d[key], typ)


def optional(d, key, typ, default):
    if key not in d or d[key] is None:
        return default
    return coerce(key, d[key], typ)


def coerce(key, v, typ):
    if typ is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"config.json: '{key}' must be true or false, got {v!r}")
        return v
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
        return v
    if typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
        return float(v)
    if typ is str:
        if not isinstance(v, str):
            raise ConfigError(f"config.json: '{key}' must be a string, got {v!r}")
        return v
    raise TypeError(typ)
