"""What a part is, and the registry that builds parts from ``PartSpec``s.

A part owns its sizes and constants (constructor parameters), the names and shapes of its tensors
(``tensor_specs``), their device layout (``bind``) and its computation (``forward``).  It never looks at
the model configuration or at other layers.  Categories and the interface of each:

  norm          forward(x_f32[T,H], out_dtype, rows=None) -> [R,H]
  position      encode_and_store(qkv_f32, positions, slot_mapping, kv_cache, num_heads, num_kv_heads,
                                 page_size, batch=None) -> q[T,NH*HD]
  mixer         cache_spec() -> KVCacheSpec | StateSpec | None
                forward(x[T,H], batch, cache, residual_f32[T,H])      (adds its output into residual)
  feed_forward  forward(x[T,H], residual_f32[T,H])                     (adds its output into residual)
  block         built from a LayerSpec; forward(residual, batch, cache)
  embedding     forward(token_ids) -> residual_f32[T,H]
  lm_head       forward(x[R,H]) -> logits_f32[R,V]
"""
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from ..config.base import ConfigError, PartSpec
from ..weights.loader import TensorSpec

CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block", "embedding", "lm_head")
_REGISTRY = {c: {} for c in CATEGORIES}


@dataclass(frozen=True)
class Runtime:
    """Where and in which precision parts compute.  ``dtype`` is the type of activations, matrices and
    cache: torch.bfloat16 (tensor-core kernels) or torch.float32 (true 32-bit kernels everywhere)."""
    device: torch.device
    dtype: torch.dtype

    @property
    def full_precision(self):
        return self.dtype == torch.float32


@dataclass(frozen=True)
class KVCacheSpec:
    """A mixer that keeps keys and values: pages of [2, num_kv_heads, page_size, head_dim].
    ``window``: only the last ``window`` positions are ever read (None: all of them)."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """A mixer that keeps per-request state of fixed size: one row of ``shape`` per request slot."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


def register_part(category, kind, cls, replace=False):
    if category not in _REGISTRY:
        raise ConfigError(f"unknown part category {category!r}; known: {CATEGORIES}")
    if kind in _REGISTRY[category] and not replace:
        raise ConfigError(f"{category} part {kind!r} is already registered")
    _REGISTRY[category][kind] = cls


def unregister_part(category, kind):
    _REGISTRY[category].pop(kind, None)


def registered_parts(category):
    return sorted(_REGISTRY[category])


def replay_of(part):
    """(key, tensors) if ``part`` declares that its launches in one layer differ from its launches in another layer of
    the same shape only by the addresses of its own device tensors, else None.  A part declares it with
    ``replay_tensors()`` (its device tensors in a fixed order, None where an optional one is absent) and ``replay_key()``
    (everything else that shapes its launches: sizes, constants, types); the model then runs one such layer through
    Python, notes the launches, and repeats them for the other layers with the addresses exchanged.  A part that keeps
    host state per layer, or runs device work that is not one of ``forge_b200.kernels``' launches, must not declare it."""
    tensors = getattr(part, "replay_tensors", None)
    key = getattr(part, "replay_key", None)
    if tensors is None or key is None:
        return None
    t, k = tensors(), key()
    return None if t is None or k is None else (k, list(t))


def is_graph_safe(part):
    """True if the part and every part inside it declare ``graph_safe``."""
    if not getattr(part, "graph_safe", False):
        return False
    subs = getattr(part, "sub_parts", None)
    return all(is_graph_safe(p) for p in (subs() if subs else []))


def build_part(category, spec: PartSpec, rt: Runtime):
    try:
        cls = _REGISTRY[category][spec.kind]
    except KeyError:
        raise ConfigError(f"no {category} part named {spec.kind!r}; known: {registered_parts(category)}") from None
    return cls(rt=rt, **spec.params)


class Part:
    """Base of all parts.  Subclasses define ``tensor_specs`` and ``bind``.

    ``graph_safe``: the part's ``forward`` may be captured once in a CUDA graph and replayed for later decode
    steps.  That holds only for a part that takes everything that changes from step to step (positions,
    request slots, block tables, context lengths) from the batch's DEVICE tensors inside its kernels, and plans
    nothing from the batch's host lists.  A part has to say so itself; the default is no, and a model with one
    part that does not say so decodes through the ordinary step.  A part made of other parts answers for them
    (``sub_parts``)."""
    graph_safe = False

    def sub_parts(self):
        """The parts this part is made of (for questions that a whole layer has to answer)."""
        return []

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]):
        """Takes the part's tensors (CPU or device, as stored in the file) and keeps device copies in the
        layout its kernels want."""

    # helpers -------------------------------------------------------------------------------------
    def _matrix(self, t):
        """Matrices compute in the runtime's dtype."""
        return t.to(device=self.rt.device, dtype=self.rt.dtype).contiguous()

    def _vector_f32(self, t):
        """Norm weights and biases are read in 32-bit by every kernel."""
        return t.to(device=self.rt.device, dtype=torch.float32).contiguous()
