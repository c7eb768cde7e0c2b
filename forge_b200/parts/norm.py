"""RMSNorm:  y = x * rsqrt(mean(x^2) + eps) * w   (reference: src/operators/cuda/cuda_rms_norm.cu:10-36)."""
from .. import kernels
from ..weights.loader import TensorSpec
from .base import Part, register_part


class RMSNorm(Part):
    graph_safe = True
    def __init__(self, rt, size, eps, names=None):
        self.rt, self.size, self.eps = rt, int(size), float(eps)
        self.names = {"weight": "weight", **(names or {})}
        self.weight = None

    def tensor_specs(self):
        return {self.names["weight"]: TensorSpec((self.size,), role="norm")}

    def bind(self, tensors):
        self.weight = self._vector_f32(tensors[self.names["weight"]])

    def replay_tensors(self):
        return [self.weight] if type(self) is RMSNorm else None

    def replay_key(self):
        return ("rmsnorm", self.size, self.eps, self.rt.dtype)

    def forward(self, x, out_dtype=None, rows=None):
        """x: fp32 [T,size] (the residual stream); returns [T or len(rows), size] in ``out_dtype``."""
        return kernels.rmsnorm(x, self.weight, self.eps, out_dtype or self.rt.dtype, rows=rows)


register_part("norm", "rmsnorm", RMSNorm, replace=True)
