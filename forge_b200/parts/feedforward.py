"""SwiGLU feed-forward:  residual += ( silu(x.Wg^T) * (x.Wu^T) ) . Wd^T
(reference: src/inference/engines/generic_engine.cpp:776-780, 809, 1080).  Gate and up are one matrix
product: their rows are interleaved at load time (row 2j = gate j, row 2j+1 = up j) so the product's
epilogue sees each (gate, up) pair side by side.
"""
import torch

from ..weights.loader import TensorSpec
from .base import Part, register_part
from .linear import Linear

DEFAULT_NAMES = {"gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj"}


class SwiGLU(Part):
    graph_safe = True
    def __init__(self, rt, hidden_size, intermediate_size, names=None):
        self.rt, self.hidden_size, self.intermediate_size = rt, hidden_size, intermediate_size
        self.names = {**DEFAULT_NAMES, **(names or {})}
        self.gate_up = self.down = None

    def tensor_specs(self):
        n, H, I = self.names, self.hidden_size, self.intermediate_size
        return {n["gate"] + ".weight": TensorSpec((I, H)), n["up"] + ".weight": TensorSpec((I, H)),
                n["down"] + ".weight": TensorSpec((H, I))}

    def bind(self, tensors):
        n = self.names
        g, u = tensors[n["gate"] + ".weight"], tensors[n["up"] + ".weight"]
        gu = torch.stack([g, u], dim=1).reshape(2 * self.intermediate_size, self.hidden_size)
        self.gate_up = Linear(self._matrix(gu), None, self.rt)
        self.down = Linear(self._matrix(tensors[n["down"] + ".weight"]), None, self.rt)

    def replay_tensors(self):
        return self.gate_up.replay_tensors() + self.down.replay_tensors() if type(self) is SwiGLU else None

    def replay_key(self):
        return ("swiglu", self.gate_up.replay_key(), self.down.replay_key())

    def forward(self, x, residual):
        act = self.gate_up.forward(x, epilogue="swiglu")          # [T,I] in the activation type
        self.down.forward(act, accumulate_into=residual)


register_part("feed_forward", "swiglu", SwiGLU, replace=True)
