"""Token embedding and output head.

embedding: residual[t,:] = E[id_t,:] (fp32 residual stream).  lm_head: logits = x . W^T in fp32, with
W = E when the embeddings are tied and the file has no head of its own
(reference: src/inference/engines/transformer_engine.cpp:495-522, src/model/model_weights.cpp:28-33).
"""
from .. import kernels
from ..weights.loader import TensorSpec
from .base import Part, register_part
from .linear import Linear


class TokenEmbedding(Part):
    graph_safe = True
    def __init__(self, rt, vocab_size, hidden_size, names=None):
        self.rt, self.vocab_size, self.hidden_size = rt, vocab_size, hidden_size
        self.names = {"weight": "weight", **(names or {})}
        self.table = None

    def tensor_specs(self):
        return {self.names["weight"]: TensorSpec((self.vocab_size, self.hidden_size), role="embedding")}

    def bind(self, tensors):
        self.table = self._matrix(tensors[self.names["weight"]])

    def output_table(self):
        """The table as an output head reads it when the two are tied: [vocab, hidden] in the compute dtype."""
        return self.table

    def forward(self, token_ids, status=None):
        return kernels.embedding(token_ids, self.table, status=status)


class LMHead(Part):
    graph_safe = True
    def __init__(self, rt, vocab_size, hidden_size, tied=False, names=None):
        self.rt, self.vocab_size, self.hidden_size, self.tied = rt, vocab_size, hidden_size, bool(tied)
        self.names = {"weight": "weight", **(names or {})}
        self.linear = None

    def tensor_specs(self):
        return {self.names["weight"]: TensorSpec((self.vocab_size, self.hidden_size), required=not self.tied)}

    def bind(self, tensors, shared_table=None):
        w = tensors.get(self.names["weight"])
        if w is None:
            if not self.tied or shared_table is None:
                raise ValueError("lm_head: no weight and nothing to tie to")
            self.linear = Linear(shared_table, None, self.rt)
        else:
            self.linear = Linear(self._matrix(w), None, self.rt)

    def forward(self, x):
        return self.linear.forward(x)


register_part("embedding", "embedding", TokenEmbedding, replace=True)
register_part("lm_head", "lm_head", LMHead, replace=True)
