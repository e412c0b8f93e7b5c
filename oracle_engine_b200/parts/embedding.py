"""Token embedding and output head.

`token_embedding`: x = E[token] as float32 (core/model.cpp:352-358); an id outside the
table is an error, not clamped.  `lm_head`: logits = W x in float32, W a separate matrix
or, when tied, the embedding table (core/model.cpp:482-492)."""
from __future__ import annotations

import torch

from ..csrc import ops
from .linear import matmul_nt
from .registry import EMBEDDINGS, HEADS, Part
from .spec import TensorDecl


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Part):
    """params: vocab_size, hidden_size, name."""
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.V = int(self._need("vocab_size"))
        self.D = int(self._need("hidden_size"))
        self.name = prefix + self._need("name")
        self.table = None
        self.err = None

    def tensors(self):
        return [TensorDecl(self.name, (self.V, self.D))]

    def load(self, get):
        self.table = self.rt.to_compute(get(self.name))
        self.err = torch.zeros(1, dtype=torch.int32, device=self.rt.device)

    def forward(self, ids, n_tokens, out=None):
        """The residual stream [n_tokens, hidden] float32 (written into `out` if given)."""
        x = self.rt.empty(n_tokens, self.D, dtype=torch.float32) if out is None else out
        ops.embed_gather(x, self.table, ids, self.err)
        return x


@HEADS.register("lm_head")
class LMHead(Part):
    """params: vocab_size, hidden_size, tied, name; `embedding` is handed in when tied."""
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.V = int(self._need("vocab_size"))
        self.D = int(self._need("hidden_size"))
        self.tied = bool(self._need("tied"))
        self.name = prefix + self.params.get("name", "lm_head.weight")
        self.embedding = self.params.get("embedding")
        self.weight = None

    def tensors(self):
        return [] if self.tied else [TensorDecl(self.name, (self.V, self.D))]

    def load(self, get):
        self.weight = self.embedding.table if self.tied else self.rt.to_compute(get(self.name))

    def weight_bytes(self):
        return 0 if self.weight is None else self.weight.numel() * self.weight.element_size()

    def flops(self, start, count):
        return count * 2.0 * self.V * self.D

    def forward(self, xn):
        logits = self.rt.empty(xn.shape[0], self.V, dtype=torch.float32)
        matmul_nt(self.rt, logits, xn, self.weight)
        return logits
