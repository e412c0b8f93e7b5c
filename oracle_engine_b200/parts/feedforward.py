"""Feed-forward `swiglu`: g = Wg h, u = Wu h, a = g/(1+exp(-g)) * u, x += Wd a  (dense, no
routing).  Reference: core/model.cpp:452-473 and :636-643.  The gate and up projections
are fused into one matrix product at load ([Wg; Wu])."""
from __future__ import annotations

import torch

from ..csrc import ops
from .linear import matmul_nt
from .registry import FEED_FORWARDS, Part
from .spec import TensorDecl

_NAMES = {"gate": "mlp.gate_proj.weight", "up": "mlp.up_proj.weight", "down": "mlp.down_proj.weight"}


@FEED_FORWARDS.register("swiglu")
class SwiGLU(Part):
    graph_safe = True
    """params: hidden_size, intermediate_size, tensor_names (optional overrides)."""

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D = int(self._need("hidden_size"))
        self.FF = int(self._need("intermediate_size"))
        self.names = {k: prefix + v for k, v in {**_NAMES, **self.params.get("tensor_names", {})}.items()}
        self.w_gu = self.w_down = None

    def tensors(self):
        return [TensorDecl(self.names["gate"], (self.FF, self.D)), TensorDecl(self.names["up"], (self.FF, self.D)),
                TensorDecl(self.names["down"], (self.D, self.FF))]

    def load(self, get):
        to = self.rt.to_compute
        self.w_gu = torch.cat([to(get(self.names["gate"])), to(get(self.names["up"]))], 0)
        self.w_down = to(get(self.names["down"]))

    def forward(self, h, residual, ctx):
        T = h.shape[0]
        gu = self.rt.empty(T, 2 * self.FF)
        matmul_nt(self.rt, gu, h, self.w_gu)
        a = self.rt.empty(T, self.FF)
        ops.swiglu(a, gu)
        matmul_nt(self.rt, residual, a, self.w_down, accumulate=True)
