"""Feed-forward `swiglu`: g = Wg h, u = Wu h, a = g/(1+exp(-g)) * u, x += Wd a  (dense, no
routing).  Reference: core/model.cpp:452-473 and :636-643.  The gate and up projections
are fused into one matrix product at load ([Wg; Wu])."""
from __future__ import annotations

import torch

from ..csrc import ops
from .linear import chain_flags, matmul_nt
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
        gate, up = to(get(self.names["gate"])), to(get(self.names["up"]))
        # On the tensor-core path the activation is fused into the product's epilogue, which
        # wants gate and up rows of a feature side by side: rows g0, u0, g1, u1, ...
        self.fused = self.rt.dtype == torch.bfloat16 and self.rt.tensor_cores and self.D % 8 == 0
        if self.fused:
            self.w_gu = torch.stack([gate, up], 1).reshape(2 * self.FF, self.D).contiguous()
        else:
            self.w_gu = torch.cat([gate, up], 0)
        self.w_down = to(get(self.names["down"]))

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_gu, self.w_down) if t is not None)

    def flops(self, start, count):
        return count * 2.0 * 3 * self.D * self.FF

    def first_weights(self):
        return self.w_gu

    def forward(self, h, residual, ctx):
        T = h.shape[0]
        a = self.rt.empty(T, self.FF)
        if self.fused:
            from ..csrc import ops_tc
            ops_tc.gemm(a, h, self.w_gu, swiglu=True, early=chain_flags("ffn_in", T), then=self.w_down)
        else:
            gu = self.rt.empty(T, 2 * self.FF)
            matmul_nt(self.rt, gu, h, self.w_gu)
            ops.swiglu(a, gu)
        matmul_nt(self.rt, residual, a, self.w_down, accumulate=True, early=chain_flags("ffn_out", T),
                  then=self.rt.next_weights)
