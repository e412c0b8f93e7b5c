"""Norms.  `rms_norm`: y = (x / sqrt(mean(x^2) + eps)) * w on the float32 residual stream,
computed in float32 and stored in the compute dtype (reference: core/ops.cpp:149-195; the
epsilon is a parameter here, always passed)."""
from __future__ import annotations

from ..csrc import ops
from .registry import NORMS, Part
from .spec import TensorDecl


@NORMS.register("rms_norm")
class RMSNorm(Part):
    graph_safe = True
    """params: size, eps, name (tensor name under the prefix)."""

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.size = int(self._need("size"))
        self.eps = float(self._need("eps"))
        self.name = prefix + self._need("name")
        self.weight = None

    def tensors(self):
        return [TensorDecl(self.name, (self.size,), "ones_normal")]

    def load(self, get):
        self.weight = self.rt.to_f32(get(self.name))

    def weight_bytes(self):
        return 0 if self.weight is None else self.weight.numel() * self.weight.element_size()

    def forward(self, x):
        y = self.rt.empty(*x.shape)
        ops.rmsnorm(y, x, self.weight, self.eps)
        return y
