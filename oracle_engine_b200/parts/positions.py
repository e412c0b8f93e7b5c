"""Position encodings.  `rotary`: rotate-half RoPE with optional llama3 frequency scaling.

The reference computes theta_i = pos / base^(2i/hd) and its cosine and sine per token
(core/ops.cpp:461-466) and has no frequency scaling.  Here the inverse frequencies are
computed once on the host in double precision, scaled as config.json's `rope_scaling`
says, and turned into float32 cos/sin tables [max_positions, hd/2] that the kernels read.

llama3 scaling, with f_i = base^(-2i/hd) and wavelength l_i = 2 pi / f_i:
  l_i < orig/high_freq_factor          keep f_i
  l_i > orig/low_freq_factor           f_i / factor
  otherwise  s = (orig/l_i - low)/(high - low);  f_i' = (1-s) f_i/factor + s f_i
"""
from __future__ import annotations

import math

import torch

from .registry import POSITIONS, Part


def rotary_inv_freq(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    half = head_dim // 2
    f = torch.tensor([theta ** (-(2.0 * i) / head_dim) for i in range(half)], dtype=torch.float64)
    if not scaling:
        return f
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    out = f.clone()
    for i in range(half):
        fi = f[i].item()
        wavelen = 2.0 * math.pi / fi
        if wavelen < orig / high:
            continue
        if wavelen > orig / low:
            out[i] = fi / factor
        else:
            s = (orig / wavelen - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


@POSITIONS.register("rotary")
class Rotary(Part):
    """params: head_dim, theta, scaling (None or the llama3 dict), max_positions."""

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.head_dim = int(self._need("head_dim"))
        if self.head_dim % 2:
            raise ValueError(f"rotary: head_dim {self.head_dim} must be even")
        self.max_positions = int(self._need("max_positions"))
        self.inv_freq = rotary_inv_freq(self.head_dim, float(self._need("theta")), self.params.get("scaling"))
        self.cos = self.sin = None

    def tables(self):
        """(cos, sin), float32 [max_positions, head_dim/2] on the device."""
        if self.cos is None:
            pos = torch.arange(self.max_positions, dtype=torch.float64)
            ang = pos[:, None] * self.inv_freq[None, :]
            self.cos = torch.cos(ang).to(torch.float32).to(self.rt.device).contiguous()
            self.sin = torch.sin(ang).to(torch.float32).to(self.rt.device).contiguous()
        return self.cos, self.sin


@POSITIONS.register("none")
class NoPosition(Part):
    """No position encoding: queries and keys are used as projected."""

    def tables(self):
        return None, None
