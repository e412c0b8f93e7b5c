"""What every part is built with: the compute precision and the device.

`dtype` is the type of activations, matrix weights and the cache: bfloat16 (serving; the
tensor-core kernels) or float32 (the true 32-bit path: CUDA-core products, no reduced-
precision mode anywhere).  The residual stream, norms, softmax, rotary tables and logits
are float32 in both.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {name}")
        return name
    try:
        return DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {name!r}") from None


@dataclass
class Runtime:
    dtype: torch.dtype
    device: torch.device
    tensor_cores: bool = True          # bf16 only: use the tcgen05 / mma kernels where they take the shape
    # A hint for the part that runs now: the weight matrix that the part after it streams first (or
    # None).  The model and the block set it before they call a part; a part's last product may ask
    # the first megabytes of it into the L2 while its own epilogue runs (csrc/ops_tc.py: gemm(then=)).
    next_weights: torch.Tensor | None = None

    def empty(self, *shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)

    def to_compute(self, t: torch.Tensor) -> torch.Tensor:
        """A stored matrix in the compute dtype (bf16 -> float32 is exact; a 32-bit
        matrix is rounded to bf16 only for the bf16 path)."""
        return t.to(device=self.device, dtype=self.dtype).contiguous()

    def to_f32(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.device, dtype=torch.float32).contiguous()
