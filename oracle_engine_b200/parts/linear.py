"""out (+)= a @ w.T for the parts: picks the kernel by precision and shape.

bfloat16 goes to the tensor-core kernels (csrc/gemm_tcgen05.cu) where they take the shape;
float32, and shapes those kernels refuse, go to the CUDA-core kernel (csrc/gemm_simple.cu).
The choice depends only on the runtime and on the weight's shape, never on the data.
Role of the reference's projections through `gemm_q` / `gemv_q` / `ops::matmul`
(core/model.cpp:370-381, 537-547).
"""
from __future__ import annotations

import torch

from ..csrc import ops


def matmul_nt(rt, out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, accumulate: bool = False,
              early: bool = False) -> None:
    """early: the product may start while the kernel before it drains (see csrc/gemm_skinny.cu)."""
    if rt.dtype == torch.bfloat16 and rt.tensor_cores:
        from ..csrc import ops_tc
        if ops_tc.gemm_supported(a, w, out):
            ops_tc.gemm(out, a, w, accumulate=accumulate, early=early)
            return
    ops.gemm_simple(out, a, w, accumulate=accumulate)
