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


# How a product for a handful of tokens (the weight-streaming kernel, csrc/gemm_skinny.cu) is
# chained to its neighbours in the stream:
START_EARLY = 1     # it may start, and request its first weights, while the kernel before it drains
TRIGGER_LATE = 2    # the kernel after it may be scheduled only when its CTAs have streamed their weights
# A kernel that starts early behind a long kernel whose trigger comes at its top sits on the SMs
# while that kernel still needs them: START_EARLY belongs behind a short kernel or a TRIGGER_LATE one.


def matmul_nt(rt, out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, accumulate: bool = False,
              early: int = 0) -> None:
    """early: START_EARLY and TRIGGER_LATE flags (above); other kernels ignore them."""
    if rt.dtype == torch.bfloat16 and rt.tensor_cores:
        from ..csrc import ops_tc
        if ops_tc.gemm_supported(a, w, out):
            ops_tc.gemm(out, a, w, accumulate=accumulate, early=int(early))
            return
    ops.gemm_simple(out, a, w, accumulate=accumulate)
