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
# What consecutive kernels gain by overlapping is a third of a decode step, and which flags give it
# depends on the kernels' forms, so the four products of a block take theirs from this table, found by
# varying one product at a time inside the 28-layer model (3B shape; ms a step at 1 / 8 / 16 sequences:
# 1.60 / 1.71 / 2.11 with these, 2.38 at 16 with the flags of 8 and the tcgen05 kernel for the large weights).
_CHAIN_FLAGS = {
    # product:   up to 8 tokens,               9 to 16 tokens
    "mixer_in":  (START_EARLY,                 START_EARLY),
    "mixer_out": (START_EARLY | TRIGGER_LATE,  TRIGGER_LATE),
    "ffn_in":    (START_EARLY | TRIGGER_LATE,  START_EARLY | TRIGGER_LATE),
    "ffn_out":   (START_EARLY,                 START_EARLY | TRIGGER_LATE),
}


def chain_flags(product: str, n_tokens: int) -> int:
    """START_EARLY / TRIGGER_LATE for one of a block's four products in a step of n_tokens rows."""
    return _CHAIN_FLAGS[product][0 if n_tokens <= 8 else 1]


def matmul_nt(rt, out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, accumulate: bool = False,
              early: int = 0, then: torch.Tensor | None = None) -> None:
    """early: START_EARLY and TRIGGER_LATE flags (above); other kernels ignore them.
    then: the weight matrix of the product that runs after this one (a hint, see ops_tc.gemm)."""
    if rt.dtype == torch.bfloat16 and rt.tensor_cores:
        from ..csrc import ops_tc
        if ops_tc.gemm_supported(a, w, out):
            ops_tc.gemm(out, a, w, accumulate=accumulate, early=int(early), then=then)
            return
    ops.gemm_simple(out, a, w, accumulate=accumulate)
