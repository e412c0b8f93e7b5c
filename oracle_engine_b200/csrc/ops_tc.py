"""Entry points of the tensor-core kernels (bfloat16 serving path)."""
from __future__ import annotations


def gemm_supported(a, w, out) -> bool:
    return False


def attention_supported(head_dim, n_heads, n_kv_heads) -> bool:
    return False
