"""Which attention kernels a step uses: chosen by precision, head size and whether the
step is a prompt or single decoded tokens; never by the data.

float32, and head sizes the tensor-core kernels do not take, use the one-path kernel of
csrc/attention.cu; bfloat16 uses the tensor-core prefill kernel and the split-KV decode
kernel of csrc/attention_mma.cu.
"""
from __future__ import annotations

import torch

from ..csrc import ops


def rope_and_cache(rt, qkv, cos, sin, cache, ctx, H, KVH, hd, owns_cache) -> None:
    ops.rope_kv_write(qkv, cos, sin, cache.storage if owns_cache else None, cache.tables, ctx.tok_seq,
                      ctx.tok_pos, H, KVH, hd, owns_cache)


def attend(rt, out, qkv, cache, ctx, H, KVH, hd, window, scale) -> None:
    if rt.dtype == torch.bfloat16 and rt.tensor_cores:
        from ..csrc import ops_tc
        if ops_tc.attention_supported(hd, H, KVH):
            ops_tc.attention(out, qkv, cache.storage, cache.tables, ctx, H, KVH, hd, window, scale)
            return
    ops.attn_paged(out, qkv, cache.storage, cache.tables, ctx.tok_seq, ctx.tok_pos, H, KVH, hd, window, scale)
