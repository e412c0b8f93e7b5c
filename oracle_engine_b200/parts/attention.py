"""Mixer `gqa_attention`: grouped-query attention over the paged cache.

q = Wq h, k = Wk h, v = Wv h (no bias); q and k rotated by the position encoding; k and
v written to the token's row of the cache; query head h attends through KV head
h // (H/KVH) to the keys of its own sequence up to its own position (all of them, or the
last `window`); x += Wo o.  Reference: core/model.cpp:370-444 (decode) and :570-630
(prefill); here one code path serves both, reading keys and values from the cache.

The three projections are fused into one matrix product at load ([Wq; Wk; Wv]); an entry
that reads another entry's cache projects q only.
"""
from __future__ import annotations

import math

import torch

from ..csrc import ops
from .linear import chain_flags, matmul_nt
from .registry import MIXERS, Part
from .spec import TensorDecl, attention_cache_need

_NAMES = {"q": "self_attn.q_proj.weight", "k": "self_attn.k_proj.weight", "v": "self_attn.v_proj.weight",
          "o": "self_attn.o_proj.weight"}


@MIXERS.register("gqa_attention")
class GQAAttention(Part):
    graph_safe = True
    """params: hidden_size, num_heads, num_kv_heads, head_dim, position (a position
    encoding object or None), window (0 = all keys), scale (default head_dim^-1/2),
    tensor_names (optional overrides of q/k/v/o names under the prefix)."""

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D = int(self._need("hidden_size"))
        self.H = int(self._need("num_heads"))
        self.KVH = int(self._need("num_kv_heads"))
        self.hd = int(self._need("head_dim"))
        if self.H % self.KVH:
            raise ValueError(f"gqa_attention: {self.H} heads are not a multiple of {self.KVH} KV heads")
        if self.hd % 2 or not 2 <= self.hd <= ops.MAX_HEAD_DIM:
            raise ValueError(f"gqa_attention: head_dim {self.hd} is outside what the attention kernels take "
                             f"(even, 2..{ops.MAX_HEAD_DIM})")
        self.window = int(self.params.get("window", 0) or 0)
        self.scale = float(self.params.get("scale") or 1.0 / math.sqrt(self.hd))
        self.position = self.params.get("position")
        self.names = {k: prefix + v for k, v in {**_NAMES, **self.params.get("tensor_names", {})}.items()}
        self.w_qkv = self.w_o = None

    def tensors(self):
        q, kv = self.H * self.hd, self.KVH * self.hd
        return [TensorDecl(self.names["q"], (q, self.D)), TensorDecl(self.names["k"], (kv, self.D)),
                TensorDecl(self.names["v"], (kv, self.D)), TensorDecl(self.names["o"], (self.D, q))]

    def load(self, get):
        to = self.rt.to_compute
        self.w_qkv = torch.cat([to(get(self.names["q"])), to(get(self.names["k"])), to(get(self.names["v"]))], 0)
        self.w_o = to(get(self.names["o"]))

    def cache_need(self):
        return attention_cache_need(self.KVH, self.hd, self.window)

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o) if t is not None)

    def cache_bytes_per_query(self, context):
        seen = min(context, self.window) if self.window else context
        return seen * 2 * self.KVH * self.hd * (2 if self.rt.dtype == torch.bfloat16 else 4)

    def flops(self, start, count):
        products = 2.0 * self.D * (2 * self.H + 2 * self.KVH) * self.hd        # q, k, v and o projections
        # positions seen by the tokens: sum over t = start + 1 .. start + count of t (or min(t, window))
        first, last = start + 1, start + count
        tri = lambda a, b: (a + b) * (b - a + 1) / 2.0 if b >= a else 0.0      # noqa: E731
        if self.window:
            w = self.window
            seen = tri(first, min(last, w)) + w * max(0, last - max(first, w + 1) + 1)
        else:
            seen = tri(first, last)
        return count * products + 4.0 * self.H * self.hd * seen                  # q.k and p.v

    def first_weights(self):
        return self.w_qkv

    def forward(self, h, residual, ctx, cache, state, owns_cache=True):
        T = h.shape[0]
        q_width = self.H * self.hd
        width = q_width + (2 * self.KVH * self.hd if owns_cache else 0)
        qkv = self.rt.empty(T, width)
        # how the products are chained to their neighbours in the stream: parts/linear.py
        matmul_nt(self.rt, qkv, h, self.w_qkv[:width], early=chain_flags("mixer_in", T))
        cos, sin = self.position.tables() if self.position is not None else (None, None)
        from . import attention_dispatch as ad
        o = self.rt.empty(T, q_width)
        ad.mixer_core(self.rt, o, qkv, cos, sin, cache, ctx, self.H, self.KVH, self.hd, self.window, self.scale,
                      owns_cache)
        matmul_nt(self.rt, residual, o, self.w_o, accumulate=True, early=chain_flags("mixer_out", T),
                  then=self.rt.next_weights)
