"""Arrangements of a layer's parts.  `pre_norm`: x += mixer(norm(x)); x += ffn(norm(x)),
the reference's layer (core/model.cpp:361-474).  The mixer and the feed-forward add their
outputs into the float32 residual stream themselves (fused into their last product)."""
from __future__ import annotations

from .registry import BLOCKS


@BLOCKS.register("pre_norm")
class PreNormBlock:
    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.ffn_norm = ffn_norm

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward) if p is not None]

    def first_weights(self):
        """The weight matrix this block streams first (a hint for the part that runs before it), or None."""
        return _first_weights(self.mixer)

    def forward(self, x, ctx, cache, state, owns_cache=True):
        rt = getattr(self.mixer, "rt", None)
        after = getattr(rt, "next_weights", None)          # what the model says comes after this block
        h = self.mixer_norm.forward(x)
        if rt is not None:
            rt.next_weights = _first_weights(self.feed_forward) if self.feed_forward is not None else after
        self.mixer.forward(h, x, ctx, cache, state, owns_cache)
        if self.feed_forward is not None:
            h = self.ffn_norm.forward(x)
            if rt is not None:
                rt.next_weights = after
            self.feed_forward.forward(h, x, ctx)
        if rt is not None:
            rt.next_weights = None


def _first_weights(part):
    f = getattr(part, "first_weights", None)
    return f() if f is not None else None
