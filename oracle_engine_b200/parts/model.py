"""DecoderModel: a ModelSpec built into parts, and the forward pass of one step.

The model is generic: it reads a `ModelSpec` (parts/spec.py), builds every part through
the registries and runs the layers in the order the schedule gives.  It holds no sizes of
its own and does not know which architecture the spec came from.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .registry import BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS
from .spec import ModelSpec, TensorDecl

# importing the modules registers the built-in parts
from . import attention, block, embedding, feedforward, norms, positions  # noqa: F401,E402


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime):
        self.spec = spec
        self.rt = runtime
        self.positions = {name: POSITIONS.get(ps.kind)(ps.params, "", runtime)
                          for name, ps in spec.positions.items()}
        self.embedding = EMBEDDINGS.get(spec.embedding.kind)(spec.embedding.params, "", runtime)
        head_params = dict(spec.head.params, embedding=self.embedding)
        self.head = HEADS.get(spec.head.kind)(head_params, "", runtime)
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm.params, "", runtime)
        self.layers = [self._build_layer(ls) for ls in spec.layers]
        self.schedule = list(spec.schedule)

    def _build_layer(self, ls):
        mparams = dict(ls.mixer.params)
        if isinstance(mparams.get("position"), str):
            mparams["position"] = self.positions[mparams["position"]]
        mixer = MIXERS.get(ls.mixer.kind)(mparams, ls.prefix, self.rt)
        ffn = None if ls.feed_forward is None else \
            FEED_FORWARDS.get(ls.feed_forward.kind)(ls.feed_forward.params, ls.prefix, self.rt)
        mnorm = NORMS.get(ls.mixer_norm.kind)(ls.mixer_norm.params, ls.prefix, self.rt)
        fnorm = None if ls.ffn_norm is None else NORMS.get(ls.ffn_norm.kind)(ls.ffn_norm.params, ls.prefix, self.rt)
        return BLOCKS.get(ls.block)(mixer, ffn, mnorm, fnorm)

    # ------------------------------------------------------------------ weights
    def _all_parts(self):
        parts = [self.embedding, self.final_norm, self.head]
        for layer in self.layers:
            parts.extend(layer.parts())
        return parts

    def tensors(self) -> list[TensorDecl]:
        """Every weight the model reads, each name once."""
        seen: dict[str, TensorDecl] = {}
        for p in self._all_parts():
            for d in p.tensors():
                old = seen.get(d.name)
                if old is not None and old.shape != d.shape:
                    raise ValueError(f"tensor {d.name} is declared with shapes {old.shape} and {d.shape}")
                seen[d.name] = d
        return list(seen.values())

    def load(self, get) -> None:
        for p in self._all_parts():
            p.load(get)
        for pos in self.positions.values():
            pos.tables()

    # ------------------------------------------------------------------ cache / state needs
    def cache_needs(self):
        """Per schedule entry: the CacheNeed of its mixer, or None if it owns no cache."""
        out = []
        for e in self.schedule:
            need = self.layers[e.layer].mixer.cache_need()
            out.append(need if e.cache_from is None else None)
        for i, e in enumerate(self.schedule):
            if e.cache_from is not None:
                mine = self.layers[e.layer].mixer.cache_need()
                if mine != out[e.cache_from]:
                    raise ValueError(f"schedule[{i}] reads the cache of entry {e.cache_from}, whose layout "
                                     f"{out[e.cache_from]} differs from its own {mine}")
        return out

    def state_needs(self):
        """Per schedule entry: dict name -> StateNeed of its mixer."""
        return [dict(self.layers[e.layer].mixer.state_need()) for e in self.schedule]

    # ------------------------------------------------------------------ one step
    def forward(self, ctx, cache_views, state_views):
        """Runs the step's tokens through the schedule; returns float32 logits
        [n_want, vocab] at ctx.want_rows, or None if nothing is wanted."""
        x = self.embedding.forward(ctx.token_ids, ctx.n_tokens)
        for i, e in enumerate(self.schedule):
            owner = i if e.cache_from is None else e.cache_from
            self.layers[e.layer].forward(x, ctx, cache_views[owner], state_views[i], e.cache_from is None)
        if ctx.n_want == 0:
            return None
        xr = self.rt.empty(ctx.n_want, x.shape[1], dtype=torch.float32)
        ops.gather_rows_f32(xr, x, ctx.want_rows)
        return self.head.forward(self.final_norm.forward(xr))
