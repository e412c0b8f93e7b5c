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

    # ------------------------------------------------------------------ what a step costs
    def step_bytes(self, contexts) -> int:
        """Bytes a step has to read from memory: every weight it uses once, and for each of its
        sequences (newest token at `contexts[i]` positions) the cache that every schedule entry's
        mixer reads.  Summed from the parts; the roofline of a decode step."""
        weights = sum(p.weight_bytes() for p in self._all_parts())
        cache = 0
        for e in self.schedule:
            mixer = self.layers[e.layer].mixer
            cache += sum(mixer.cache_bytes_per_query(int(c)) for c in contexts)
        return int(weights + cache)

    def step_flops(self, starts, counts, n_want) -> float:
        """Floating-point operations of a step whose sequence i brings counts[i] tokens on top of
        starts[i] cached ones, with the head applied to n_want rows."""
        total = 0.0
        for e in self.schedule:
            for part in self.layers[e.layer].parts():
                total += sum(part.flops(int(st), int(n)) for st, n in zip(starts, counts))
        return total + self.head.flops(0, n_want)

    # ------------------------------------------------------------------ one step
    def forward(self, ctx, cache_views, state_views):
        """Runs the step's tokens through the schedule; returns float32 logits
        [n_want, vocab] at ctx.want_rows, or None if nothing is wanted."""
        x = self.embed(ctx)
        self.run_entries(x, ctx, cache_views, state_views, 0, len(self.schedule))
        return self.logits(x, ctx)

    # The forward pass in stages: stage 0 is the embedding, stage 1 + i schedule entry i, the last
    # stage the final norm and head.  `stages()` groups them into runs that can (or cannot) be
    # captured in a CUDA graph, so that one part that must run eagerly (a mixer that reads its state
    # on the host, say) does not take the graphs away from every other layer.
    def embed(self, ctx, out=None):
        return self.embedding.forward(ctx.token_ids, ctx.n_tokens, out)

    def run_entries(self, x, ctx, cache_views, state_views, lo: int, hi: int) -> None:
        for i in range(lo, hi):
            e = self.schedule[i]
            owner = i if e.cache_from is None else e.cache_from
            # a hint for the entry's last product: the weights the next entry streams first
            nxt = self.layers[self.schedule[i + 1].layer] if i + 1 < len(self.schedule) else None
            first = getattr(nxt, "first_weights", None)
            self.rt.next_weights = first() if first is not None else None
            self.layers[e.layer].forward(x, ctx, cache_views[owner], state_views[i], e.cache_from is None)
        self.rt.next_weights = None

    def logits(self, x, ctx):
        if ctx.n_want == 0:
            return None
        xr = self.rt.empty(ctx.n_want, x.shape[1], dtype=torch.float32)
        ops.gather_rows_f32(xr, x, ctx.want_rows)
        return self.head.forward(self.final_norm.forward(xr))

    def stages(self) -> list[tuple[bool, int, int]]:
        """[(graph_safe, first stage, one past the last stage)]: maximal runs of stages that are all
        safe to capture in a CUDA graph, or all not."""
        ok = lambda parts: all(getattr(p, "graph_safe", False) for p in parts)          # noqa: E731
        flags = [ok([self.embedding])] + [ok(self.layers[e.layer].parts()) for e in self.schedule] + \
                [ok([self.final_norm, self.head])]
        runs, lo = [], 0
        for i in range(1, len(flags) + 1):
            if i == len(flags) or flags[i] != flags[lo]:
                runs.append((flags[lo], lo, i))
                lo = i
        return runs

    def run_stages(self, x, ctx, cache_views, state_views, lo: int, hi: int):
        """Runs stages lo .. hi - 1 on the residual stream `x` (stage 0 fills it); returns the
        logits if the last stage is among them, else None."""
        n = len(self.schedule)
        if lo == 0:
            self.embed(ctx, out=x)
        self.run_entries(x, ctx, cache_views, state_views, max(lo, 1) - 1, min(hi, n + 1) - 1)
        return self.logits(x, ctx) if hi == n + 2 else None
