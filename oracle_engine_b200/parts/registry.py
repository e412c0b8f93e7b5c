"""Registries of the kinds of parts a layer is built from, and the interface of each.

A part is a class registered under a name; a `PartSpec(kind, params)` picks it.  All
parts are built as `cls(params, prefix, runtime)` where `params` holds every size and
constant the part needs, `prefix` is the tensor-name prefix of its layer and `runtime`
(engine/runtime.py) gives the compute dtype and device.  No part knows which model it is
in.  Interfaces:

Every part
    tensors() -> list[TensorDecl]        weights it reads (full names, shapes)
    load(get)                            takes them: get(name) -> CUDA tensor as stored
                                         (bfloat16, or float32 if the file holds 32-bit)
    weight_bytes(), cache_bytes_per_query(context), flops(start, count)
                                         what it reads and computes (for rooflines; default 0)

Mixer  (MIXERS; e.g. attention)
    cache_need() -> CacheNeed | None     what it keeps per token in the paged cache
    state_need() -> dict[str, StateNeed] fixed-size per-sequence state it keeps
    forward(h, residual, ctx, cache, state, owns_cache)
        h        [T, hidden] activations (compute dtype) of the step's tokens
        residual [T, hidden] float32; the mixer ADDS its output into it
        ctx      StepContext (engine/batch.py): per-token sequence index and position,
                 per-sequence slot / start / length, the group's page tables
        cache    CacheView: the entry's tensors as its CacheNeed declared them (attention:
                 cache.kv [pages, 2, kv_heads, PAGE, head_dim]) and the page tables
        state    dict name -> tensor [slots, *shape] (index rows with ctx.seq_slot)
        owns_cache  False when the entry reads another entry's cache (write nothing)

FeedForward  (FEED_FORWARDS; dense or routed)
    forward(h, residual, ctx)            adds its output into residual

Norm  (NORMS)
    forward(x) -> tensor                 x float32 [T, hidden] -> compute dtype

PositionEncoding  (POSITIONS)            built once per model and name, shared by mixers
    tables(max_positions)                whatever its mixers read (e.g. cos/sin tables)

Block  (BLOCKS)                          the arrangement of mixer, feed-forward and norms
    forward(x, ctx, cache, state, owns_cache)   x float32 [T, hidden], updated in place
"""
from __future__ import annotations


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._items: dict[str, type] = {}

    def register(self, name: str):
        def deco(cls):
            if name in self._items:
                raise ValueError(f"{self.what} {name!r} is already registered")
            self._items[name] = cls
            cls.kind = name
            return cls
        return deco

    def unregister(self, name: str) -> None:
        self._items.pop(name, None)

    def get(self, name: str) -> type:
        try:
            return self._items[name]
        except KeyError:
            known = ", ".join(sorted(self._items)) or "(none)"
            raise KeyError(f"unknown {self.what} {name!r}; registered: {known}") from None

    def names(self):
        return sorted(self._items)

    def __contains__(self, name):
        return name in self._items


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
BLOCKS = Registry("block arrangement")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("output head")


class Part:
    """Base of every part: holds params, prefix and runtime; no weights by default."""
    kind = "?"

    def __init__(self, params: dict, prefix: str, runtime):
        self.params = dict(params)
        self.prefix = prefix
        self.rt = runtime

    def tensors(self):
        return []

    def load(self, get) -> None:
        pass

    def cache_need(self):
        return None

    def state_need(self):
        return {}

    # What a part costs, for rooflines (a bench sums these over the model; it needs no knowledge of
    # the architecture).  Defaults: a part that streams no weights and computes next to nothing.
    def weight_bytes(self) -> int:
        """Bytes of weights the part reads in a step, whatever the number of tokens."""
        return 0

    def cache_bytes_per_query(self, context: int) -> int:
        """Bytes of cache a mixer reads for ONE sequence whose newest token sees `context` positions."""
        return 0

    def flops(self, start: int, count: int) -> float:
        """Floating-point operations for `count` tokens of one sequence at positions start ..
        start + count - 1 (each sees the positions up to its own)."""
        return 0.0

    def _need(self, key: str):
        try:
            return self.params[key]
        except KeyError:
            raise KeyError(f"{type(self).__name__} ({self.kind}) needs parameter {key!r}") from None
