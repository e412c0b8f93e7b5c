"""The data description of a model: which parts make each layer, and in what order the
layers run.

An architecture's `build_spec(config)` returns a `ModelSpec`.  Nothing below it knows
which model it is in: every part gets its sizes and constants from its `PartSpec`.

* `PartSpec(kind, params)` names a registered part (parts/registry.py) and its parameters.
* `LayerSpec` puts a mixer, a feed-forward and their norms together in an arrangement
  (`block`), under a tensor-name prefix.  Layers may differ from one another.
* `ModelSpec.schedule` is the order in which layers run: a list of `ScheduleEntry`.  An
  entry may name a layer that another entry also names (the weights are shared; each entry
  still has a cache of its own), and `cache_from` lets an entry read the cache that an
  earlier entry wrote instead of writing one (it then computes no keys or values).

The reference has one fixed arrangement, x += Attn(RMSNorm(x)); x += FFN(RMSNorm(x)),
L times (core/model.cpp:361-474); here that order is the data a Llama spec holds.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class TensorDecl:
    """A weight a part needs: full name in the file, shape, and how random weights fill it
    ("normal": N(0, std); "ones_normal": 1 + N(0, norm_std))."""
    name: str
    shape: tuple[int, ...]
    init: str = "normal"


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: dict = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    prefix: str                        # e.g. "model.layers.3."
    mixer: PartSpec
    feed_forward: Optional[PartSpec]
    mixer_norm: PartSpec
    ffn_norm: Optional[PartSpec]
    block: str = "pre_norm"            # arrangement of the four (parts/block.py)


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int                         # index into ModelSpec.layers
    cache_from: Optional[int] = None   # index of an earlier schedule entry whose cache is read


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer keeps per token in the paged cache.

    `tensors`: ((name, per-token shape), ...), one entry per tensor the mixer keeps.  A tensor
    whose per-token shape is (a, ..., z) is stored per page as [a, ..., PAGE, z] (the page's
    tokens run along the last but one axis, so that a token's innermost vector is contiguous
    and a page of one outer index is one block).  Attention keeps one tensor "kv" of shape
    (2, kv_heads, head_dim); a mixer that keeps one latent vector per token would declare
    (("latent", (rank,)),), keys and values of different widths two tensors.
    `kind`: "full" (every position) or "window" (the last `window` of them; older pages are
    given back).  Entries with equal needs share one group of storage and page tables."""
    kind: str
    tensors: tuple
    window: int = 0

    def elements_per_token(self) -> int:
        n = 0
        for _, shape in self.tensors:
            e = 1
            for d in shape:
                e *= int(d)
            n += e
        return n


def attention_cache_need(kv_heads: int, head_dim: int, window: int = 0) -> CacheNeed:
    """Keys and values of grouped-query attention: one tensor "kv", per page [2, kv_heads, PAGE, head_dim]."""
    return CacheNeed("window" if window else "full", (("kv", (2, int(kv_heads), int(head_dim))),), int(window))


@dataclass(frozen=True)
class StateNeed:
    """Per-sequence state of fixed size that a part keeps: one tensor of `shape` per
    sequence, zeroed when a sequence starts."""
    shape: tuple[int, ...]
    dtype: Any                         # torch dtype


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    final_norm: PartSpec
    head: PartSpec
    positions: dict                    # name -> PartSpec of a position encoding
    layers: tuple
    schedule: tuple
    stop_ids: tuple = ()
    bos_id: Optional[int] = None
    ignored_tensors: tuple = ()        # name suffixes a file may hold that the model does not read

    def __post_init__(self):
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule[{i}] names layer {e.layer}, there are {len(self.layers)}")
            if e.cache_from is not None:
                if not 0 <= e.cache_from < i:
                    raise ValueError(f"schedule[{i}].cache_from must name an earlier entry, got {e.cache_from}")
                if self.schedule[e.cache_from].cache_from is not None:
                    raise ValueError(f"schedule[{i}].cache_from names an entry that owns no cache")
