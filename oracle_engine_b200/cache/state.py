"""Per-sequence state of fixed size, beside the cache: one row per slot.

Parts that keep state which does not grow with the sequence (a recurrent or
convolutional mixer's state, for instance) declare it with `state_need()`; the sampler
keeps its random-number counter and its window of recent tokens here too.  Each declared
tensor is stored as [slots, *shape] on the device and its row is zeroed when a slot is
handed to a new sequence.  The Llama decoder's own mixers declare none.

In the reference this is loop state of `Engine::generate` and members of `Sampler`
(core/engine.cpp:118-138, core/sampler.hpp:41-43).
"""
from __future__ import annotations

import torch


class StateStore:
    def __init__(self, n_slots: int, device):
        self.n_slots = n_slots
        self.device = device
        self._tensors: dict[tuple, torch.Tensor] = {}

    def add(self, owner, name: str, need) -> torch.Tensor:
        key = (owner, name)
        if key in self._tensors:
            raise ValueError(f"state {key} is declared twice")
        t = torch.zeros((self.n_slots, *need.shape), dtype=need.dtype, device=self.device)
        self._tensors[key] = t
        return t

    def views(self, owner) -> dict[str, torch.Tensor]:
        return {name: t for (o, name), t in self._tensors.items() if o == owner}

    def get(self, owner, name: str) -> torch.Tensor:
        return self._tensors[(owner, name)]

    def reset(self, slot: int) -> None:
        for t in self._tensors.values():
            t[slot].zero_()

    def total_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._tensors.values())
