"""The sampler: picks one token per row of logits on the device.

Order of operations as in the reference (core/sampler.cpp:91-97): repeat penalty over the
last `repeat_last_n` recorded tokens, temperature, then first-maximum argmax if the
temperature is <= 0, else softmax, top-k, top-p and one draw.  Its per-sequence state
(generator seed, number of draws, ring of recent tokens) lives in the fixed-size state
store, one row per slot, so that a sequence's draws do not depend on what else is in the
batch.  The kernels are in csrc/sampling.cu.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..parts.spec import StateNeed

OWNER = "sampler"
HISTORY_CAPACITY = 256        # most recent tokens kept per sequence for the repeat penalty


class Sampler:
    def __init__(self, state_store, device):
        self.device = device
        self.rng_seed = state_store.add(OWNER, "rng_seed", StateNeed((), torch.int64))
        self.rng_counter = state_store.add(OWNER, "rng_counter", StateNeed((), torch.int32))
        self.hist = state_store.add(OWNER, "history", StateNeed((HISTORY_CAPACITY,), torch.int32))
        self.hist_count = state_store.add(OWNER, "history_count", StateNeed((), torch.int32))

    def start_sequence(self, slot: int, seed: int, prompt, params) -> None:
        """Seeds the slot's generator and records the prompt without its last token, as
        the reference does before generating (core/engine.cpp:118-122)."""
        self.rng_seed[slot] = int(seed)
        self.rng_counter[slot] = 0
        recorded = list(prompt[:-1])
        if params.repeat_penalty > 1.0 and recorded:
            if params.repeat_last_n > HISTORY_CAPACITY:
                raise ValueError(f"repeat_last_n {params.repeat_last_n} exceeds the {HISTORY_CAPACITY} tokens kept")
            tail = recorded[-HISTORY_CAPACITY:]
            count = len(recorded)
            ring = torch.zeros(HISTORY_CAPACITY, dtype=torch.int32)
            for j, tok in enumerate(tail):
                ring[(count - len(tail) + j) % HISTORY_CAPACITY] = int(tok)
            self.hist[slot].copy_(ring)
            self.hist_count[slot] = count
        else:
            self.hist_count[slot] = 0

    def sample(self, logits: torch.Tensor, row_slot: torch.Tensor, params, out: torch.Tensor | None = None):
        """logits float32 [R, V] (overwritten unless greedy without penalty); row_slot int32 [R].
        Returns int32 [R] on the device."""
        R = logits.shape[0]
        if out is None:
            out = torch.empty(R, dtype=torch.int32, device=logits.device)
        if params.temperature <= 0.0 and params.repeat_penalty <= 1.0:
            ops.argmax_rows(logits, out)
            return out
        use_hist = params.repeat_penalty > 1.0
        ops.sample_rows(logits, out, row_slot, params.temperature, params.top_k, params.top_p,
                        params.repeat_penalty, params.repeat_last_n, self.rng_seed, self.rng_counter,
                        self.hist if use_hist else None, self.hist_count if use_hist else None, record=True)
        return out
