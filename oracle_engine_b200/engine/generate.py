"""The generation loop above the step function.

Requests (token-id prompts of unequal length) are taken in batches.  A batch starts
together: all its prompts go through one step, which yields each sequence's first new
token; after that every still-active sequence brings one token per step.  A sequence ends
on a stop token (which is not emitted), at `n_predict` new tokens, or when its slot is
full; it then drops out of the following steps while the others go on.  When the whole
batch has ended its slots are given back and the next batch starts in them.

The loop is written against a small backend interface (alloc / free / step / sample) so
that its decisions can be tested without a GPU.  Reference: `Engine::generate`,
core/engine.cpp:83-148 (prefill, then sample / stop check / emit per token); the
reference takes one request at a time and feeds the last prompt token through its decode
path, where this loop reads the first logits from the prompt step itself.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .batch import SequenceStep


@dataclass
class GenerationResult:
    tokens: list = field(default_factory=list)
    finish_reason: str = ""           # "stop", "length", "context"


class GenerationBackend:
    """What the loop needs from an engine."""
    max_seq_len: int

    def alloc(self, request_index: int, prompt, params) -> int: ...
    def free(self, slot: int) -> None: ...
    def step(self, seqs) -> object: ...                     # logits for the wanted rows
    def sample(self, logits, slots, params) -> list: ...    # one token id per row, on the host


def run_generation(backend: GenerationBackend, prompts, params, batch_size: int | None = None,
                   stop_ids=(), on_token=None) -> list[GenerationResult]:
    params.validate()
    prompts = [list(p) for p in prompts]
    for i, p in enumerate(prompts):
        if not p:
            raise ValueError(f"request {i}: an empty prompt cannot be generated from")
        if len(p) > backend.max_seq_len:
            raise ValueError(f"request {i}: prompt of {len(p)} tokens exceeds the context of "
                             f"{backend.max_seq_len}")
    stop = set() if params.ignore_eos else set(stop_ids if params.stop_ids is None else params.stop_ids)
    results = [GenerationResult() for _ in prompts]
    if batch_size is None or batch_size < 1:
        batch_size = max(1, len(prompts))
    for b0 in range(0, len(prompts), batch_size):
        batch = list(range(b0, min(len(prompts), b0 + batch_size)))
        slots: dict[int, int] = {}
        try:
            for i in batch:
                slots[i] = backend.alloc(i, prompts[i], params)
            if params.n_predict == 0:
                for i in batch:
                    results[i].finish_reason = "length"
                continue
            length = {i: len(prompts[i]) for i in batch}
            active = list(batch)
            seqs = [SequenceStep(slots[i], prompts[i], [len(prompts[i]) - 1]) for i in active]
            while active:
                logits = backend.step(seqs)
                tokens = backend.sample(logits, [slots[i] for i in active], params)
                nxt, seqs = [], []
                for i, tok in zip(active, tokens):
                    tok = int(tok)
                    if tok in stop:
                        results[i].finish_reason = "stop"
                        continue
                    results[i].tokens.append(tok)
                    if on_token is not None:
                        on_token(i, tok)
                    if len(results[i].tokens) >= params.n_predict:
                        results[i].finish_reason = "length"
                    elif length[i] + 1 > backend.max_seq_len:
                        results[i].finish_reason = "context"
                    else:
                        length[i] += 1
                        nxt.append(i)
                        seqs.append(SequenceStep(slots[i], [tok], [0]))
                active = nxt
        finally:
            for s in slots.values():
                backend.free(s)
    return results
