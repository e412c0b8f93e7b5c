"""The generation loop above the step function.

Requests (token-id prompts of unequal length) are taken in batches.  A batch starts
together: all its prompts go through one step, which yields each sequence's first new
token; after that every still-active sequence brings one token per step.  A sequence ends
on a stop token (which is not emitted), at `n_predict` new tokens, or when its slot is
full; it then drops out of the following steps while the others go on.  When the whole
batch has ended its slots are given back and the next batch starts in them.

With a backend that supports it the loop runs one step ahead of the host: the next step is
queued, fed with the sampled tokens where they lie on the device, before the host has read
those tokens, so the device does not idle while the host decides.  The tokens, their order
and the finish reasons are the same either way.

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

    # A backend that can run one step ahead of the host sets `supports_lookahead` and has:
    #   sample_async(logits, slots, params) -> handle     sampling started, tokens not yet read
    #   read(handle) -> list                               the tokens of that sampling, on the host
    #   step_ahead(slots, handle) -> logits                one token further for these sequences,
    #                                                      fed with the handle's tokens where they lie
    supports_lookahead = False


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
    lookahead = bool(getattr(backend, "supports_lookahead", False))
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

            def accept(i, tok) -> bool:
                """Takes request i's next sampled token; True if the request goes on."""
                if tok in stop:
                    results[i].finish_reason = "stop"
                    return False
                results[i].tokens.append(tok)
                if on_token is not None:
                    on_token(i, tok)
                if len(results[i].tokens) >= params.n_predict:
                    results[i].finish_reason = "length"
                    return False
                if length[i] + 1 > backend.max_seq_len:
                    results[i].finish_reason = "context"
                    return False
                length[i] += 1
                return True

            def ends_by_count(i) -> bool:
                """Request i ends with its next token whatever that token is."""
                return len(results[i].tokens) + 1 >= params.n_predict or length[i] + 1 > backend.max_seq_len

            while active:
                logits = backend.step(seqs)
                act_slots = [slots[i] for i in active]
                if not lookahead:
                    tokens = [int(t) for t in backend.sample(logits, act_slots, params)]
                    went_on = [accept(i, t) for i, t in zip(active, tokens)]
                    seqs = [SequenceStep(slots[i], [t], [0]) for i, t, ok in zip(active, tokens, went_on) if ok]
                    active = [i for i, ok in zip(active, went_on) if ok]
                    continue
                # One step ahead: while the host still waits for the tokens of step k, step k + 1 of
                # the same sequences is already queued, fed with those tokens where they lie.  It
                # is queued only if no sequence can end by its count; a stop token that ends one all
                # the same leaves a step that ran with a row too many, whose other rows stand
                # (a row does not depend on the rest of the batch).
                pending = backend.sample_async(logits, act_slots, params)
                while True:
                    ahead = None
                    if not any(ends_by_count(i) for i in active):
                        ahead = backend.sample_async(backend.step_ahead(act_slots, pending), act_slots, params)
                    tokens = [int(t) for t in backend.read(pending)]
                    went_on = [accept(i, t) for i, t in zip(active, tokens)]
                    if ahead is not None and all(went_on):
                        pending = ahead
                        continue
                    if ahead is not None:
                        tokens = [int(t) for t in backend.read(ahead)]
                        went_on = [ok and accept(i, t) for i, t, ok in zip(active, tokens, went_on)]
                    seqs = [SequenceStep(slots[i], [t], [0]) for i, t, ok in zip(active, tokens, went_on) if ok]
                    active = [i for i, ok in zip(active, went_on) if ok]
                    break
        finally:
            for s in slots.values():
                backend.free(s)
    return results
