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

    # Optional: check() raises if the device reported an error since the last call (a bounded wait
    # that ran out, a token id outside the vocabulary); the loop calls it once per batch.

    # A backend that can run one step ahead of the host sets `supports_lookahead` and has:
    #   sample_async(logits, slots, params) -> handle     sampling started, tokens not yet read
    #   read(handle) -> list                               the tokens of that sampling, on the host
    #   step_ahead(slots, handle) -> logits                one token further for these sequences,
    #                                                      fed with the handle's tokens where they lie
    supports_lookahead = False


def run_generation(backend: GenerationBackend, prompts, params, batch_size: int | None = None,
                   stop_ids=(), on_token=None, max_step_tokens: int | None = None) -> list[GenerationResult]:
    """max_step_tokens: the most prompt tokens one step takes (None: every prompt whole, in the
    batch's first step).  With a limit, prompts are cut into portions, in request order: a
    portion that does not end its prompt wants no logits; a request whose prompt is complete
    decodes one token per step in the same steps in which later requests still bring portions;
    a request that got no room in a step is left out of it.  The tokens are the same either way."""
    params.validate()
    prompts = [list(p) for p in prompts]
    for i, p in enumerate(prompts):
        if not p:
            raise ValueError(f"request {i}: an empty prompt cannot be generated from")
        if len(p) > backend.max_seq_len:
            raise ValueError(f"request {i}: prompt of {len(p)} tokens exceeds the context of "
                             f"{backend.max_seq_len}")
    if max_step_tokens is not None and max_step_tokens < 1:
        raise ValueError("max_step_tokens must be at least 1")
    stop = set() if params.ignore_eos else set(stop_ids if params.stop_ids is None else params.stop_ids)
    results = [GenerationResult() for _ in prompts]
    if batch_size is None or batch_size < 1:
        batch_size = max(1, len(prompts))
    lookahead = bool(getattr(backend, "supports_lookahead", False))
    check = getattr(backend, "check", None)
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
            fed = {i: 0 for i in batch}            # prompt tokens given to the step function so far
            last = {}                              # request -> its newest token, to be fed next
            active = list(batch)

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

            def next_step():
                """The next step's sequences and the requests whose logits it yields, in order."""
                room = max_step_tokens
                seqs, sampled = [], []
                for i in active:
                    if fed[i] == len(prompts[i]):                      # decoding: its newest token
                        seqs.append(SequenceStep(slots[i], [last[i]], [0]))
                        sampled.append(i)
                        continue
                    n = len(prompts[i]) - fed[i]
                    if room is not None:
                        n = min(n, room)
                        room -= n
                    if n == 0:
                        continue                                       # no room in this step
                    ends = fed[i] + n == len(prompts[i])
                    seqs.append(SequenceStep(slots[i], prompts[i][fed[i]:fed[i] + n], [n - 1] if ends else []))
                    fed[i] += n
                    if ends:
                        sampled.append(i)
                return seqs, sampled

            def take(sampled, tokens):
                """Accepts one sampled token per request of `sampled`; drops the requests that end."""
                nonlocal active
                ended = set()
                for i, t in zip(sampled, tokens):
                    if accept(i, int(t)):
                        last[i] = int(t)
                    else:
                        ended.add(i)
                active = [i for i in active if i not in ended]
                return not ended

            while active:
                seqs, sampled = next_step()
                logits = backend.step(seqs)
                if not sampled:
                    continue                                           # portions only: nothing to sample yet
                act_slots = [slots[i] for i in sampled]
                all_decoding = all(fed[i] == len(prompts[i]) for i in active)
                if not (lookahead and all_decoding and sampled == active):
                    take(sampled, backend.sample(logits, act_slots, params))
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
                    rows = list(active)
                    all_on = take(rows, backend.read(pending))
                    if ahead is not None and all_on:
                        pending = ahead
                        continue
                    if ahead is not None:
                        tokens = backend.read(ahead)
                        alive = [(i, t) for i, t in zip(rows, tokens) if i in active]
                        take([i for i, _ in alive], [t for _, t in alive])
                    break
            if check is not None:
                check()                # device-side error flags, read once per batch; raises
        finally:
            for s in slots.values():
                backend.free(s)
    return results
