"""What the C API calls: plain functions over `Engine`, with C arrays given as addresses.

The C side (oe_capi.cpp) only passes integers and strings and turns exceptions into
`oe_last_error()`; every array is read or written here, through numpy views of the caller's
memory.  No model code: each function is a few lines over the public `Engine`.
"""
from __future__ import annotations

import ctypes

import numpy as np

_ON_TOKEN = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_int, ctypes.c_void_p)


def _ints(addr: int, n: int) -> np.ndarray:
    """The caller's n 32-bit integers at `addr` (a view, not a copy)."""
    if n == 0:
        return np.zeros(0, dtype=np.int32)
    if not addr:
        raise ValueError("a null pointer where an array is needed")
    return np.ctypeslib.as_array((ctypes.c_int32 * n).from_address(addr))


def load(model_dir: str, dtype: str, max_tokens: int):
    from ..engine.engine import Engine
    if dtype not in ("bfloat16", "float32"):
        raise ValueError(f"dtype must be bfloat16 or float32, not {dtype!r}")
    if max_tokens < 1:
        raise ValueError("max_tokens must be at least 1")
    return Engine.from_pretrained(model_dir, dtype=dtype, max_tokens=int(max_tokens))


def vocab_size(engine) -> int:
    return int(engine.spec.vocab_size)


def max_seq_len(engine) -> int:
    return int(engine.max_seq_len)


def alloc_slot(engine) -> int:
    return int(engine.alloc())


def free_slot(engine, slot: int) -> int:
    engine.free(int(slot))
    return 0


def step(engine, n_seqs: int, slots: int, tokens: int, q_lens: int, want: int, n_want: int, out: int) -> int:
    from ..engine.batch import SequenceStep
    if n_seqs < 1:
        raise ValueError("a step needs at least one sequence")
    lens = _ints(q_lens, n_seqs)
    wants = _ints(n_want, n_seqs)
    if (lens < 0).any() or (wants < 0).any():
        raise ValueError("negative count in q_lens or n_want")
    toks = _ints(tokens, int(lens.sum()))
    places = _ints(want, int(wants.sum()))
    seqs, t, w = [], 0, 0
    for i, slot in enumerate(_ints(slots, n_seqs)):
        seqs.append(SequenceStep(int(slot), toks[t:t + lens[i]].tolist(), places[w:w + wants[i]].tolist()))
        t += int(lens[i])
        w += int(wants[i])
    if w and not out:
        raise ValueError("logits_out is null but logits are wanted")
    logits = engine.step(seqs)
    if logits is None:
        return 0
    rows, vocab = logits.shape
    host = logits.float().cpu().contiguous().numpy()
    ctypes.memmove(out, host.ctypes.data, host.nbytes)
    return int(rows)


def generate(engine, n_prompts: int, tokens: int, lens: int, n_predict: int, temperature: float, top_p: float,
             top_k: int, repeat_penalty: float, repeat_last_n: int, seed: int, ignore_eos: int, batch_size: int,
             max_step_tokens: int, out_tokens: int, out_lens: int, on_token: int, user: int) -> int:
    from ..sampling.params import GenParams
    if n_prompts < 1:
        raise ValueError("generation needs at least one prompt")
    plens = _ints(lens, n_prompts)
    if (plens < 1).any():
        raise ValueError("every prompt needs at least one token")
    toks = _ints(tokens, int(plens.sum()))
    prompts, t = [], 0
    for n in plens:
        prompts.append(toks[t:t + n].tolist())
        t += int(n)
    params = GenParams(n_predict=n_predict, temperature=temperature, top_p=top_p, top_k=top_k,
                       repeat_penalty=repeat_penalty, repeat_last_n=repeat_last_n, seed=seed,
                       ignore_eos=bool(ignore_eos))
    callback = None
    if on_token:
        fn = _ON_TOKEN(on_token)
        callback = lambda i, tok: fn(int(i), int(tok), user or None)      # noqa: E731
    got = _ints(out_tokens, n_prompts * n_predict)          # refused before anything runs if a pointer is null
    counts = _ints(out_lens, n_prompts)
    outs = engine.generate(prompts, params, batch_size=batch_size or None, on_token=callback,
                           max_step_tokens=max_step_tokens or None)
    for i, new in enumerate(outs):
        counts[i] = len(new)
        got[i * n_predict:i * n_predict + len(new)] = new
    return 0
