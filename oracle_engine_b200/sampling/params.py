"""Generation and sampling options, with the reference's names, defaults and meanings.

`GenParams` (core/engine.hpp:25-32): n_predict 256, temperature 0.7, top_p 0.9,
repeat_penalty 1.15, repeat_last_n 64.  `top_k` is not an option of the reference's
command line; `Engine::generate` fixes it at 40 (core/engine.cpp:106), which is the
default here.  temperature <= 0 means greedy (first maximum); temperature == 1 leaves the
logits unscaled (core/sampler.cpp:35-39, 50).  `seed`, `stop_ids` and `ignore_eos` are
this library's own: the reference seeds from the clock (core/engine.cpp:109-111) and
stops on one token it finds by name (core/engine.cpp:128-131).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class GenParams:
    n_predict: int = 256
    temperature: float = 0.7
    top_p: float = 0.9
    top_k: int = 40
    repeat_penalty: float = 1.15
    repeat_last_n: int = 64
    seed: int = 0                          # sequence i draws from seed + i
    stop_ids: Optional[tuple] = None       # None: the model's eos ids
    ignore_eos: bool = False

    @staticmethod
    def greedy(n_predict: int = 256, **kw) -> "GenParams":
        return GenParams(n_predict=n_predict, temperature=0.0, top_p=1.0, top_k=0, repeat_penalty=1.0, **kw)

    def validate(self) -> None:
        if self.n_predict < 0:
            raise ValueError("n_predict must be >= 0")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0 (0 = all tokens)")
        if self.repeat_penalty <= 0:
            raise ValueError("repeat_penalty must be > 0")
        if self.repeat_last_n < 0:
            raise ValueError("repeat_last_n must be >= 0")
