"""Each request alone and whole: engine logits at every position against the plain implementation."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

# bf16 keeps 8 bits of mantissa: activations are rounded to a relative 2^-9 at every layer
# boundary; logits here are O(1), so 0.05 absolute leaves room for a few layers of rounding
# while a wrong position, head or key shows up as O(1).
TOL = {"float32": 2e-4, "bfloat16": 5e-2}


def _tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "E"])
def test_whole_prompt_logits(model_dirs, plain_models, name, dtype):
    from oracle_engine_b200 import SequenceStep
    from oracle_engine_b200.engine.engine import Engine
    eng = Engine.from_pretrained(model_dirs[name], dtype=dtype, max_tokens=1024)
    plain = plain_models[name]
    vocab = plain.cfg["vocab_size"]
    for n, seed in ((1, 1), (7, 2), (70, 3), (100, 4)):
        toks = _tokens(n, vocab, seed)
        slot = eng.alloc()
        got = eng.step([SequenceStep(slot, toks, list(range(n)))]).float().cpu().numpy()
        eng.free(slot)
        want = plain.logits(toks).numpy()
        err = np.abs(got - want).max()
        assert err < TOL[dtype], f"{name} {dtype} n={n}: max abs err {err}"
    eng.cache.check()
