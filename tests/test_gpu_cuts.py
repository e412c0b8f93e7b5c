"""The same requests under every way of cutting the work: whole, with the last 32 tokens one
by one, and in batches of unequal lengths with slots used again; all against the plain model."""
import numpy as np
import pytest

import helpers
from helpers import TOL

pytestmark = pytest.mark.gpu

LENGTHS = [1, 9, 40, 100, 65, 64, 130, 33]


def _requests(cfg, seed0=10):
    limit = cfg["max_position_embeddings"]
    return [helpers.random_tokens(min(n, limit), cfg["vocab_size"], seed0 + i) for i, n in enumerate(LENGTHS)]


@pytest.fixture(scope="module")
def sharp_dirs(model_dirs, tmp_path_factory):
    return {k: helpers.sharpen(model_dirs[k], tmp_path_factory.mktemp(f"sharp_{k}"), 6.0) for k in ("A", "B", "E")}


def _check(got, plain, requests, tol, what):
    for i, toks in enumerate(requests):
        want = plain.logits(toks).numpy()
        assert not np.isnan(got[i]).any(), f"{what}: request {i} has positions without logits"
        err = np.abs(got[i] - want)
        worst = int(err.max(axis=1).argmax())
        assert err.max() < tol, f"{what}: request {i} (len {len(toks)}) first bad position " \
                                f"{int((err.max(axis=1) >= tol).argmax())}, worst {worst}: {err.max()}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_cuts_agree_with_plain(model_dirs, plain_models, tmp_path, name, dtype):
    from oracle_engine_b200.engine.engine import Engine
    plain = plain_models[name]
    requests = _requests(plain.cfg)
    # room for one batch of three at a time only: slots and pages must be used again
    eng = Engine.from_pretrained(model_dirs[name], dtype=dtype, max_tokens=448)
    runs = {}
    whole = helpers.whole_steps(requests)
    runs["whole"] = (whole, helpers.TraceRunner(eng, tmp_path / "whole").run(whole))
    tail = helpers.tail_steps(requests, 32)
    runs["tail"] = (tail, helpers.TraceRunner(eng, tmp_path / "tail").run(tail))
    prompt_lens = [1, 4, 17, 60, 64, 33, 100, 33]
    bat = helpers.batched_steps(requests, prompt_lens, 3)
    runs["batched"] = (bat, helpers.TraceRunner(eng, tmp_path / "bat").run(bat))
    eng.cache.check()
    assert eng.cache.slots.n_free == eng.cache.n_slots
    got = {k: helpers.collect(s, o, requests) for k, (s, o) in runs.items()}
    for k in got:
        _check(got[k], plain, requests, TOL[dtype], f"{name} {dtype} {k}")
    if dtype == "float32":
        # the 32-bit path computes every row in a fixed order: cuts give identical bits
        for k in ("tail", "batched"):
            for i in range(len(requests)):
                assert np.array_equal(got["whole"][i], got[k][i]), f"{name} float32: {k} differs from whole, request {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sharp_attention_far_keys(sharp_dirs, tmp_path, dtype):
    """Peaked softmax over several pages: a far key, a page edge or a stale slot shows."""
    import plain_llama
    from oracle_engine_b200.engine.engine import Engine
    for name in ("A", "B", "E"):
        plain = plain_llama.PlainLlama(sharp_dirs[name])
        limit = plain.cfg["max_position_embeddings"]
        lens = [min(limit, n) for n in (127, 128, 129, 300, 63, 65)]
        requests = [helpers.random_tokens(n, plain.cfg["vocab_size"], 50 + i) for i, n in enumerate(lens)]
        eng = Engine.from_pretrained(sharp_dirs[name], dtype=dtype, max_tokens=640)
        prompt_lens = [max(1, n - 40) for n in lens]
        bat = helpers.batched_steps(requests, prompt_lens, 2)
        out = helpers.TraceRunner(eng, tmp_path / f"sharp_{name}").run(bat)
        got = helpers.collect(bat, out, requests)
        # sharper softmax amplifies bf16 rounding of the scores; logits stay O(1)
        _check(got, plain, requests, TOL[dtype] * (1 if dtype == "float32" else 3), f"sharp {name} {dtype}")
        eng.cache.check()


def test_trace_run_cli(model_dirs, plain_models, tmp_path):
    """bin/trace_run as a program: protocol, files, exit code."""
    plain = plain_models["B"]
    requests = _requests(plain.cfg)[:5]
    steps = helpers.batched_steps(requests, [1, 4, 17, 60, 64], 2)
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        helpers.run_trace_cli(model_dirs["B"], dtype, steps, out, 256)
        vocab = plain.cfg["vocab_size"]
        outputs = {s["step"]: np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab) for s in steps}
        got = helpers.collect(steps, outputs, requests)
        _check(got, plain, requests, TOL[dtype], f"cli {dtype}")
