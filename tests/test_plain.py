"""The plain implementation itself: against the reference's own model code (golden logits
made by tests/golden/make_golden.py) and against independent restatements of each part."""
import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_llama as pl

GOLDEN = Path(__file__).parent / "golden"


@pytest.mark.parametrize("case", ["A", "B0"])
def test_against_reference_model_code(case, tmp_path):
    """Same weights (a function of config and seed), same tokens: the plain model's logits
    equal those of the reference's forward_prefill and of its token-by-token forward."""
    from oracle_engine_b200 import LlamaConfig, write_model_folder
    meta = json.loads((GOLDEN / f"{case}.json").read_text())
    golden = np.load(GOLDEN / f"{case}.npy")
    write_model_folder(tmp_path, LlamaConfig.from_dict(meta["config"]), seed=meta["seed"])
    got = pl.PlainLlama(tmp_path).logits(meta["tokens"]).numpy()
    assert np.abs(got).max() > 0.3
    for row, how in enumerate(meta["rows"]):
        err = np.abs(got - golden[row]).max()
        assert err < 2e-6, f"{case} vs reference {how}: {err}"


def test_rms_norm_by_loops():
    x = torch.randn(3, 10, dtype=torch.float64)
    w = torch.randn(10, dtype=torch.float64)
    y = pl.rms_norm(x, w, 1e-3)
    for r in range(3):
        ss = sum(float(v) ** 2 for v in x[r]) / 10
        for i in range(10):
            assert abs(float(y[r, i]) - float(x[r, i]) / math.sqrt(ss + 1e-3) * float(w[i])) < 1e-12


def test_rope_properties():
    inv = pl.rope_inv_freq(8, 10000.0, None)
    assert torch.allclose(inv, torch.tensor([1.0, 0.1, 0.01, 0.001], dtype=torch.float64))
    x = torch.randn(5, 2, 8, dtype=torch.float64)
    pos = torch.tensor([0, 1, 2, 50, 7])
    y = pl.rope_rotate(x, pos, inv)
    assert torch.allclose(y[0], x[0])                                     # position 0 is the identity
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))                  # rotations keep lengths
    # pair (i, i + half) rotates by pos * f_i
    p, i = 3, 1
    a = 50 * 0.1
    assert abs(float(y[p, 0, i]) - (float(x[p, 0, i]) * math.cos(a) - float(x[p, 0, i + 4]) * math.sin(a))) < 1e-12
    assert abs(float(y[p, 0, i + 4]) - (float(x[p, 0, i]) * math.sin(a) + float(x[p, 0, i + 4]) * math.cos(a))) < 1e-12
    # scores depend on the distance between positions only
    q, k = torch.randn(1, 1, 8, dtype=torch.float64), torch.randn(1, 1, 8, dtype=torch.float64)
    s1 = (pl.rope_rotate(q, torch.tensor([9]), inv) * pl.rope_rotate(k, torch.tensor([4]), inv)).sum()
    s2 = (pl.rope_rotate(q, torch.tensor([105]), inv) * pl.rope_rotate(k, torch.tensor([100]), inv)).sum()
    assert abs(float(s1 - s2)) < 1e-9


def test_llama3_scaling_regions():
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}
    base = pl.rope_inv_freq(32, 500000.0, None)
    got = pl.rope_inv_freq(32, 500000.0, sc)
    wl = 2 * math.pi / base
    seen = set()
    for i in range(16):
        if wl[i] < 64 / 4:
            assert got[i] == base[i]
            seen.add("high")
        elif wl[i] > 64 / 1:
            assert abs(float(got[i] - base[i] / 8)) < 1e-18
            seen.add("low")
        else:
            s = (64 / float(wl[i]) - 1.0) / 3.0
            assert abs(float(got[i]) - ((1 - s) * float(base[i]) / 8 + s * float(base[i]))) < 1e-15
            assert base[i] / 8 < got[i] < base[i]
            seen.add("mid")
    assert seen == {"high", "mid", "low"}
    assert torch.equal(pl.rope_inv_freq(32, 500000.0, {"rope_type": "default"}), base)


def test_llama3_scaling_pinned_by_literals_and_continuity():
    """The llama3 frequency scaling, which the reference does not have, pinned by things that are not
    the formula typed again: values worked out apart (40-digit decimal arithmetic) for the benchmark
    model's constants, continuity at both boundaries, and monotony.  The plain function and the
    product's (parts/positions.py) must both give them.

    By hand for i = 32: f = 500000^(-1/2) = 1/707.10678 = 1.41421356e-3, wavelength 2 pi / f = 4442.88,
    between 8192/4 and 8192/1, so s = (8192 / 4442.88 - 1) / 3 = 0.281283 and
    f' = f ((1 - s) / 32 + s) = 1.41421356e-3 x 0.3037428 = 4.295568e-4."""
    from oracle_engine_b200.parts.positions import rotary_inv_freq
    sc = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 8192}
    table = {0: 1.0, 28: 3.211445994753e-3, 29: 2.118406996780e-3, 32: 4.295567965594e-4,
             34: 9.708287802628e-5, 35: 2.389053088491e-5, 63: 7.672314972286e-8}
    for fn in (pl.rope_inv_freq, rotary_inv_freq):
        got = fn(128, 500000.0, sc)
        for i, want in table.items():
            assert abs(float(got[i]) / want - 1.0) < 1e-11, (fn.__module__, i, float(got[i]), want)
        assert all(float(got[i]) > float(got[i + 1]) for i in range(63))                # strictly falling
        # Continuity: a frequency whose wavelength is exactly orig / high keeps its value from both
        # sides, one at orig / low is divided by the factor from both sides.  theta and head_dim are
        # chosen so that f_1 = theta^(-1/2) has exactly that wavelength (up to rounding).
        for bound, ratio in ((8192.0 / 4.0, 1.0), (8192.0 / 1.0, 1.0 / 32.0)):
            f_edge = 2.0 * math.pi / bound
            for nudge in (1.0 - 1e-9, 1.0 + 1e-9):
                theta = (1.0 / (f_edge * nudge)) ** 2                                   # head_dim 4: f_1 = theta^(-2/4)
                got2 = fn(4, theta, sc)
                assert abs(float(got2[1]) / (f_edge * nudge * ratio) - 1.0) < 1e-7, (bound, nudge)


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    n, H, KVH, hd = 9, 6, 2, 4
    q, k, v = (torch.randn(n, h, hd, dtype=torch.float64) for h in (H, KVH, KVH))
    o = pl.causal_attention(q, k, v).reshape(n, H, hd)
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 0.3, -2.0
    o2 = pl.causal_attention(q, k2, v2).reshape(n, H, hd)
    assert torch.allclose(o[:5], o2[:5]) and not torch.allclose(o[5:], o2[5:])      # no look-ahead
    assert torch.allclose(o[0, 4], v[0, 1])                                          # head 4 reads KV head 1
    # by hand for one query
    t, h = 6, 3
    s = torch.tensor([float(q[t, h] @ k[j, 1]) / 2.0 for j in range(t + 1)], dtype=torch.float64)
    p = torch.exp(s - s.max())
    p /= p.sum()
    assert torch.allclose(o[t, h], (p[:, None] * v[: t + 1, 1]).sum(0))
    ow = pl.causal_attention(q, k, v, window=3).reshape(n, H, hd)
    s = s[-3:]
    p = torch.exp(s - s.max())
    p /= p.sum()
    assert torch.allclose(ow[t, h], (p[:, None] * v[t - 2: t + 1, 1]).sum(0))
    assert torch.allclose(ow[:3], o[:3])


def test_swiglu_and_softmax():
    x = torch.randn(4, 6, dtype=torch.float64)
    wg, wu, wd = (torch.randn(*s, dtype=torch.float64) for s in ((5, 6), (5, 6), (6, 5)))
    g, u = x @ wg.T, x @ wu.T
    want = (g * torch.sigmoid(g) * u) @ wd.T
    assert torch.allclose(pl.swiglu_ffn(x, wg, wu, wd), want)
    s = pl.softmax_rows(torch.tensor([[1000.0, 1001.0, 999.0]], dtype=torch.float64))
    assert abs(float(s.sum()) - 1) < 1e-12 and s[0, 1] > s[0, 0] > s[0, 2]


def test_sampling_chain():
    lg = torch.tensor([0.5, 2.0, 2.0, -1.0, 1.0])
    assert pl.greedy(lg) == 1                                                  # first maximum
    assert pl.sample(lg, 0.0, 40, 0.9, 0.99) == 1                              # T <= 0 is greedy
    # repeat penalty: positive logits divided, negative multiplied, in order, twice if recorded twice
    pen = pl.repeat_penalty(lg, [1, 3, 1, 9], 2.0, 64)
    assert pen.tolist() == [0.5, 0.5, 2.0, -2.0, 1.0]
    assert pl.repeat_penalty(lg, [1, 3, 0], 2.0, 2).tolist() == [0.25, 2.0, 2.0, -2.0, 1.0]
    assert pl.sample(lg, 0.0, 0, 1.0, 0.0, history=[1], penalty=2.0) == 2
    p = pl.softmax_rows(lg.double() / 0.5)
    # top-k 2 keeps tokens 1 and 2 (equal mass): u below one half gives 1, above gives 2
    assert pl.sample(lg, 0.5, 2, 1.0, 0.49) == 1 and pl.sample(lg, 0.5, 2, 1.0, 0.51) == 2
    # top-p cuts where the running sum (by probability, ties by index) reaches it
    assert pl.sample(lg, 0.5, 0, float(p[1]) - 1e-9, 0.999) == 1
    assert pl.sample(lg, 0.5, 0, float(p[1]) + 1e-9, 0.999) == 2
    # all kept: inverse CDF in index order
    c = torch.cumsum(p, 0)
    for u in (0.0, 0.3, 0.6, 0.9, 0.999999):
        want = int((c > u * float(c[-1])).nonzero()[0])
        assert pl.sample(lg, 0.5, 0, 1.0, u) == want
    us = [pl.uniform_from_counter(7, i) for i in range(2000)]
    assert all(0 <= u < 1 for u in us) and abs(sum(us) / 2000 - 0.5) < 0.03
    assert pl.uniform_from_counter(7, 3) != pl.uniform_from_counter(8, 3)


def test_generate_stops_without_emitting(plain_models):
    m = plain_models["A"]
    out = pl.generate(m, [3, 4, 5], 5)
    assert len(out) == 5
    assert pl.generate(m, [3, 4, 5], 5, stop_ids=(out[2],)) == out[:out.index(out[2])]


def fnv1a(tokens) -> int:
    """The checksum the reference's bench prints for its greedy tokens (benchmark/bench_engine.cpp:233-242)."""
    h = 1469598103934665603
    for t in tokens:
        h ^= int(t) & 0xFFFFFFFF
        h = (h * 1099511628211) & ((1 << 64) - 1)
    return h


def test_greedy_tokens_hash_to_the_checksum_of_the_references_own_bench(tmp_path):
    """tests/golden/bench_checksum_B0.json holds the checksum that the reference's unmodified benchmark
    program printed for 64 greedy tokens after its 128-token prompt, on this model (made by
    tests/golden/make_bench_checksum.py); the plain model's greedy generation gives the same tokens."""
    import json
    from oracle_engine_b200 import LlamaConfig, write_model_folder
    g = json.loads((GOLDEN / "bench_checksum_B0.json").read_text())
    write_model_folder(tmp_path / "m", LlamaConfig.from_dict(g["config"]), seed=g["seed"], std=g["std"])
    toks = pl.generate(pl.PlainLlama(tmp_path / "m"), g["prompt"], g["gen_tokens"])
    assert len(set(toks)) > 20
    assert f"{fnv1a(toks):016x}" == g["gen_checksum"]
