"""Schedules beyond "whole prompt, then one token each": prompts that arrive in pieces over a cached
prefix, steps that mix prompt pieces with single tokens, and the real head geometry at real context
lengths across the context-class boundaries.  All through Engine.step, all against the plain model."""
import numpy as np
import pytest
import torch

import helpers
from helpers import TOL

pytestmark = pytest.mark.gpu


def _compare(got, plain, requests, tol, what):
    for i, toks in enumerate(requests):
        want = plain.logits(toks).numpy()
        assert not np.isnan(got[i]).any(), f"{what}: request {i} has positions without logits"
        err = np.abs(got[i] - want).max(axis=1)
        assert err.max() < tol, f"{what}: request {i} (len {len(toks)}) first bad position " \
                                f"{int((err >= tol).argmax())}, worst {int(err.argmax())}: {err.max()}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "E"])
def test_pieces_and_mixed_steps_agree_with_plain(model_dirs, plain_models, tmp_path, name, dtype):
    from oracle_engine_b200.engine.engine import Engine
    plain = plain_models[name]
    limit, vocab = plain.cfg["max_position_embeddings"], plain.cfg["vocab_size"]
    lens = [min(n, limit) for n in (200, 130, 65, 300, 1, 37, 96, 69, 101)]
    requests = [helpers.random_tokens(n, vocab, 400 + i) for i, n in enumerate(lens)]
    eng = Engine.from_pretrained(model_dirs[name], dtype=dtype, max_tokens=1024)
    runs = {}
    whole = helpers.whole_steps(requests)
    runs["whole"] = (whole, helpers.TraceRunner(eng, tmp_path / "whole").run(whole))
    # (a) each request alone, in pieces of 37, 90, 1, 64, 2, 150 tokens: from the second piece on the
    # prompt kernels run over a cached prefix (90 tokens x the group is wide enough for the tcgen05 one)
    plans = [helpers.cut(n, [37, 90, 1, 64, 2, 150]) for n in lens]
    chunked = helpers.piece_steps(requests, plans, batch_size=1)
    runs["chunked"] = (chunked, helpers.TraceRunner(eng, tmp_path / "chunked").run(chunked))
    # (b) batches of three whose steps mix a prompt piece of one request with single tokens of
    # another while a third ends; the next batch starts in the slots they leave
    def mixed_plan(i, n):
        shapes = ([40, 1, 1, 1, 1, 50], [1, 1, 60, 1, 1, 1, 1], [100, 1])[i % 3]
        plan, left = [], n
        for s in shapes:
            if left <= 0:
                break
            plan.append(min(s, left))
            left -= plan[-1]
        return plan + [1] * left if left < 8 else plan + helpers.cut(left, [1, 33, 1, 1, 70])
    plans = [mixed_plan(i, n) for i, n in enumerate(lens)]
    mixed = helpers.piece_steps(requests, plans, batch_size=3)
    assert any(len({len(e["tokens"]) for e in s["entries"]}) > 1 and min(len(e["tokens"]) for e in s["entries"]) == 1
               for s in mixed)
    runs["mixed"] = (mixed, helpers.TraceRunner(eng, tmp_path / "mixed").run(mixed))
    eng.cache.check()
    assert eng.cache.slots.n_free == eng.cache.n_slots
    got = {k: helpers.collect(s, o, requests) for k, (s, o) in runs.items()}
    for k in got:
        _compare(got[k], plain, requests, TOL[dtype], f"{name} {dtype} {k}")
    if dtype == "float32":
        for k in ("chunked", "mixed"):
            for i in range(len(requests)):
                assert np.array_equal(got["whole"][i], got[k][i]), f"{name} float32: {k} differs from whole, request {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generate_with_a_token_budget(model_dirs, plain_models, dtype):
    """Engine.generate with prompts cut into portions (mixed steps included) gives the tokens of the
    plain model's whole-sequence generation, as it does without a budget."""
    import plain_llama as pl
    from oracle_engine_b200 import GenParams
    from oracle_engine_b200.engine.engine import Engine
    plain = plain_models["B"]
    vocab = plain.cfg["vocab_size"]
    prompts = [helpers.random_tokens(n, vocab, 500 + i) for i, n in enumerate((70, 3, 41, 1, 100))]
    eng = Engine.from_pretrained(model_dirs["B"], dtype=dtype, max_tokens=1024)
    want = [pl.generate(plain, p, 6) for p in prompts]
    params = GenParams.greedy(6, ignore_eos=True)
    same = lambda a, b: sum(x == y for x, y in zip(sum(a, []), sum(b, [])))             # noqa: E731
    whole = eng.generate(prompts, params)
    for budget in (16, 64, 1):
        for ahead in (True, False):
            got = eng.generate(prompts, params, max_step_tokens=budget, lookahead=ahead, batch_size=3)
            # 32-bit: the same bits under every cut; bfloat16 may flip a near tie when the cut changes a kernel
            assert got == whole if dtype == "float32" else same(got, whole) >= 28, (budget, ahead)
    assert whole == want if dtype == "float32" else same(whole, want) >= 28
    eng.cache.check()


# ------------------------------------------------------------------------------------------
# the benchmark's head geometry (24 query heads over 8 KV heads of 128) at real context lengths
# ------------------------------------------------------------------------------------------
REAL_HEADS = dict(architectures=["LlamaForCausalLM"], vocab_size=512, hidden_size=256, intermediate_size=512,
                  num_hidden_layers=2, num_attention_heads=24, num_key_value_heads=8, head_dim=128,
                  rms_norm_eps=1e-5, rope_theta=500000.0,
                  rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                                "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
                  max_position_embeddings=8192, tie_word_embeddings=False, eos_token_id=1)


@pytest.fixture(scope="module")
def real_heads(tmp_path_factory):
    import plain_llama
    from oracle_engine_b200 import LlamaConfig, write_model_folder
    base = tmp_path_factory.mktemp("real_heads")
    write_model_folder(base / "m", LlamaConfig.from_dict(REAL_HEADS), seed=21, std=0.05)
    folder = helpers.sharpen(base / "m", base / "sharp", 2.0)        # peaked softmax: single far keys decide
    return folder, plain_llama.PlainLlama(folder, device="cuda")


def _tolerance(want) -> float:
    """bfloat16 against the plain model at this model's logit scale (a few units, where the tiny
    configurations have about one): the bound the real-width tests use, 3 % of the scale plus 0.02."""
    return 0.03 * float(np.abs(want).max()) + 0.02


class _Seen:
    """Hears of every kernel launch (csrc/ops.py: OBSERVER)."""

    def __init__(self):
        self.log = []

    def mark(self, what, detail):
        self.log.append((what, detail))

    def attention(self):
        return [(w, (d or {}).get("splits") or (d or {}).get("cluster")) for w, d in self.log if w.startswith("attention")]


def test_one_sequence_across_both_context_class_boundaries(real_heads, tmp_path):
    """4,300 tokens: a prompt, decoding across 1,536 tokens, a prompt piece of 2,450 tokens over the
    cached prefix, decoding across 4,096 tokens; with the class boundaries where serving has them.
    Every decoded position and the rows of the prompt pieces are compared with the plain model, and
    each class must have used the decode kernel and the number of CTAs per pair its rule names."""
    from oracle_engine_b200.csrc import ops, ops_tc
    from oracle_engine_b200.engine import batch
    from oracle_engine_b200.engine.engine import Engine
    assert batch.CONTEXT_CLASS_TOKENS == [768, 1536, 4096]
    folder, plain = real_heads
    toks = helpers.random_tokens(4300, 512, 77)
    plan = [1500] + [1] * 100 + [2450] + [1] * 250
    steps = helpers.piece_steps([toks], [plan])
    eng = Engine.from_pretrained(folder, dtype="bfloat16", max_tokens=4352, use_graphs=False)
    seen = _Seen()
    ops.OBSERVER[0] = seen
    try:
        out = helpers.TraceRunner(eng, tmp_path / "one").run(steps)
    finally:
        ops.OBSERVER[0] = None
    got = helpers.collect(steps, out, [toks])[0]
    want = plain.logits(toks).cpu().numpy()
    err = np.abs(got - want).max(axis=1)
    tol = _tolerance(want)
    assert err.max() < tol, f"first bad position {int((err >= tol).argmax())}: {err.max()} (tolerance {tol})"
    eng.check_device_errors()
    # which decode kernel ran in each class (the decoding here runs in classes 1 to 3): the one whose warps
    # split the keys, and, 8 (sequence, KV head) pairs being few, with clusters of 4 CTAs and, past 4,096 tokens, of 8
    kinds = set(seen.attention())
    clusters = sorted(c for w, c in kinds if w == "attention_decode_warps")
    assert clusters == sorted({ops_tc.decode_warps_cluster(1, c, 8) for c in (1, 2, 3)}) == [4, 8]
    assert not any(w == "attention_mma" for w, _ in kinds)
    assert ("attention_tcgen05", None) in kinds            # the prompt pieces


def test_sixty_four_sequences_across_the_first_boundary(real_heads, tmp_path):
    """64 sequences of 1,460 to 1,523 tokens decode 90 tokens each, across 1,536: 512 (sequence, KV
    head) pairs go to one-warp CTAs with rings of three tiles up to 1,536 tokens (four CTAs an SM) and to
    two-warp CTAs beyond.  CUDA
    graphs on, as in serving; every decoded position against the plain model."""
    from oracle_engine_b200.csrc import ops_tc
    from oracle_engine_b200.engine.engine import Engine
    folder, plain = real_heads
    n = 64
    assert ops_tc.decode_warps_shape(n, 1, 128, 8) == (1, 3) and ops_tc.decode_warps_shape(n, 2, 128, 8) == (2, 3)
    lens = [1460 + i + 90 for i in range(n)]
    requests = [helpers.random_tokens(m, 512, 900 + i) for i, m in enumerate(lens)]
    steps = helpers.batched_steps(requests, [1460 + i for i in range(n)], n)
    # only the decoded positions are wanted: the prompt step would return 97,000 rows otherwise
    steps[0]["entries"] = [dict(e, want=[len(e["tokens"]) - 1]) for e in steps[0]["entries"]]
    eng = Engine.from_pretrained(folder, dtype="bfloat16", max_tokens=n * 1664)
    out = helpers.TraceRunner(eng, tmp_path / "b64").run(steps)
    classes = {key[1] for key, g in eng.stepper._graphs.items() if g.graph is not None}
    assert classes == {1, 2}
    eng.check_device_errors()
    worst = 0.0
    for i, toks in enumerate(requests):
        want = plain.logits(toks).cpu().numpy()
        tol = _tolerance(want)
        pos = 1460 + i - 1                      # the prompt's last position, then one per step
        for s in steps:
            ids = [e["id"] for e in s["entries"]]
            if f"r{i}" not in ids:
                continue
            r = ids.index(f"r{i}")
            err = np.abs(out[s["step"]][r] - want[pos]).max()
            worst = max(worst, err)
            assert err < tol, f"request {i} position {pos}: {err}"
            pos += 1
        assert pos == len(toks)
    eng.cache.check()


@pytest.mark.parametrize("hidden,heads,kv_heads,head_dim,ffn,factor", [(3072, 24, 8, 128, 8192, 32.0),      # Llama 3.2 3B
                                                                       (2048, 32, 8, 64, 8192, 32.0),       # 3.2 1B
                                                                       (4096, 32, 8, 128, 14336, 8.0)])     # 3.1 8B
def test_real_widths_against_plain(tmp_path, hidden, heads, kv_heads, head_dim, ffn, factor):
    """Two layers with the widths of the benchmark models and a small vocabulary, against the plain
    model: a prompt step of 64 unequal prompts (the tensor-core products at thousands of rows), decode
    steps of 64 sequences (swap-AB products whose K splits add up in a cluster, narrow gate/up tiles),
    of 24 (tcgen05 products and the weight-streaming kernel side by side) and of 8."""
    import plain_llama
    from oracle_engine_b200 import LlamaConfig, write_model_folder
    from oracle_engine_b200.engine.engine import Engine
    raw = dict(architectures=["LlamaForCausalLM"], vocab_size=2048, hidden_size=hidden, intermediate_size=ffn,
               num_hidden_layers=2, num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
               rms_norm_eps=1e-5, rope_theta=500000.0,
               rope_scaling={"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0,
                             "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
               max_position_embeddings=4096, tie_word_embeddings=False, eos_token_id=1)
    folder = tmp_path / "wide"
    write_model_folder(folder, LlamaConfig.from_dict(raw), seed=3, device="cuda")
    plain = plain_llama.PlainLlama(folder, device="cuda")
    n = 64
    # 64 sequences decode 3 tokens, then 24 of them 2 more, then 12 of them 2 more, then 8 of them 2 more
    decoded = [9 if i < 8 else 7 if i < 12 else 5 if i < 24 else 3 for i in range(n)]
    prompt_lens = [20 + (i * 7) % 64 for i in range(n)]
    requests = [helpers.random_tokens(p + d, 2048, 600 + i) for i, (p, d) in enumerate(zip(prompt_lens, decoded))]
    steps = helpers.batched_steps(requests, prompt_lens, n)
    assert [len(s["entries"]) for s in steps] == [64, 64, 64, 64, 24, 24, 12, 12, 8, 8]
    eng = Engine.from_pretrained(str(folder), dtype="bfloat16", max_tokens=n * 128)
    out = helpers.TraceRunner(eng, tmp_path / "wide_out").run(steps)
    eng.check_device_errors()
    got = helpers.collect(steps, out, requests)
    worst, scale = 0.0, 0.0
    for i, toks in enumerate(requests):
        want = plain.logits(toks).cpu().numpy()
        scale = max(scale, float(np.abs(want).max()))
        worst = max(worst, float(np.abs(got[i] - want).max()))
    assert scale > 0.5 and worst < 0.03 * scale + 0.02, f"max abs err {worst} at logit scale {scale}"
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_steps_run_as_captured_graphs(model_dirs, plain_models, tmp_path, dtype):
    """Steps of up to 256 tokens that are no decode steps (short prompts, pieces, prompts mixed with
    single tokens) run as CUDA graphs of their padded shape: four rounds of the same shapes with other
    tokens, so that each shape is run directly, captured and replayed; wanted rows as in generation (the
    last of a prompt) and all rows.  Every wanted row against the plain model, and the engine without
    graphs gives the same float32 bits."""
    from oracle_engine_b200.engine.engine import Engine
    plain = plain_models["B"]
    vocab = plain.cfg["vocab_size"]
    shapes = [[23, 1, 1, 40, 1], [60, 1, 1], [1, 9, 1, 1, 30], [100, 1, 1, 1]]      # pieces of the requests of a round
    # (the first step of a round has 184 tokens: the 256-token shape; the others the smaller ones)
    requests, plans = [], []
    for r in range(4):
        for j, shape in enumerate(shapes):
            requests.append(helpers.random_tokens(sum(shape), vocab, 1000 + 10 * r + j))
            plans.append(shape)
    steps = helpers.piece_steps(requests, plans, batch_size=len(shapes))
    per_round = max(len(shape) for shape in shapes)
    assert len(steps) == 4 * per_round
    for k, s in enumerate(steps):                          # every other step of a round wants only each entry's last row
        if (k % per_round) % 2 == 0:
            s["entries"] = [dict(e, want=[len(e["tokens"]) - 1]) for e in s["entries"]]
    outs = {}
    for graphs in (True, False):
        eng = Engine.from_pretrained(model_dirs["B"], dtype=dtype, max_tokens=1024, use_graphs=graphs)
        outs[graphs] = helpers.TraceRunner(eng, tmp_path / f"g{int(graphs)}").run(steps)
        if graphs:
            used = [g for g in eng.stepper._token_graphs.values() if g.graph is not None]
            assert used and max(g.runs for g in used) >= 3, "no short step was captured and replayed"
        eng.cache.check()
    logits = [plain.logits(toks).numpy() for toks in requests]
    pos = [0] * len(requests)
    for s in steps:
        row = 0
        for e in s["entries"]:
            i = int(e["id"][1:])
            for w in e["want"]:
                got, want = outs[True][s["step"]][row], logits[i][pos[i] + w]
                assert np.abs(got - want).max() < TOL[dtype], f"step {s['step']} request {i} position {pos[i] + w}"
                if dtype == "float32":
                    assert np.array_equal(got, outs[False][s["step"]][row])
                row += 1
            pos[i] += len(e["tokens"])
