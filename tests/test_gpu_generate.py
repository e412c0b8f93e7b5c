"""Generation through the Python entry point: greedy and temperature against the plain
implementation, stop tokens, batches one after another with slots used again, long
decoding, and the first tokens of a sequence."""
import numpy as np
import pytest
import torch

import helpers
import plain_llama as pl
from helpers import TOL

pytestmark = pytest.mark.gpu


def _engine(model_dirs, name, dtype, **kw):
    from oracle_engine_b200.engine.engine import Engine
    return Engine.from_pretrained(model_dirs[name], dtype=dtype, **kw)


def _check_greedy(plain, prompt, got, margin):
    """Every generated token is the plain model's argmax, or within `margin` of it."""
    seq = list(prompt)
    for tok in got:
        lg = plain.logits(seq)[-1]
        assert lg.max().item() - lg[tok].item() <= margin, f"token {tok} at position {len(seq)}"
        seq.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_workload_a(model_dirs, plain_models, dtype):
    """Tiny A: prompts of 5, 11 and 17 tokens, 8 greedy steps each."""
    from oracle_engine_b200 import GenParams
    eng = _engine(model_dirs, "A", dtype, max_tokens=256)
    plain = plain_models["A"]
    prompts = [helpers.random_tokens(n, 256, 20 + i) for i, n in enumerate((5, 11, 17))]
    got = eng.generate(prompts, GenParams.greedy(8, ignore_eos=True))
    assert [len(g) for g in got] == [8, 8, 8]
    if dtype == "float32":
        assert got == [pl.generate(plain, p, 8) for p in prompts]
    for p, g in zip(prompts, got):
        _check_greedy(plain, p, g, 0.0 if dtype == "float32" else 2 * TOL[dtype])
    eng.cache.check()
    assert eng.cache.slots.n_free == eng.cache.n_slots


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_workload_b(model_dirs, plain_models, dtype):
    """Tiny B: prompts of 1, 9, 40 and 100 tokens, 12 steps at temperature 0.8, each
    sequence drawing from its own generator."""
    from oracle_engine_b200 import GenParams
    eng = _engine(model_dirs, "B", dtype, max_tokens=512)
    plain = plain_models["B"]
    prompts = [helpers.random_tokens(n, 384, 30 + i) for i, n in enumerate((1, 9, 40, 100))]
    params = GenParams(n_predict=12, temperature=0.8, top_k=0, top_p=1.0, repeat_penalty=1.0, seed=77, ignore_eos=True)
    got = eng.generate(prompts, params)
    for i, (p, g) in enumerate(zip(prompts, got)):
        seq = list(p)
        for step, tok in enumerate(g):
            lg = plain.logits(seq)[-1]
            u = pl.uniform_from_counter(77 + i, step)
            want = pl.sample(lg, 0.8, 0, 1.0, u)
            if tok != want:
                # allowed only when u falls within rounding of the boundary between the two tokens
                prob = pl.softmax_rows(lg / 0.8)
                c = torch.cumsum(prob, 0)
                edge = min(abs(float(c[min(tok, want)]) - u), abs(float(c[max(tok, want)]) - u))
                assert edge < (1e-5 if dtype == "float32" else 2e-2), f"request {i} step {step}: {tok} vs {want}"
            seq.append(tok)
    eng.cache.check()


def test_temperature_seed_is_per_request(model_dirs):
    from oracle_engine_b200 import GenParams
    eng = _engine(model_dirs, "B", "float32", max_tokens=256)
    p = helpers.random_tokens(9, 384, 31)
    params = GenParams(n_predict=10, temperature=1.0, top_k=0, top_p=1.0, repeat_penalty=1.0, seed=5, ignore_eos=True)
    a = eng.generate([p, p, p], params)
    assert a[0] != a[1] or a[1] != a[2]                    # same prompt, seeds 5, 6, 7
    b = eng.generate([p], params)                          # alone: the same draws as request 0 in the batch
    assert b[0] == a[0]
    c = eng.generate([p, p], GenParams(n_predict=10, temperature=1.0, top_k=0, top_p=1.0, repeat_penalty=1.0,
                                       seed=6, ignore_eos=True), batch_size=1)
    assert c[0] == a[1] and c[1] == a[2]                   # batches one after another reuse slot 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_chain_repeat_penalty_topk_topp(model_dirs, plain_models, dtype):
    from oracle_engine_b200 import GenParams
    eng = _engine(model_dirs, "C", dtype, max_tokens=256)
    plain = plain_models["C"]
    prompts = [helpers.random_tokens(n, 331, 40 + i) for i, n in enumerate((3, 20))]
    params = GenParams(n_predict=10, temperature=0.9, top_k=12, top_p=0.8, repeat_penalty=1.3, repeat_last_n=8, seed=3,
                       ignore_eos=True)
    got = eng.generate(prompts, params)
    for i, (p, g) in enumerate(zip(prompts, got)):
        seq = list(p)
        for step, tok in enumerate(g):
            lg = plain.logits(seq)[-1]
            hist = list(p[:-1]) + g[:step]
            want = pl.sample(lg, 0.9, 12, 0.8, pl.uniform_from_counter(3 + i, step), hist, 1.3, 8)
            if dtype == "float32":
                assert tok == want, f"request {i} step {step}"
            else:
                kept = pl.repeat_penalty(lg.double(), hist, 1.3, 8)
                assert kept[tok] >= kept.topk(14).values[-1] - 0.1        # inside (about) the top-k set
            seq.append(tok)


def test_stop_tokens_batches_and_slot_reuse(model_dirs, plain_models):
    """Seven requests in batches of three with a cache for one batch only: sequences that
    hit a stop id end earlier (the stop id is not emitted), slots and pages are used again."""
    from oracle_engine_b200 import GenParams
    eng = _engine(model_dirs, "A", "float32", max_tokens=320, n_slots=3)
    plain = plain_models["A"]
    prompts = [helpers.random_tokens(n, 256, 60 + i) for i, n in enumerate((5, 1, 30, 64, 9, 65, 2))]
    free_run = [pl.generate(plain, p, 20) for p in prompts]
    stop = {free_run[0][3], free_run[4][0], free_run[5][10]}
    want = [pl.generate(plain, p, 20, stop_ids=stop) for p in prompts]
    res = eng.generate(prompts, GenParams.greedy(20, stop_ids=tuple(stop)), batch_size=3, return_results=True)
    assert [r.tokens for r in res] == want
    assert [r.finish_reason for r in res] == ["stop" if len(w) < 20 else "length" for w in want]
    assert any(len(w) < 20 for w in want) and any(len(w) == 20 for w in want)
    eng.cache.check()
    assert eng.cache.slots.n_free == 3
    # without the step ahead of the host: the same tokens, and in both ways with sampling
    # (a step that ran with a sequence that had just stopped changes nothing for the others)
    res = eng.generate(prompts, GenParams.greedy(20, stop_ids=tuple(stop)), batch_size=3, return_results=True,
                       lookahead=False)
    assert [r.tokens for r in res] == want
    sampled = GenParams(n_predict=20, temperature=0.9, top_k=12, top_p=0.8, repeat_penalty=1.3, repeat_last_n=8,
                        seed=5, stop_ids=tuple(stop))
    heard = []
    one = eng.generate(prompts, sampled, batch_size=3, on_token=lambda i, t: heard.append((i, t)))
    two = eng.generate(prompts, sampled, batch_size=3, lookahead=False)
    assert one == two and any(len(o) < 20 for o in one)
    assert sorted(heard) == sorted((i, t) for i, o in enumerate(one) for t in o)
    eng.cache.check()
    assert eng.cache.slots.n_free == 3
    # the model's own eos ids stop a sequence unless told otherwise
    eos = plain.cfg["eos_token_id"]
    forced = [t for t in range(256) if t != eos][:3]
    assert eng.spec.stop_ids == (eos,)
    out = eng.generate([forced], GenParams.greedy(30))
    assert eos not in out[0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_the_first_token(model_dirs, plain_models, tmp_path, dtype):
    """A one-token prompt, then 300 tokens one by one (five pages, graph replay), two
    sequences of different phase in one batch."""
    from oracle_engine_b200.engine.engine import Engine
    plain = plain_models["B"]
    eng = Engine.from_pretrained(model_dirs["B"], dtype=dtype, max_tokens=704)
    requests = [helpers.random_tokens(n, 384, 80 + i) for i, n in enumerate((301, 260))]
    steps = helpers.batched_steps(requests, [1, 3], 2)
    out = helpers.TraceRunner(eng, tmp_path / "long").run(steps)
    got = helpers.collect(steps, out, requests)
    for i, toks in enumerate(requests):
        want = plain.logits(toks).numpy()
        err = np.abs(got[i] - want).max(axis=1)
        assert err.max() < TOL[dtype], f"request {i}: first bad position {int((err >= TOL[dtype]).argmax())}"
    assert eng.stepper.use_graphs and eng.stepper._graphs[(2, 0)].graph is not None
    eng.cache.check()


def test_decoding_across_the_context_classes(model_dirs, plain_models, tmp_path, monkeypatch):
    """Decode graphs are kept per context class (kernels may be chosen by it): sequences that grow
    across the boundaries while they decode, with the boundaries moved down to 96 and 170 tokens so
    that the tiny model crosses them."""
    from oracle_engine_b200.engine import batch, step
    from oracle_engine_b200.engine.engine import Engine
    monkeypatch.setattr(batch, "CONTEXT_CLASS_TOKENS", [96, 170])
    plain = plain_models["E"]
    eng = Engine.from_pretrained(model_dirs["E"], dtype="bfloat16", max_tokens=704)
    requests = [helpers.random_tokens(n, plain.cfg["vocab_size"], 90 + i) for i, n in enumerate((200, 140))]
    steps = helpers.batched_steps(requests, [70, 90], 2)
    out = helpers.TraceRunner(eng, tmp_path / "classes").run(steps)
    got = helpers.collect(steps, out, requests)
    for i, toks in enumerate(requests):
        want = plain.logits(toks).numpy()
        err = np.abs(got[i] - want).max(axis=1)
        assert err.max() < TOL["bfloat16"], f"request {i}: first bad position {int((err >= TOL['bfloat16']).argmax())}"
    graphs = eng.stepper._graphs
    for key in ((2, 0), (2, 1), (1, 1), (1, 2)):
        assert graphs[key].graph is not None, key
    eng.cache.check()


def test_many_sequences_decoding_across_the_context_classes(model_dirs, plain_models, tmp_path, monkeypatch):
    """50 sequences (100 (sequence, KV head) pairs) that grow across both class boundaries while
    they decode: in every class such a batch goes to the kernel whose warps split the keys, one CTA
    per pair; the logits are those of the plain model at every position, and shorter sequences leave
    the batch on the way."""
    from oracle_engine_b200.csrc import ops_tc
    from oracle_engine_b200.engine import batch
    from oracle_engine_b200.engine.engine import Engine
    monkeypatch.setattr(batch, "CONTEXT_CLASS_TOKENS", [96, 170])
    plain = plain_models["E"]
    kvh, heads, hd = plain.cfg["num_key_value_heads"], plain.cfg["num_attention_heads"], plain.cfg["head_dim"]
    n = 50
    assert ops_tc.decode_uses_warps(n, 1, hd, heads, kvh) and ops_tc.decode_uses_warps(n, 2, hd, heads, kvh)
    assert ops_tc.decode_warps_cluster(n, 1, kvh) == 1 and ops_tc.decode_warps_cluster(n, 2, kvh) == 1
    eng = Engine.from_pretrained(model_dirs["E"], dtype="bfloat16", max_tokens=n * 256)
    lens = [200 if i % 5 else 120 + i for i in range(n)]
    requests = [helpers.random_tokens(m, plain.cfg["vocab_size"], 300 + i) for i, m in enumerate(lens)]
    steps = helpers.batched_steps(requests, [60 + (i % 7) for i in range(n)], n)
    out = helpers.TraceRunner(eng, tmp_path / "many").run(steps)
    got = helpers.collect(steps, out, requests)
    for i, toks in enumerate(requests):
        want = plain.logits(toks).numpy()
        err = np.abs(got[i] - want).max(axis=1)
        assert err.max() < TOL["bfloat16"], f"request {i}: first bad position {int((err >= TOL['bfloat16']).argmax())}"
    classes = {key[1] for key, g in eng.stepper._graphs.items() if g.graph is not None}
    assert classes == {0, 1, 2}
    eng.cache.check()


@pytest.mark.parametrize("n", [1, 3, 6])
def test_few_sequences_decoding_across_the_context_classes(n, model_dirs, plain_models, tmp_path, monkeypatch):
    """Few sequences that grow across both class boundaries while they decode: in the longer classes
    2, 4 or 8 CTAs (a thread-block cluster) share each (sequence, KV head) and add up through the
    cluster's shared memory; the new token's tile may lie in any of them.  Every decoded position
    against the plain model."""
    from oracle_engine_b200.csrc import ops_tc
    from oracle_engine_b200.engine import batch
    from oracle_engine_b200.engine.engine import Engine
    monkeypatch.setattr(batch, "CONTEXT_CLASS_TOKENS", [64, 96, 170])
    plain = plain_models["E"]
    kvh = plain.cfg["num_key_value_heads"]
    sizes = [ops_tc.decode_warps_cluster(n, c, kvh) for c in (0, 1, 2, 3)]
    assert sizes[0] == 1 and sizes[1] > 1 and sizes[2] == sizes[1] and sizes[3] >= sizes[2]
    eng = Engine.from_pretrained(model_dirs["E"], dtype="bfloat16", max_tokens=n * 256)
    lens = [230 - 7 * i for i in range(n)]
    requests = [helpers.random_tokens(m, plain.cfg["vocab_size"], 700 + i) for i, m in enumerate(lens)]
    steps = helpers.batched_steps(requests, [40 + 3 * i for i in range(n)], n)
    out = helpers.TraceRunner(eng, tmp_path / "few").run(steps)
    got = helpers.collect(steps, out, requests)
    for i, toks in enumerate(requests):
        want = plain.logits(toks).numpy()
        err = np.abs(got[i] - want).max(axis=1)
        assert err.max() < TOL["bfloat16"], f"request {i}: first bad position {int((err >= TOL['bfloat16']).argmax())}"
    classes = {key[1] for key, g in eng.stepper._graphs.items() if g.graph is not None}
    assert classes == {0, 1, 2, 3}
    eng.cache.check()


def test_refusals(model_dirs):
    from oracle_engine_b200 import GenParams, SequenceStep
    from oracle_engine_b200.cache.slots import CacheFull
    from oracle_engine_b200.engine.step import StepError
    eng = _engine(model_dirs, "A", "float32", max_tokens=128)
    with pytest.raises(ValueError, match="exceeds the context"):
        eng.generate([[1] * 200], GenParams.greedy(2))
    slot = eng.alloc()
    with pytest.raises(StepError, match="outside the vocabulary"):
        eng.step([SequenceStep(slot, [1, 256], [0])])
    with pytest.raises(StepError, match="not allocated"):
        eng.step([SequenceStep(slot + 1, [1], [0])])
    with pytest.raises(StepError, match="twice"):
        eng.step([SequenceStep(slot, [1], [0]), SequenceStep(slot, [2], [0])])
    eng.step([SequenceStep(slot, [1] * 100, [])])
    other = eng.alloc()
    with pytest.raises(CacheFull):
        eng.step([SequenceStep(other, [1] * 100, [])])       # 128 tokens of cache: two pages, both taken
    eng.free(slot)
    eng.step([SequenceStep(other, [1] * 100, [99])])
    eng.free(other)
    eng.cache.check()


def test_command_line_generates_the_same_tokens(model_dirs, plain_models, tmp_path):
    """bin/oracle with token ids: greedy tokens of a batch, and seeded random weights from a config."""
    import json
    import subprocess
    import sys
    exe = [sys.executable, str(helpers.ROOT / "bin" / "oracle")]
    plain = plain_models["A"]
    prompts = [[3, 4, 5, 6], [9, 8]]
    r = subprocess.run(exe + ["-m", model_dirs["A"], "--tokens", "3,4,5,6", "--tokens", "9,8", "-n", "6", "--temp", "0",
                              "--dtype", "float32", "--ignore-eos"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    got = [[int(t) for t in line.split()] for line in r.stdout.strip().splitlines()]
    assert got == [pl.generate(plain, p, 6) for p in prompts]
    # streaming a single request prints the ids as they come
    r = subprocess.run(exe + ["-m", model_dirs["A"], "--tokens", "3,4,5,6", "-n", "6", "--temp", "0", "--dtype", "float32",
                              "--ignore-eos"], capture_output=True, text=True)
    assert r.returncode == 0 and [int(t) for t in r.stdout.split()] == got[0]
    cfg = tmp_path / "c.json"
    cfg.write_text((helpers.Path(model_dirs["A"]) / "config.json").read_text())
    r = subprocess.run(exe + ["--random-weights", "0", "--config", str(cfg), "--tokens", "3,4,5,6", "-n", "6", "--temp", "0",
                              "--dtype", "float32", "--ignore-eos", "--no-stream"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert [int(t) for t in r.stdout.split()] == got[0]          # seed 0 is the seed the folder was written with


def test_real_widths_bfloat16_against_float32():
    """Two layers with the widths of the benchmark model (hidden 3072, 24/8 heads of 128, FFN
    8192, vocabulary 128256): the bfloat16 kernels at their real shapes (tcgen05 tiles, swap
    and split paths, the weight-streaming kernel, the wide argmax) against the 32-bit path."""
    from oracle_engine_b200 import GenParams, LlamaConfig, SequenceStep
    from oracle_engine_b200.engine.engine import Engine
    raw = dict(architectures=["LlamaForCausalLM"], vocab_size=128256, hidden_size=3072, intermediate_size=8192,
               num_hidden_layers=2, num_attention_heads=24, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5,
               rope_theta=500000.0, rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                                                  "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
               max_position_embeddings=4096, tie_word_embeddings=True)
    cfg = LlamaConfig.from_dict(raw)
    lens = [300, 17, 130, 64, 1, 70, 200, 33, 90, 129, 5, 260]            # 12 sequences: a batch above 8 too
    prompts = [helpers.random_tokens(n, cfg.vocab_size, 200 + i) for i, n in enumerate(lens)]
    feed = [helpers.random_tokens(4, cfg.vocab_size, 300 + i) for i in range(len(lens))]
    outs = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_config(cfg, seed=3, dtype=dtype, max_tokens=12 * 384, norm_std=0.1)
        got = []
        for group in (range(0, 3), range(3, 12)):                         # 3 sequences, then 9
            idx = list(group)
            slots = [eng.alloc() for _ in idx]
            lg = eng.step([SequenceStep(s, prompts[i], [len(prompts[i]) - 1]) for s, i in zip(slots, idx)])
            step_logits = [lg.float().cpu()]
            for t in range(4):
                lg = eng.step([SequenceStep(s, [feed[i][t]], [0]) for s, i in zip(slots, idx)])
                step_logits.append(lg.float().cpu().clone())
            got.append(torch.stack(step_logits))
            for s in slots:
                eng.free(s)
        eng.check_device_errors()
        outs[dtype] = torch.cat(got, dim=1)
        del eng
        torch.cuda.empty_cache()
    ref, got = outs["float32"], outs["bfloat16"]
    scale = ref.abs().max().item()
    err = (ref - got).abs().max().item()
    assert scale > 0.5 and err < 0.03 * scale + 0.02, f"max abs err {err} at logit scale {scale}"
    # the most likely token agrees wherever the 32-bit margin is clear
    top2 = ref.topk(2, dim=-1).values
    clear = (top2[..., 0] - top2[..., 1]) > 4 * err
    assert clear.any()
    assert torch.equal(ref.argmax(-1)[clear], got.argmax(-1)[clear])


def test_generate_raises_when_a_kernel_reports_an_error(model_dirs):
    """A bounded wait that runs out inside a kernel during generation (made to, see the kernel test
    of the same path) reaches the caller of Engine.generate as an error, not as tokens; the engine
    generates as before afterwards."""
    from oracle_engine_b200 import GenParams
    from oracle_engine_b200.csrc import ops_tc
    # without graphs: a captured graph would keep the arguments its kernels were captured with, the knob's too
    eng = _engine(model_dirs, "E", "bfloat16", max_tokens=2048, use_graphs=False)
    prompts = [helpers.random_tokens(100, 389, 5)]                      # up to 128 tokens: the one-SM tcgen05 products
    good = eng.generate(prompts, GenParams.greedy(3, ignore_eos=True))
    with ops_tc.knobs(sm_count=1, gemm_waits=(2_000_000, 1)):           # the tiles of the prompt's products on one CTA
        with pytest.raises(RuntimeError, match="bounded wait"):
            eng.generate(prompts, GenParams.greedy(3, ignore_eos=True))
    assert eng.cache.slots.n_free == eng.cache.n_slots                  # the slots came back
    assert eng.generate(prompts, GenParams.greedy(3, ignore_eos=True)) == good
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_checksum_of_the_references_own_bench(tmp_path, dtype):
    """The engine's greedy tokens hash to the checksum that the reference's unmodified benchmark
    program printed on the same model and prompt (tests/golden/bench_checksum_B0.json)."""
    import json
    import plain_llama
    from test_plain import fnv1a
    from oracle_engine_b200 import GenParams, LlamaConfig, write_model_folder
    from oracle_engine_b200.engine.engine import Engine
    g = json.loads((helpers.ROOT / "tests" / "golden" / "bench_checksum_B0.json").read_text())
    write_model_folder(tmp_path / "m", LlamaConfig.from_dict(g["config"]), seed=g["seed"], std=g["std"])
    eng = Engine.from_pretrained(str(tmp_path / "m"), dtype=dtype, max_tokens=512)
    toks = eng.generate([g["prompt"]], GenParams.greedy(g["gen_tokens"], ignore_eos=True))[0]
    if dtype == "float32":
        assert f"{fnv1a(toks):016x}" == g["gen_checksum"]
        return
    # bfloat16: the same tokens up to a near tie, if there is one
    want = plain_llama.generate(plain_llama.PlainLlama(tmp_path / "m"), g["prompt"], g["gen_tokens"])
    k = next((i for i, (a, b) in enumerate(zip(toks, want)) if a != b), None)
    if k is not None:
        lg = plain_llama.PlainLlama(tmp_path / "m").logits(g["prompt"] + want[:k])[-1]
        assert float(lg[want[k]] - lg[toks[k]]) < 0.1, f"token {k}: {toks[k]} vs {want[k]}"
        assert k > 8


def test_bench_checksum_is_the_same_on_every_run(model_dirs):
    """The bench's end-to-end arm hashes its greedy tokens (FNV-1a, as the reference's bench does,
    benchmark/bench_engine.cpp:233-242): two runs give the same checksum, and so does a run that does
    not queue a step ahead of the host; unequal prompts as in the quoted workloads."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench", helpers.ROOT / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert bench.fnv1a([]) == 1469598103934665603 and bench.fnv1a([1]) != bench.fnv1a([2])     # the reference's offset
    eng = _engine(model_dirs, "E", "bfloat16", max_tokens=4096)
    lengths = [40, 7, 130, 64, 1]
    runs = [bench.time_e2e(eng, lengths, steps=12, warmup=3, vocab=389, lookahead=ahead) for ahead in (True, True, False)]
    assert runs[0]["tokens"] == len(lengths) * 16
    assert runs[0]["checksum"] == runs[1]["checksum"] == runs[2]["checksum"]
    assert runs[0]["h2d_bytes_per_step"] > 0 and runs[0]["d2h_bytes_per_step"] == 4 * len(lengths)
    dec = bench.time_decode(eng, lengths, steps=6, warmup=3, vocab=389, regions=3)
    assert dec["regions"] == 3 and dec["ms_min"] <= dec["ms_per_step"] <= dec["ms_max"] and dec["launches"] > 0
    weights = eng.model.step_bytes([])
    assert dec["step_bytes"] > weights > 0
    eng.cache.check()
