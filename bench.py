#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on the Llama 3.2 3B shape (random weights).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]
    python bench.py --shape 1b --workload baseline      # 16 prompts of 64..2,048 tokens, 128 steps
    python bench.py --shape 8b --workload baseline      # 32 prompts of 128..4,096 tokens, 256 steps
    python bench.py --profile [--batch 64]              # device time per kind of kernel, on standard error
    python bench.py --impl reference --steps K          # the reference's own benchmark program (CPU)

Prints ONE JSON line.  `value` is decoded tokens per second at the given batch (default
8), timed on the device with CUDA events over exactly K decode steps after W warm-up
steps (the median of five such regions, each a fresh batch; `regions` gives the spread);
every sequence has a 512-token random prompt and a slot in a cache sized for a context of
8,192 tokens per sequence.  `e2e` is the same through the Python entry point
`Engine.generate` (host token ids in, host token ids out, every step's inputs copied from
pinned host memory and its tokens read back into pinned host memory; the loop queues step
k + 1 while the host still waits for step k's tokens, as `generate` always does, and the time is
taken between the arrivals of a sequence's tokens on the host).  `prefill` is one 2,048-token prompt,
`points` are decode at batch 1 and 64, `roofline` compares the bytes a decode step has to
read (every weight once, the cache of the live requests; summed from what the model's parts
report) with the measured HBM bandwidth.  `e2e.checksum` is the FNV-1a hash of the greedy
tokens of the end-to-end run: the same on every run.

Method as in the reference's bench (benchmark/bench_engine.cpp:221-278): prefill and
generation timed apart, greedy, warm-up discarded; synthetic token ids instead of its
tiled sentence.  The engine runs on one GPU: for --gpus N > 1 one line says so, exit 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The benchmark model: the Llama 3.2 3B shape (28 layers, hidden 3072, 24/8 heads of 128, FFN 8192, vocab 128256)
LLAMA_3B = dict(architectures=["LlamaForCausalLM"], vocab_size=128256, hidden_size=3072, intermediate_size=8192,
                num_hidden_layers=28, num_attention_heads=24, num_key_value_heads=8, head_dim=128,
                rms_norm_eps=1e-5, rope_theta=500000.0,
                rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                              "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
                max_position_embeddings=131072, tie_word_embeddings=True, bos_token_id=128000,
                eos_token_id=128001)
# Further shapes of the same architecture (not the headline): --shape 1b | 8b
LLAMA_1B = dict(LLAMA_3B, hidden_size=2048, num_hidden_layers=16, num_attention_heads=32, num_key_value_heads=8,
                head_dim=64, intermediate_size=8192)
LLAMA_8B = dict(LLAMA_3B, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                head_dim=128, intermediate_size=14336, tie_word_embeddings=False,
                rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                              "high_freq_factor": 4.0, "original_max_position_embeddings": 8192})
SHAPES = {"3b": ("llama-3.2-3b-shape", LLAMA_3B, 8192), "1b": ("llama-3.2-1b-shape", LLAMA_1B, 4096),
          "8b": ("llama-3.1-8b-shape", LLAMA_8B, 8192)}
PROMPT_LEN = 512
PREFILL_TOKENS = 2048
SEED = 2


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"])),
                    "source": "measured"}
        except (KeyError, ValueError, OSError):
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 50 ms while it is open."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __enter__(self):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()

    def summary(self):
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        os.unlink(self.file.name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def fnv1a(tokens) -> int:
    """FNV-1a over token ids, as the reference's bench hashes its greedy tokens
    (benchmark/bench_engine.cpp:233-242): the determinism check of a run."""
    h = 1469598103934665603
    for t in tokens:
        h ^= int(t) & 0xFFFFFFFF
        h = (h * 1099511628211) & ((1 << 64) - 1)
    return h


def random_prompts(lengths, vocab, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (int(n),), generator=g).tolist() for n in lengths]


def workload(shape: str, kind: str, batch: int, steps: int):
    """(prompt lengths, decode steps, context) of a run.  "fixed": `batch` prompts of 512 tokens (the
    headline configuration's workload).  "baseline": the workload the shape is quoted with: 3b as fixed;
    1b: 16 prompts of 64..2,048 tokens (seed 3), 128 steps, context 4,096; 8b: 32 prompts of 128..4,096
    tokens (seed 4), 256 steps, context 8,192."""
    import torch
    context = SHAPES[shape][2]
    if kind == "baseline" and shape in ("1b", "8b"):
        n, lo, hi, k, seed = (16, 64, 2048, 128, 3) if shape == "1b" else (32, 128, 4096, 256, 4)
        g = torch.Generator().manual_seed(seed)
        return torch.randint(lo, hi + 1, (n,), generator=g).tolist(), k, context
    return [PROMPT_LEN] * batch, steps, context


def time_decode(engine, lengths, steps, warmup, vocab, regions=5, settle_ms=0):
    """Device time of exactly `steps` decode steps (step function + greedy token choice on the
    device) after `warmup` untimed ones, for a batch whose prompts have the given lengths.  The
    whole thing (fresh slots, the prompts in one step, warm-up, the timed steps) is done `regions`
    times and the median region is reported, with the spread (the reference takes the median of its
    runs, benchmark/bench_engine.cpp:262-268).  The next tokens are fixed random ids so that nothing
    waits for the host."""
    import torch
    from oracle_engine_b200 import GenParams, SequenceStep
    from oracle_engine_b200.csrc import ops
    batch = len(lengths)
    prompts = random_prompts(lengths, vocab, 1000 + batch)
    feed = random_prompts([warmup + steps] * batch, vocab, 2000 + batch)
    params = GenParams.greedy(1)
    out = torch.empty(batch, dtype=torch.int32, device=engine.device)
    times, launches = [], 0
    for _ in range(regions):
        slots = [engine.alloc() for _ in range(batch)]
        row_slot = torch.tensor(slots, dtype=torch.int32, device=engine.device)
        try:
            engine.step([SequenceStep(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
            if settle_ms > 0:
                torch.cuda.synchronize()
                time.sleep(settle_ms / 1e3)

            def one(i):
                logits = engine.step([SequenceStep(s, [feed[b][i]], [0]) for b, s in enumerate(slots)])
                engine.sampler.sample(logits, row_slot, params, out)

            for i in range(warmup):
                one(i)
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            launches0 = ops.LAUNCHES[0]
            start.record()
            for i in range(warmup, warmup + steps):
                one(i)
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop))
            launches = ops.LAUNCHES[0] - launches0
            engine.check_device_errors()
        finally:
            for s in slots:
                engine.free(s)
    ms = statistics.median(times)
    # the bytes a step has to read, at the middle of the timed region
    contexts = [n + warmup + (steps + 1) / 2.0 for n in lengths]
    return {"ms_per_step": ms / steps, "ms_min": min(times) / steps, "ms_max": max(times) / steps,
            "regions": regions, "tok_s": batch * steps / (ms / 1e3), "launches": launches,
            "step_bytes": engine.model.step_bytes(contexts)}


def time_e2e(engine, lengths, steps, warmup, vocab, lookahead=True):
    """The same decode steps through Engine.generate's loop: host ids in, host ids out, greedy.
    Returns the rate between the arrivals of a sequence's tokens on the host, the bytes copied
    per step, and the FNV-1a checksum of everything that was generated."""
    from oracle_engine_b200 import GenParams
    from oracle_engine_b200.engine.engine import _Backend
    from oracle_engine_b200.engine.generate import run_generation
    batch = len(lengths)
    prompts = random_prompts(lengths, vocab, 1000 + batch)
    stamps = []

    def on_token(i, tok):
        if i == 0:                      # the token is on the host: its step has run and been read back
            stamps.append(time.perf_counter())

    backend = _Backend(engine)
    backend.supports_lookahead = bool(lookahead)
    params = GenParams.greedy(warmup + steps + 1, ignore_eos=True)
    results = run_generation(backend, prompts, params, batch_size=batch, stop_ids=(), on_token=on_token)
    dt = stamps[warmup + steps] - stamps[warmup]
    n_steps = warmup + steps + 1
    tokens = [t for r in results for t in r.tokens]
    return {"tok_s": batch * steps / dt, "ms_per_step": dt / steps * 1e3,
            "h2d_bytes_per_step": int(backend.h2d_bytes / n_steps), "d2h_bytes_per_step": int(backend.d2h_bytes / n_steps),
            "checksum": f"{fnv1a(tokens):016x}", "tokens": len(tokens)}


def time_prefill(engine, lengths, vocab, runs=9, warmup=3, settle_ms=0):
    """Median device time of ONE step that takes prompts of the given lengths (packed, no padding),
    wanting the last place of each; returns (ms, flops of that step).

    settle_ms: the device is left idle that long before every step, so that each is timed alone, at the
    clocks a lone prompt step gets.  Back to back (0) a dozen steps of 10 ms are a sustained load under the
    power cap (2,048 tokens: 11.6 against 10.1 ms), which is what the measured bf16 figures distinguish as
    "sustained" (1,354 TFLOP/s) and "burst" (1,631, the denominator used here)."""
    import torch
    from oracle_engine_b200 import SequenceStep
    prompts = random_prompts(lengths, vocab, 3000)
    times = []
    for r in range(warmup + runs):
        slots = [engine.alloc() for _ in prompts]
        torch.cuda.synchronize()
        if settle_ms > 0:
            time.sleep(settle_ms / 1e3)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.step([SequenceStep(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        stop.record()
        torch.cuda.synchronize()
        for s in slots:
            engine.free(s)
        if r >= warmup:
            times.append(start.elapsed_time(stop))
    engine.check_device_errors()
    return statistics.median(times), engine.model.step_flops([0] * len(lengths), lengths, len(lengths))


GRID_BATCHES = (1, 2, 3, 4, 6, 8, 10, 12, 16, 17, 24, 32, 33, 48, 64, 96, 128)
GRID_CONTEXTS = (128, 512, 1400, 2048, 6000)
GRID_PROMPTS = (16, 64, 128, 192, 256, 384, 512, 768, 1024, 1536, 2048, 4096, 8192)


def decode_grid(cfg, dtype, warmup, settle_ms, file):
    """The decode step over batch sizes and contexts: ms a step and, in brackets, the step's bytes over
    its time as a fraction of the measured HBM figure.  A cliff between neighbours in this table is how the
    faults of the launch chain were found (a kernel timed alone does not show them)."""
    from oracle_engine_b200.engine.engine import Engine
    pk = peaks()
    print("sequences  " + "  ".join(f"{c:>6d} tokens" for c in GRID_CONTEXTS), file=file, flush=True)
    for batch in GRID_BATCHES:
        cells = []
        for plen in GRID_CONTEXTS:
            if batch * (plen + 128) > 420000:            # keeps the cache under 50 GB
                cells.append("       -     ")
                continue
            engine = Engine.from_config(cfg, seed=SEED, dtype=dtype, max_tokens=batch * (plen + 128),
                                        max_seq_len=8192, n_slots=batch)
            d = time_decode(engine, [plen] * batch, 30, warmup, cfg.vocab_size, 3, settle_ms)
            frac = d["step_bytes"] / (d["ms_per_step"] * 1e-3) / 1e9 / pk["hbm_gbs"]
            cells.append(f"{d['ms_per_step']:6.3f} ({frac:4.2f})")
            del engine
        print(f"{batch:9d}  " + "  ".join(cells), file=file, flush=True)
    # one prompt alone, over its length: ms of the step and its flops over the measured bf16 figure
    engine = Engine.from_config(cfg, seed=SEED, dtype=dtype, max_tokens=2 * 8192, max_seq_len=8192, n_slots=2)
    print("prompt tokens      ms   tokens/s   of the bf16 figure", file=file, flush=True)
    for n in GRID_PROMPTS:
        ms, flops = time_prefill(engine, [n], cfg.vocab_size, runs=5, warmup=3)
        print(f"{n:13d}  {ms:6.2f}  {n / ms * 1e3:9.0f}   {flops / (ms * 1e-3) / 1e12 / pk['bf16_tflops']:.3f}", file=file, flush=True)


def profile_decode(engine, lengths, vocab, file):
    """Device time per kind of kernel of the prompt step (events between the launches) and of one
    decode step (events inside the captured graph), as tables on `file`.  An event between two
    kernels costs a few microseconds and keeps the second from starting while the first drains, so
    the decode step is also timed plain, and the table's last column takes each launch's share of
    the difference off again."""
    import torch
    from oracle_engine_b200 import GenParams, SequenceStep
    from oracle_engine_b200.engine.profile import KernelProfile
    batch = len(lengths)
    prompts = random_prompts(lengths, vocab, 1000 + batch)
    feed = random_prompts([40] * batch, vocab, 2000 + batch)
    out = torch.empty(batch, dtype=torch.int32, device=engine.device)
    greedy = GenParams.greedy(1)

    def run(first, count, slots, row_slot):
        for i in range(first, first + count):
            logits = engine.step([SequenceStep(s, [feed[b][i]], [0]) for b, s in enumerate(slots)])
            engine.sampler.sample(logits, row_slot, greedy, out)

    for profiled in (False, True):
        slots = [engine.alloc() for _ in range(batch)]
        row_slot = torch.tensor(slots, dtype=torch.int32, device=engine.device)
        try:
            if not profiled:
                engine.step([SequenceStep(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
                run(0, 8, slots, row_slot)                          # captures the plain graph
                torch.cuda.synchronize()
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                run(8, 20, slots, row_slot)
                stop.record()
                torch.cuda.synchronize()
                plain_us = start.elapsed_time(stop) / 20 * 1e3
                engine.stepper._graphs.clear()                      # the next capture gets the events
                continue
            with KernelProfile() as prompt_prof:                    # the second prompt step: nothing is loaded or allocated in it
                engine.step([SequenceStep(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
            prompt_prof.report(file, f"prompt step ({sum(lengths)} tokens; the first launch's time is the host's preparation)")
            with KernelProfile() as prof:                           # open before the decode graph is captured
                run(0, 8, slots, row_slot)
            prof.events = []                                        # the eager first step and the token choices: not the graph
            inside = sum(us for _, us in prof.graph_totals().values())
            per_launch = max(0.0, inside - plain_us) / max(1, len(prof.graph_events))
            print(f"decode step at batch {batch}: {plain_us:.1f} us plain, {inside:.1f} us with an event after every "
                  f"launch ({per_launch:.2f} us per launch, taken off in the last column)", file=file)
            if per_launch > 8.0:
                print("  (the events cost this step more than a launch usually does: its kernels normally start while their "
                      "predecessors drain; read the first column as upper bounds and the last as a rough share)", file=file)
            totals = prof.graph_totals()
            for kind, (n, us) in sorted(totals.items(), key=lambda kv: -kv[1][1]):
                net = max(0.0, us / n - per_launch)
                print(f"  {kind:<40s} {n:5d} x {us / n:8.1f} us  -> {net:8.1f} us  {100 * net * n / plain_us:5.1f} %", file=file)
        finally:
            for s in slots:
                engine.free(s)


def reference_arm(args) -> int:
    """Runs the reference's own benchmark program (benchmark/bench_engine.cpp, compiled unmodified
    by baseline/build_reference.py into baseline/_ref/) on the benchmark model: the Llama 3.2 3B
    shape with this library's seeded random weights, exported as a BF16 GGUF.  The reference is a
    CPU engine for one sequence with its context fixed at 512 tokens, so its numbers are decode at
    batch 1 after a 127-token prompt, and a prefill of 127 tokens: not the configuration of the
    other arm, which `same_config: false` says."""
    why = None
    exe = os.path.join(ROOT, "baseline", "_ref", "oracle_bench")
    if not os.path.isfile(exe):
        src = os.environ.get("ORACLE_REFERENCE_SRC")
        try:
            if not src:
                raise RuntimeError("set ORACLE_REFERENCE_SRC to the reference's source tree")
            sys.path.insert(0, os.path.join(ROOT, "baseline"))
            import build_reference
            from pathlib import Path
            build_reference.build(Path(src))
        except Exception as e:                               # noqa: BLE001 - reported as the reason
            why = f"the reference's benchmark program is not built (baseline/build_reference.py: {e})"
    if args.gpus != 1:
        why = "the reference runs one sequence on the CPU of one machine; there is nothing to launch on several GPUs"
    if why is None:
        try:
            return _run_reference(args, exe)
        except Exception as e:                               # noqa: BLE001
            why = f"the reference's benchmark program failed here: {e}"
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def _run_reference(args, exe) -> int:
    import torch
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import gguf_export
    from oracle_engine_b200 import LlamaConfig
    from oracle_engine_b200.engine.runtime import Runtime
    from oracle_engine_b200.models.llama import build_spec
    from oracle_engine_b200.parts.model import DecoderModel
    from oracle_engine_b200.weights.random_init import RandomSource
    model_name, shape_cfg, _ = SHAPES[args.shape]
    raw = dict(shape_cfg)
    layers_full = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = LlamaConfig.from_dict(raw)
    device = "cuda" if torch.cuda.is_available() else "cpu"
    model = DecoderModel(build_spec(cfg), Runtime(torch.float32, torch.device("cpu")))
    source = RandomSource(model.tensors(), SEED, torch.bfloat16, device)
    n_prompt, n_gen = 128, max(1, args.steps)
    with tempfile.TemporaryDirectory() as tmp:
        size = gguf_export.write_gguf(os.path.join(tmp, "model.gguf"), cfg, source)
        out_json = os.path.join(tmp, "out.json")
        t0 = time.perf_counter()
        # its own rule: the first run is a warm-up and is thrown away (bench_engine.cpp:246-259)
        proc = subprocess.run([exe, "-m", os.path.join(tmp, "model.gguf"), "-p", str(n_prompt), "-g", str(n_gen),
                               "-r", "2", "--json", out_json], capture_output=True, text=True)
        wall = time.perf_counter() - t0
        if proc.returncode != 0:
            raise RuntimeError(f"exit {proc.returncode}: {proc.stderr[-300:]}")
        rep = json.loads(open(out_json).read())
    gen, pre = rep["generation_tok_s"]["median"], rep["prefill_tok_s"]["median"]
    line = {
        "impl": "reference",
        "metric": "decode tok/s at batch 1 (%s, bf16 weights, fp32 arithmetic, CPU); prefill tok/s at %d tokens"
                  % (model_name, rep["prompt_tokens"]),
        "value": round(gen, 3), "unit": "tokens/s", "n_gpus": 1, "steps": n_gen, "warmup": args.warmup,
        "ms_per_step": round(1e3 / gen, 3) if gen > 0 else None, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 weights, fp32 compute", "same_config": False,
        "why_not_same_config": "the reference is a CPU engine for one sequence with its context fixed at 512 tokens "
                               "(core/model.cpp:64): batch 1, a 127-token prompt, no GPU",
        "data": "the reference's tiled sentence as byte-level ids, random-init weights N(0, 0.02) from seed 2",
        "config": {"model": model_name, "global_batch": 1, "seq_len": 512, "parallelism": "cpu, %d threads" % rep["threads"],
                   "layers": cfg.num_hidden_layers, "layers_full": layers_full, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "ffn": cfg.intermediate_size, "vocab": cfg.vocab_size, "prompt_len": rep["prompt_tokens"],
                   "file": "BF16 GGUF, %.1f GB" % (size / 1e9), "compiler": rep["compiler"], "flags": rep["flags"]},
        "e2e": {"value": round(gen, 3), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "note": "the program's own loop: host token in, host token out, no device"},
        "gpu_launches": 0,
        "prefill": {"value": round(pre, 3), "tokens": rep["prompt_tokens"]},
        "checksum": rep["gen_checksum"], "peak_rss_mb": rep["peak_rss_mb"], "wall_s": round(wall, 1),
    }
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--shape", default="3b", choices=sorted(SHAPES), help="3b is the headline configuration")
    ap.add_argument("--workload", default="fixed", choices=["fixed", "baseline"],
                    help="fixed: --batch prompts of 512 tokens; baseline: the workload the shape is quoted with "
                         "(1b: 16 prompts of 64..2,048 tokens, 128 steps; 8b: 32 prompts of 128..4,096 tokens, 256 steps)")
    ap.add_argument("--regions", type=int, default=5, help="timed regions of --steps steps; the median is reported")
    ap.add_argument("--settle-ms", type=int, default=100,
                    help="idle time between a region's prompt step and its warm-up steps, and before every timed "
                         "prompt step (see time_decode, time_prefill; 0: none)")
    ap.add_argument("--grid", action="store_true",
                    help="print the decode step's time over batch sizes and context lengths on standard error, "
                         "and nothing else")
    ap.add_argument("--profile", action="store_true",
                    help="print device time per kind of kernel of a prompt step and a decode step on standard error, "
                         "and nothing else")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(json.dumps({"error": f"--gpus {args.gpus}: this engine runs on one GPU; nothing was measured"}))
        return 2
    args.warmup = max(args.warmup, 3)

    import torch
    from oracle_engine_b200 import LlamaConfig
    from oracle_engine_b200.engine.engine import Engine

    model_name, shape_cfg, _ = SHAPES[args.shape]
    lengths, steps, context = workload(args.shape, args.workload, args.batch, args.steps)
    baseline_load = args.workload == "baseline" and args.shape in ("1b", "8b")
    batch = len(lengths)
    raw = dict(shape_cfg)
    layers_full = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = LlamaConfig.from_dict(raw)
    pk = peaks()
    if args.grid:
        decode_grid(cfg, args.dtype, args.warmup, args.settle_ms, sys.stderr)
        return 0
    points_wanted = not args.no_points and not baseline_load and not args.profile
    max_batch = max(batch, 64) if points_wanted else batch
    engine = Engine.from_config(cfg, seed=SEED, dtype=args.dtype, max_tokens=max_batch * context,
                                max_seq_len=context, n_slots=max_batch)
    if args.profile:
        profile_decode(engine, lengths, cfg.vocab_size, sys.stderr)
        return 0

    with ClockSampler() as clocks:
        dec = time_decode(engine, lengths, steps, args.warmup, cfg.vocab_size, max(1, args.regions), args.settle_ms)
    clock_info = clocks.summary()
    e2e = time_e2e(engine, lengths, steps, args.warmup, cfg.vocab_size)
    points = {}
    if points_wanted:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(time_decode(engine, [PROMPT_LEN] * b, min(steps, 128), args.warmup,
                                                       cfg.vocab_size, 3, args.settle_ms)["tok_s"], 1)
    prefill = None
    if not args.no_prefill:
        pre_lengths = lengths if baseline_load else [PREFILL_TOKENS]
        ms, fl = time_prefill(engine, pre_lengths, cfg.vocab_size, settle_ms=args.settle_ms)
        prefill = {"value": round(sum(pre_lengths) / (ms / 1e3), 1), "tokens": sum(pre_lengths), "ms": round(ms, 3),
                   "frac": round(fl / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
        if args.settle_ms > 0:                     # the same steps back to back: a sustained load under the power cap
            ms_b2b, _ = time_prefill(engine, pre_lengths, cfg.vocab_size, runs=5)
            prefill["ms_back_to_back"] = round(ms_b2b, 3)
            prefill["settle_ms"] = args.settle_ms

    achieved = dec["step_bytes"] / (dec["ms_per_step"] / 1e3) / 1e9
    names = {"3b": "Llama 3.2 3B shape", "1b": "Llama 3.2 1B shape", "8b": "Llama 3.1 8B shape"}
    prompts_text = "%d..%d" % (min(lengths), max(lengths)) if baseline_load else str(PROMPT_LEN)
    line = {
        "metric": "decode tok/s at batch %d (%s, %s); prefill tok/s at %s tokens%s"
                  % (batch, names[args.shape], "bf16" if args.dtype == "bfloat16" else "fp32",
                     "{:,}".format(prefill["tokens"] if prefill else PREFILL_TOKENS),
                     "; points at batch 1 and 64" if points_wanted else ""),
        "value": round(dec["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": args.warmup, "ms_per_step": round(dec["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic token ids, random-init weights N(0, 0.02) from seed 2",
        "config": {"model": model_name, "global_batch": batch, "seq_len": context,
                   "parallelism": "single-gpu", "layers": cfg.num_hidden_layers, "layers_full": layers_full,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "ffn": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "prompt_len": prompts_text, "prefill_tokens": prefill["tokens"] if prefill else PREFILL_TOKENS,
                   "tied_head": cfg.tie_word_embeddings,
                   "rope": "llama3 factor %g" % cfg.rope_scaling.factor,
                   "l2": "inputs larger than L2 (weights %.1f GB per step)" % (engine.model.step_bytes([]) / 1e9),
                   "peaks": pk["source"], "workload": args.workload, "settle_ms_after_prompt": args.settle_ms},
        "regions": {"n": dec["regions"], "ms_per_step_min": round(dec["ms_min"], 4),
                    "ms_per_step_max": round(dec["ms_max"], 4), "reported": "median"},
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tokens/s", "ms_per_step": round(e2e["ms_per_step"], 4),
                "h2d_bytes_per_step": e2e["h2d_bytes_per_step"], "d2h_bytes_per_step": e2e["d2h_bytes_per_step"],
                "checksum": e2e["checksum"], "tokens": e2e["tokens"]},
        "gpu_launches": dec["launches"],
        "clocks": clock_info,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(dec["step_bytes"])},
        "points": points,
    }
    if prefill is not None:
        line["prefill"] = prefill
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
