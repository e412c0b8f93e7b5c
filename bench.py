#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on the Llama 3.2 3B shape (random weights).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]

Prints ONE JSON line.  `value` is decoded tokens per second at the given batch (default
8), timed on the device with CUDA events over exactly K decode steps after W warm-up
steps; every sequence has a 512-token random prompt and a slot in a cache sized for a
context of 8,192 tokens per sequence.  `e2e` is the same through the Python entry point
`Engine.generate` (host token ids in, host token ids out, every step's inputs copied from
pinned host memory and its tokens read back into pinned host memory; the loop queues step
k + 1 while the host still waits for step k's tokens, as `generate` always does, and the time is
taken between the arrivals of a sequence's tokens on the host).  `prefill` is one 2,048-token prompt,
`points` are decode at batch 1 and 64, `roofline` compares the bytes a decode step has to
read (every weight once, the cache of the live requests) with the measured HBM bandwidth.

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
CONTEXT = 8192
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


def model_numbers(cfg):
    """Bytes a decode step must read and flops of a prompt, from the configuration."""
    D, FF, V, L = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size, cfg.num_hidden_layers
    H, KVH, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    per_layer = (H * hd * D) + 2 * (KVH * hd * D) + (D * H * hd) + 3 * D * FF
    head = V * D
    weight_bytes = 2 * (L * per_layer + head) + 4 * (2 * L + 1) * D
    kv_bytes_per_token = 2 * L * 2 * KVH * hd
    return {"matmul_params_per_layer": per_layer, "head_params": head, "weight_bytes": weight_bytes,
            "kv_bytes_per_token": kv_bytes_per_token}


def prefill_flops(cfg, T):
    n = model_numbers(cfg)
    L, H, hd = cfg.num_hidden_layers, cfg.num_attention_heads, cfg.head_dim
    gemm = 2.0 * T * L * n["matmul_params_per_layer"] + 2.0 * n["head_params"]      # head on the last row only
    attn = L * 2.0 * 2.0 * H * hd * (T * (T + 1) / 2.0)                              # causal QK^T and PV
    return gemm + attn


def random_prompts(n, length, vocab, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n, length), generator=g).tolist()


def time_decode(engine, batch, steps, warmup, vocab):
    """Device time of exactly `steps` decode steps (step function + greedy token choice on
    the device) at `batch`; the next tokens are fixed random ids so that nothing waits for
    the host."""
    import torch
    from oracle_engine_b200 import GenParams, SequenceStep
    from oracle_engine_b200.csrc import ops
    prompts = random_prompts(batch, PROMPT_LEN, vocab, 1000 + batch)
    feed = random_prompts(batch, warmup + steps, vocab, 2000 + batch)
    slots = [engine.alloc() for _ in range(batch)]
    params = GenParams.greedy(1)
    row_slot = torch.tensor(slots, dtype=torch.int32, device=engine.device)
    out = torch.empty(batch, dtype=torch.int32, device=engine.device)
    try:
        engine.step([SequenceStep(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])

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
        ms = start.elapsed_time(stop)
        launches = ops.LAUNCHES[0] - launches0
        mean_ctx = PROMPT_LEN + warmup + (steps + 1) / 2.0
        engine.check_device_errors()
    finally:
        for s in slots:
            engine.free(s)
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "launches": launches,
            "mean_context": mean_ctx}


def time_e2e(engine, batch, steps, warmup, vocab):
    """The same decode steps through Engine.generate: host ids in, host ids out."""
    from oracle_engine_b200 import GenParams
    from oracle_engine_b200.engine.engine import _Backend
    from oracle_engine_b200.engine.generate import run_generation
    import torch
    prompts = random_prompts(batch, PROMPT_LEN, vocab, 1000 + batch)
    stamps = []

    def on_token(i, tok):
        if i == 0:                      # the token is on the host: its step has run and been read back
            stamps.append(time.perf_counter())

    backend = _Backend(engine)
    params = GenParams.greedy(warmup + steps + 1, ignore_eos=True)
    run_generation(backend, prompts, params, batch_size=batch, stop_ids=(), on_token=on_token)
    dt = stamps[warmup + steps] - stamps[warmup]
    n_steps = warmup + steps + 1
    return {"tok_s": batch * steps / dt, "ms_per_step": dt / steps * 1e3,
            "h2d_bytes_per_step": int(backend.h2d_bytes / n_steps), "d2h_bytes_per_step": int(backend.d2h_bytes / n_steps)}


def time_prefill(engine, vocab, runs=9, warmup=3):
    import torch
    from oracle_engine_b200 import SequenceStep
    prompt = random_prompts(1, PREFILL_TOKENS, vocab, 3000)[0]
    times = []
    for r in range(warmup + runs):
        slot = engine.alloc()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.step([SequenceStep(slot, prompt, [len(prompt) - 1])])
        stop.record()
        torch.cuda.synchronize()
        engine.free(slot)
        if r >= warmup:
            times.append(start.elapsed_time(stop))
    return statistics.median(times)


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
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a C++/CMake CPU program with no setup.py or pyproject.toml: "
                          "pip cannot install it offline, and it has no GPU or bf16 path"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": f"--gpus {args.gpus}: this engine runs on one GPU; nothing was measured"}))
        return 2
    args.warmup = max(args.warmup, 3)

    import torch
    from oracle_engine_b200 import LlamaConfig
    from oracle_engine_b200.engine.engine import Engine

    global CONTEXT
    model_name, shape_cfg, CONTEXT = SHAPES[args.shape]
    raw = dict(shape_cfg)
    layers_full = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = LlamaConfig.from_dict(raw)
    pk = peaks()
    max_batch = args.batch if args.no_points else max(args.batch, 64)
    engine = Engine.from_config(cfg, seed=SEED, dtype=args.dtype, max_tokens=max_batch * CONTEXT,
                                max_seq_len=CONTEXT, n_slots=max_batch)
    nums = model_numbers(cfg)
    itemsize = 2 if args.dtype == "bfloat16" else 4

    with ClockSampler() as clocks:
        dec = time_decode(engine, args.batch, args.steps, args.warmup, cfg.vocab_size)
    clock_info = clocks.summary()
    e2e = time_e2e(engine, args.batch, args.steps, args.warmup, cfg.vocab_size)
    points = {}
    if not args.no_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(time_decode(engine, b, min(args.steps, 128), args.warmup,
                                                       cfg.vocab_size)["tok_s"], 1)
    prefill = None
    if not args.no_prefill:
        ms = time_prefill(engine, cfg.vocab_size)
        fl = prefill_flops(cfg, PREFILL_TOKENS)
        prefill = {"value": round(PREFILL_TOKENS / (ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(ms, 3),
                   "frac": round(fl / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}

    step_bytes = nums["weight_bytes"] * itemsize / 2 + args.batch * dec["mean_context"] * nums["kv_bytes_per_token"] \
        * itemsize / 2
    achieved = step_bytes / (dec["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": "decode tok/s at batch %d (%s, %s); prefill tok/s at 2,048 tokens; points at batch 1 and 64"
                  % (args.batch, {"3b": "Llama 3.2 3B shape", "1b": "Llama 3.2 1B shape", "8b": "Llama 3.1 8B shape"}[args.shape],
                     "bf16" if args.dtype == "bfloat16" else "fp32"),
        "value": round(dec["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(dec["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic token ids, random-init weights N(0, 0.02) from seed 2",
        "config": {"model": model_name, "global_batch": args.batch, "seq_len": CONTEXT,
                   "parallelism": "single-gpu", "layers": cfg.num_hidden_layers, "layers_full": layers_full,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "ffn": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "prompt_len": PROMPT_LEN, "prefill_tokens": PREFILL_TOKENS, "tied_head": cfg.tie_word_embeddings,
                   "rope": "llama3 factor %g" % cfg.rope_scaling.factor,
                   "l2": "inputs larger than L2 (weights %.1f GB per step)" % (nums["weight_bytes"] / 1e9),
                   "peaks": pk["source"]},
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tokens/s", "ms_per_step": round(e2e["ms_per_step"], 4),
                "h2d_bytes_per_step": e2e["h2d_bytes_per_step"], "d2h_bytes_per_step": e2e["d2h_bytes_per_step"]},
        "gpu_launches": dec["launches"],
        "clocks": clock_info,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
        "points": points,
    }
    if prefill is not None:
        line["prefill"] = prefill
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
