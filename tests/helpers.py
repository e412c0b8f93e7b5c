"""Helpers shared by the GPU tests: random requests, traces, and model variants."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent

# Tolerances, fixed from the arithmetic: float32 differs from the float64 plain model by
# accumulated rounding of a few thousand fused multiply-adds on O(1) values; bfloat16
# rounds activations to 2^-9 relative at every layer boundary.
TOL = {"float32": 2e-4, "bfloat16": 5e-2}


def random_tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def sharpen(src_dir, dst_dir, factor=8.0):
    """Copies a model folder with its query and key projections scaled up, so that the
    softmax is peaked and single keys (far ones too) decide the output."""
    import plain_llama
    from oracle_engine_b200.weights.safetensors_io import ModelFiles, write_safetensors
    dst = Path(dst_dir)
    dst.mkdir(parents=True, exist_ok=True)
    (dst / "config.json").write_text((Path(src_dir) / "config.json").read_text())
    files = ModelFiles(src_dir)
    tensors = {}
    for n in files.names():
        t = files.read(n).clone()
        if n.endswith("q_proj.weight") or n.endswith("k_proj.weight"):
            t = (t.float() * factor).to(t.dtype)
        tensors[n] = t
    write_safetensors(dst / "model.safetensors", tensors)
    files.close()
    return str(dst)


class TraceRunner:
    """Runs trace steps through an engine in-process (the same `replay` that bin/trace_run calls)."""

    def __init__(self, engine, out_dir):
        self.engine = engine
        self.out = Path(out_dir)

    def run(self, steps):
        from oracle_engine_b200.engine.replay import replay
        import io
        log = io.StringIO()
        replay(self.engine, [json.dumps(s) for s in steps], self.out, log=log)
        assert log.getvalue().split() == [w for s in steps for w in ("done", str(s["step"]))]
        return self.read(steps)

    def read(self, steps):
        vocab = self.engine.spec.vocab_size
        out = {}
        for s in steps:
            n_want = sum(len(e.get("want", [])) for e in s["entries"])
            f = self.out / f"{s['step']}.f32"
            if n_want:
                out[s["step"]] = np.fromfile(f, dtype="<f4").reshape(n_want, vocab)
            else:
                assert not f.exists()
        return out


def whole_steps(requests):
    """Each request alone and whole: one step per request, every position wanted."""
    return [{"step": i, "entries": [{"id": f"r{i}", "tokens": toks, "want": list(range(len(toks)))}],
             "end": [f"r{i}"]} for i, toks in enumerate(requests)]


def tail_steps(requests, tail=32):
    """Each request alone: all but the last `tail` tokens in one step, then one by one."""
    steps, k = [], 0
    for i, toks in enumerate(requests):
        head = max(1, len(toks) - tail)
        steps.append({"step": k, "entries": [{"id": f"r{i}", "tokens": toks[:head], "want": list(range(head))}],
                      "end": []})
        k += 1
        for j in range(head, len(toks)):
            steps.append({"step": k, "entries": [{"id": f"r{i}", "tokens": [toks[j]], "want": [0]}],
                          "end": [f"r{i}"] if j == len(toks) - 1 else []})
            k += 1
        if head == len(toks):
            steps[-1]["end"] = [f"r{i}"]
    return steps


def batched_steps(requests, prompt_lens, batch_size):
    """Batches of unequal lengths, one after another: a batch's prompts in one step (all
    positions wanted), then one token each; shorter requests end earlier."""
    steps, k = [], 0
    for b0 in range(0, len(requests), batch_size):
        ids = list(range(b0, min(len(requests), b0 + batch_size)))
        done_at = {i: len(requests[i]) for i in ids}
        ended = [f"r{i}" for i in ids if prompt_lens[i] == done_at[i]]
        steps.append({"step": k, "entries": [{"id": f"r{i}", "tokens": requests[i][:prompt_lens[i]],
                                               "want": list(range(prompt_lens[i]))} for i in ids], "end": ended})
        k += 1
        pos = {i: prompt_lens[i] for i in ids}
        while True:
            live = [i for i in ids if pos[i] < done_at[i]]
            if not live:
                break
            ended = [f"r{i}" for i in live if pos[i] + 1 == done_at[i]]
            steps.append({"step": k, "entries": [{"id": f"r{i}", "tokens": [requests[i][pos[i]]], "want": [0]}
                                                  for i in live], "end": ended})
            for i in live:
                pos[i] += 1
            k += 1
    return steps


def piece_steps(requests, plans, batch_size=None, step0=0):
    """Every request goes through in the pieces its plan lists (plans[i] sums to len(requests[i])):
    in step s of a batch each live request brings its piece s, so one step may hold a long prompt
    piece of one request beside single tokens of others; a request with fewer pieces ends earlier.
    Every position is wanted."""
    steps, k = [], step0
    batch_size = batch_size or len(requests)
    for b0 in range(0, len(requests), batch_size):
        ids = list(range(b0, min(len(requests), b0 + batch_size)))
        for i in ids:
            assert sum(plans[i]) == len(requests[i]) and min(plans[i]) >= 1, (i, plans[i], len(requests[i]))
        pos = {i: 0 for i in ids}
        for s in range(max(len(plans[i]) for i in ids)):
            live = [i for i in ids if s < len(plans[i])]
            entries = []
            for i in live:
                n = plans[i][s]
                entries.append({"id": f"r{i}", "tokens": requests[i][pos[i]:pos[i] + n], "want": list(range(n))})
                pos[i] += n
            steps.append({"step": k, "entries": entries, "end": [f"r{i}" for i in live if s == len(plans[i]) - 1]})
            k += 1
    return steps


def cut(n, sizes):
    """n as a list of pieces that cycle through `sizes` (the last one is what is left)."""
    out, j = [], 0
    while n > 0:
        out.append(min(n, sizes[j % len(sizes)]))
        n -= out[-1]
        j += 1
    return out


def collect(steps, outputs, requests):
    """Reassembles per-request logits [len, vocab] from a trace's outputs."""
    vocab = next(iter(outputs.values())).shape[1]
    got = [np.full((len(r), vocab), np.nan, dtype=np.float32) for r in requests]
    cursor = [0] * len(requests)
    for s in steps:
        row = 0
        for e in s["entries"]:
            i = int(e["id"][1:])
            for w in e.get("want", []):
                got[i][cursor[i] + w] = outputs[s["step"]][row]
                row += 1
            cursor[i] += len(e["tokens"])
    return got


def run_trace_cli(model_dir, dtype, steps, out_dir, max_tokens, env=None, extra=()):
    """bin/trace_run as a subprocess, steps fed one by one after each `done`."""
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens), *extra]
    p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    for s in steps:
        p.stdin.write(json.dumps(s) + "\n")
        p.stdin.flush()
        line = p.stdout.readline().strip()
        assert line == f"done {s['step']}", f"expected 'done {s['step']}', got {line!r}"
    p.stdin.close()
    assert p.wait(timeout=120) == 0
