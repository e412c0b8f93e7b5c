"""Trace replay: feeds given token ids through the engine step by step and writes logits.

It samples nothing and owns no model code: it drives `Engine.step`, the step function
that generation uses, with the engine's own cache and kernels.

Input, one JSON object per line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
`entries` gives each request's next tokens and the places among them whose logits are
wanted; a request id seen for the first time gets a cache slot.  `end` lists requests
that are finished after the step; their slots and pages are given back.  For a step in
which something is wanted the logits are written to `<out>/<step>.f32` as little-endian
float32 [wanted, vocab], in the order of the entries and of `want`.  After every step a
line `done <step>` is printed and flushed.

The closest thing in the reference is `forward_batch`, which returns the logits of given
tokens at given positions of one sequence (core/model.hpp:84-89).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np


def replay(engine, lines, out_dir: Path, log=sys.stdout) -> int:
    from .batch import SequenceStep

    out_dir.mkdir(parents=True, exist_ok=True)
    slots: dict[str, int] = {}
    n_steps = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        seqs = []
        for ent in rec.get("entries", []):
            rid = str(ent["id"])
            if rid not in slots:
                slots[rid] = engine.alloc()
            seqs.append(SequenceStep(slots[rid], [int(t) for t in ent["tokens"]],
                                     [int(w) for w in ent.get("want", [])]))
        if seqs:
            logits = engine.step(seqs)
            if logits is not None:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                np.ascontiguousarray(arr).tofile(out_dir / f"{step}.f32")
            engine.check_device_errors()
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slots:
                engine.free(slots.pop(rid))
        print(f"done {step}", file=log, flush=True)
        n_steps += 1
    for slot in slots.values():
        engine.free(slot)
    return n_steps


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description="replay token ids through the engine, write logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64); sizes the cache")
    ap.add_argument("--no-graphs", action="store_true", help="do not capture CUDA graphs for one-token steps")
    args = ap.parse_args(argv)

    from .engine import Engine
    engine = Engine.from_pretrained(args.model, dtype=args.dtype, max_tokens=args.max_tokens,
                                    use_graphs=not args.no_graphs)
    replay(engine, sys.stdin, Path(args.out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
