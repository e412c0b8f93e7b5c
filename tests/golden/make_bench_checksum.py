#!/usr/bin/env python3
"""Runs the reference's own benchmark program on a tiny model with this library's seeded random
weights and records the checksum it prints for its greedy tokens.

    python baseline/build_reference.py /path/to/oracle-engine      # builds baseline/_ref/oracle_bench
    python tests/golden/make_bench_checksum.py /path/to/oracle-engine

The reference's bench tiles an English sentence (benchmark/bench_engine.cpp:91-95, 195-201) to the
prompt length, prefills all but the last prompt token, then decodes greedily and hashes the tokens
with FNV-1a (:221-244).  The model file written here carries a byte-level vocabulary without merge
rules (baseline/gguf_export.py), so the sentence encodes to the begin-of-text id followed by one id
per byte (core/tokenizer.cpp:210-268); the ids are stored with the checksum, so the test needs
neither the reference nor its sentence.  The model is tiny configuration B without frequency scaling and
with the norm epsilon the reference always uses (1e-5), weights N(0, 0.1) so that the tokens vary.
Output: tests/golden/bench_checksum_B0.json.
"""
import json
import re
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path[:0] = [str(ROOT), str(ROOT / "tests"), str(ROOT / "baseline")]

N_PROMPT, N_GEN = 128, 64
SEED, STD = 1, 0.1


def reference_sentence(ref: Path) -> str:
    src = (ref / "benchmark" / "bench_engine.cpp").read_text()
    block = src[src.index("REF_PROMPT ="):]
    block = block[:block.index(";")]
    return "".join(re.findall(r'"((?:[^"\\]|\\.)*)"', block))


def main():
    if len(sys.argv) < 2:
        sys.exit(__doc__)
    ref = Path(sys.argv[1])
    import torch
    import gguf_export
    from conftest import TINY_B
    from oracle_engine_b200 import LlamaConfig
    from oracle_engine_b200.engine.runtime import Runtime
    from oracle_engine_b200.models.llama import build_spec
    from oracle_engine_b200.parts.model import DecoderModel
    from oracle_engine_b200.weights.random_init import RandomSource
    raw = dict(TINY_B, rope_scaling=None, rms_norm_eps=1e-5)
    cfg = LlamaConfig.from_dict(raw)
    model = DecoderModel(build_spec(cfg), Runtime(torch.float32, torch.device("cpu")))
    source = RandomSource(model.tensors(), SEED, torch.bfloat16, "cpu", std=STD)
    base = [0] + list(reference_sentence(ref).encode())                 # begin-of-text id 0, then one id per byte
    prompt = [base[i % len(base)] for i in range(N_PROMPT)]
    exe = ROOT / "baseline" / "_ref" / "oracle_bench"
    with tempfile.TemporaryDirectory() as tmp:
        gguf_export.write_gguf(f"{tmp}/B0.gguf", cfg, source)
        subprocess.run([str(exe), "-m", f"{tmp}/B0.gguf", "-p", str(N_PROMPT), "-g", str(N_GEN), "-r", "2", "-t", "1",
                        "--json", f"{tmp}/out.json"], check=True, stdout=subprocess.DEVNULL)
        out = json.loads(Path(f"{tmp}/out.json").read_text())
    assert out["prompt_tokens"] == N_PROMPT - 1 and out["gen_tokens"] == N_GEN
    (HERE / "bench_checksum_B0.json").write_text(json.dumps(
        {"config": raw, "seed": SEED, "std": STD, "prompt": prompt, "gen_tokens": N_GEN, "gen_checksum": out["gen_checksum"],
         "made_by": "oracle_bench (benchmark/bench_engine.cpp, unmodified) -p 128 -g 64 -r 2 -t 1"}, indent=1))
    print("checksum", out["gen_checksum"])


if __name__ == "__main__":
    main()
