#!/usr/bin/env python3
"""Makes the golden logits under tests/golden/ by running the reference's own model code.

The reference (Titouan935/oracle-engine, C++17, CPU) is compiled here from its source tree
with g++, and a small driver (written for this purpose, below) calls its public
`Model::load`, `Model::forward_prefill(tokens, n, 0, out_logits)` and `Model::forward(token,
pos)`.  The model it loads is a tiny random Llama written by this library's
`write_model_folder(config, seed)` and re-exported as a GGUF v3 file with F32 tensors
(container layout: core/gguf_parser.cpp:164-198, 307-324; dimensions are stored fastest
first, core/gguf_parser.cpp:448-449).

Two cases, both inside what the reference can run (no rotary frequency scaling, and norm
epsilon 1e-5, which is what its norms use whatever the file says, core/ops.hpp:43):
  A   2 layers, 4 heads / 2 KV heads, head_dim 16, theta 1e4, tied head
  B0  3 layers, 6 heads / 2 KV heads, head_dim 32, theta 5e5, separate head
The weights are a pure function of (config, seed), so the test regenerates them and only
the token ids and the reference's logits are stored (`<case>.json`, `<case>.npy`).

Usage:  python tests/golden/make_golden.py /path/to/oracle-engine
"""
import json
import os
import struct
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

CASES = {
    "A": (dict(architectures=["LlamaForCausalLM"], vocab_size=256, hidden_size=64, intermediate_size=160,
               num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-5,
               rope_theta=10000.0, max_position_embeddings=128, tie_word_embeddings=True), 0, 14),
    "B0": (dict(architectures=["LlamaForCausalLM"], vocab_size=384, hidden_size=192, intermediate_size=512,
                num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=2, head_dim=32,
                rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=512,
                tie_word_embeddings=False), 1, 20),
}

DRIVER = r"""
#include "core/model.hpp"
#include <cstdio>
#include <cstdlib>
#include <vector>
int main(int argc, char** argv) {
    // argv: model.gguf out.bin tok0 tok1 ...
    Model m;
    if (!m.load(argv[1])) return 1;
    std::vector<int32_t> toks;
    for (int i = 3; i < argc; i++) toks.push_back(std::atoi(argv[i]));
    const int n = (int)toks.size(), V = (int)m.cfg.n_vocab;
    std::vector<float> all((size_t)2 * n * V);
    m.reset();
    m.forward_prefill(toks.data(), n, 0, all.data());                 // whole prompt
    m.reset();
    for (int t = 0; t < n; t++) {                                      // token by token
        const float* lg = m.forward(toks[t], t);
        for (int v = 0; v < V; v++) all[(size_t)(n + t) * V + v] = lg[v];
    }
    FILE* f = std::fopen(argv[2], "wb");
    std::fwrite(all.data(), sizeof(float), all.size(), f);
    std::fclose(f);
    return 0;
}
"""

GGUF_NAMES = {"self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v",
              "self_attn.o_proj": "attn_output", "mlp.gate_proj": "ffn_gate", "mlp.up_proj": "ffn_up",
              "mlp.down_proj": "ffn_down", "input_layernorm": "attn_norm", "post_attention_layernorm": "ffn_norm"}


def gguf_name(name: str) -> str:
    if name == "model.embed_tokens.weight":
        return "token_embd.weight"
    if name == "model.norm.weight":
        return "output_norm.weight"
    if name == "lm_head.weight":
        return "output.weight"
    _, _, layer, rest = name.split(".", 3)
    return f"blk.{layer}.{GGUF_NAMES[rest.rsplit('.', 1)[0]]}.weight"


def _s(text: str) -> bytes:
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, cfg: dict, tensors: dict) -> None:
    hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    kv = [("general.architecture", 8, "llama"), ("llama.block_count", 4, cfg["num_hidden_layers"]),
          ("llama.attention.head_count", 4, cfg["num_attention_heads"]),
          ("llama.attention.head_count_kv", 4, cfg["num_key_value_heads"]),
          ("llama.embedding_length", 4, cfg["hidden_size"]),
          ("llama.feed_forward_length", 4, cfg["intermediate_size"]),
          ("llama.attention.key_length", 4, hd), ("llama.vocab_size", 4, cfg["vocab_size"]),
          ("llama.rope.freq_base", 6, cfg["rope_theta"]),
          ("llama.attention.layer_norm_rms_epsilon", 6, cfg["rms_norm_eps"])]
    out = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(kv))
    for key, kind, val in kv:
        out += _s(key) + struct.pack("<I", kind)
        out += _s(val) if kind == 8 else struct.pack("<I" if kind == 4 else "<f", val)
    offset, blobs = 0, []
    for name, t in tensors.items():
        arr = t.to(torch.float32).numpy()
        dims = list(reversed(arr.shape))
        out += _s(gguf_name(name)) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", 0, offset)                    # type 0 = F32
        blob = arr.tobytes()
        blob += b"\0" * (-len(blob) % 32)
        blobs.append(blob)
        offset += len(blob)
    out += b"\0" * (-len(out) % 32)
    Path(path).write_bytes(out + b"".join(blobs))


def main():
    if len(sys.argv) < 2:
        sys.exit(__doc__)
    ref = Path(sys.argv[1])
    from oracle_engine_b200 import LlamaConfig, write_model_folder
    from oracle_engine_b200.weights.safetensors_io import ModelFiles
    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        (tmp / "driver.cpp").write_text(DRIVER)
        srcs = [str(ref / "core" / f) for f in ("model.cpp", "gguf_parser.cpp", "ops.cpp", "platform.cpp")]
        srcs.append(str(ref / "bug" / "logger.cpp"))
        exe = tmp / "driver"
        subprocess.run(["g++", "-std=c++17", "-O2", "-mavx2", "-mfma", f"-I{ref}", str(tmp / "driver.cpp"),
                        *srcs, "-o", str(exe), "-lpthread"], check=True)
        for name, (raw, seed, n) in CASES.items():
            folder = tmp / name
            write_model_folder(folder, LlamaConfig.from_dict(raw), seed=seed)
            files = ModelFiles(folder)
            write_gguf(tmp / f"{name}.gguf", raw, {k: files.read(k) for k in files.names()})
            g = torch.Generator().manual_seed(100 + seed)
            tokens = torch.randint(0, raw["vocab_size"], (n,), generator=g).tolist()
            subprocess.run([str(exe), str(tmp / f"{name}.gguf"), str(tmp / f"{name}.bin"), *map(str, tokens)],
                           check=True, stdout=subprocess.DEVNULL)
            logits = np.fromfile(tmp / f"{name}.bin", dtype="<f4").reshape(2, n, raw["vocab_size"])
            np.save(HERE / f"{name}.npy", logits)
            (HERE / f"{name}.json").write_text(json.dumps(
                {"config": raw, "seed": seed, "tokens": tokens,
                 "rows": ["forward_prefill(tokens, n, 0, out_logits)", "forward(token, pos) one by one"]}, indent=1))
            print(name, logits.shape, "prefill vs step max diff", float(np.abs(logits[0] - logits[1]).max()))


if __name__ == "__main__":
    main()
