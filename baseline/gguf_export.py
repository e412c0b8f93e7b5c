"""Writes a Llama model with this library's seeded random weights as a GGUF file that the
reference engine loads, so that `bench.py --impl reference` can run the reference's own
benchmark program on the benchmark model.

The container layout is what the reference's parser reads (core/gguf_parser.cpp:164-324:
magic, version 3, counts, typed key/values, tensor infos with the dimensions fastest
first, data aligned to 32 bytes); tensor names are its `blk.N.attn_q.weight` names
(core/model.cpp:99-112).  Matrices are stored as BF16 (type 30), norm weights as F32.
Its benchmark tokenises an English sentence, so the file also carries a byte-level
vocabulary: ids 0..255 are the 256 single-byte pieces (GPT-2's byte-to-character table,
core/tokenizer.cpp:15-36), the other ids are placeholders; with no merge rules the
sentence encodes to one id per byte.
"""
from __future__ import annotations

import struct
from pathlib import Path

import torch

GGUF_NAMES = {"self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v",
              "self_attn.o_proj": "attn_output", "mlp.gate_proj": "ffn_gate", "mlp.up_proj": "ffn_up",
              "mlp.down_proj": "ffn_down", "input_layernorm": "attn_norm", "post_attention_layernorm": "ffn_norm"}
F32, BF16 = 0, 30


def gguf_name(name: str) -> str:
    if name == "model.embed_tokens.weight":
        return "token_embd.weight"
    if name == "model.norm.weight":
        return "output_norm.weight"
    if name == "lm_head.weight":
        return "output.weight"
    _, _, layer, rest = name.split(".", 3)
    return f"blk.{layer}.{GGUF_NAMES[rest.rsplit('.', 1)[0]]}.weight"


def byte_pieces() -> list[str]:
    """The piece of each byte value: printable bytes stand for themselves, the others are
    moved to code points from 256 on."""
    keep = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    out, extra = [], 0
    for b in range(256):
        if b in keep:
            out.append(chr(b))
        else:
            out.append(chr(256 + extra))
            extra += 1
    return out


def _s(text: str) -> bytes:
    b = text.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, cfg, source, log=None) -> int:
    """cfg: a LlamaConfig; source: an object with names() and read(name) -> tensor (bfloat16 or
    float32).  Tensors are written one at a time.  Returns the file's size in bytes."""
    names = list(source.names())
    vocab = byte_pieces() + [f"<unused_{i}>" for i in range(256, cfg.vocab_size)]
    kv = [("general.architecture", 8, "llama"), ("llama.block_count", 4, cfg.num_hidden_layers),
          ("llama.attention.head_count", 4, cfg.num_attention_heads),
          ("llama.attention.head_count_kv", 4, cfg.num_key_value_heads),
          ("llama.embedding_length", 4, cfg.hidden_size), ("llama.feed_forward_length", 4, cfg.intermediate_size),
          ("llama.attention.key_length", 4, cfg.head_dim), ("llama.vocab_size", 4, cfg.vocab_size),
          ("llama.rope.freq_base", 6, cfg.rope_theta),
          ("llama.attention.layer_norm_rms_epsilon", 6, cfg.rms_norm_eps),
          ("tokenizer.ggml.bos_token_id", 4, 0), ("tokenizer.ggml.eos_token_id", 4, 1)]
    head = b"GGUF" + struct.pack("<IQQ", 3, len(names), len(kv) + 1)
    for key, kind, val in kv:
        head += _s(key) + struct.pack("<I", kind)
        head += _s(val) if kind == 8 else struct.pack("<I" if kind == 4 else "<f", val)
    head += _s("tokenizer.ggml.tokens") + struct.pack("<IIQ", 9, 8, len(vocab)) + b"".join(_s(t) for t in vocab)
    offset, infos = 0, []
    for name in names:
        info = source.info(name)
        kind = F32 if len(info.shape) == 1 else BF16
        size = (4 if kind == F32 else 2)
        for d in info.shape:
            size *= int(d)
        dims = list(reversed(info.shape))
        head += _s(gguf_name(name)) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", int(d)) for d in dims)
        head += struct.pack("<IQ", kind, offset)
        infos.append((name, kind, size))
        offset += size + (-size % 32)
    head += b"\0" * (-len(head) % 32)
    with open(path, "wb") as f:
        f.write(head)
        for name, kind, size in infos:
            t = source.read(name)
            t = t.to(torch.float32) if kind == F32 else t.to(torch.bfloat16).view(torch.int16)
            f.write(t.contiguous().cpu().numpy().tobytes())
            f.write(b"\0" * (-size % 32))
            if log is not None:
                log(name)
    return Path(path).stat().st_size
