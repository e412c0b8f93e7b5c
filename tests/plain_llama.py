"""Plain, slow implementation of the Llama dense decoder, used only by the tests.

It rests on the formulas of the reference engine (Titouan935/oracle-engine), restated
with whole-sequence float64 tensor operations on the CPU: no cache, no batching, one
function per part, and no code shared with the product package.  (`PlainLlama(folder,
device="cuda")` holds the same float64 tensors on the GPU; only the tests with sequences of
thousands of tokens use it, to stay within minutes.)  Two things the reference does not
have are taken from the model's config.json instead: the llama3 frequency scaling of the
rotary angles, and a norm epsilon that is actually passed to the norm (the reference
reads it, core/model.cpp:61, but calls rmsnorm with the default of core/ops.hpp:43).

Each function cites the reference lines whose arithmetic it restates.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

# ----------------------------------------------------------------------------------------
# files
# ----------------------------------------------------------------------------------------

_ST_DTYPES = {"F32": (np.float32, 4), "BF16": (np.uint16, 2), "F16": (np.float16, 2),
              "I32": (np.int32, 4), "I64": (np.int64, 8), "F64": (np.float64, 8)}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """Reads every tensor of a safetensors file as float64/int64 CPU tensors.

    The file is an 8-byte little-endian header length, a JSON header
    {name: {dtype, shape, data_offsets}} and the raw bytes."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        np_dtype, _ = _ST_DTYPES[info["dtype"]]
        b, e = info["data_offsets"]
        arr = np.frombuffer(raw[base + b: base + e], dtype=np_dtype)
        if info["dtype"] == "BF16":
            arr = (arr.astype(np.uint32) << 16).view(np.float32)
        t = torch.from_numpy(np.array(arr)).reshape(info["shape"])
        out[name] = t.to(torch.int64) if info["dtype"] in ("I32", "I64") else t.to(torch.float64)
    return out


def read_config(folder) -> dict:
    return json.loads((Path(folder) / "config.json").read_text())


# ----------------------------------------------------------------------------------------
# parts (one function each)
# ----------------------------------------------------------------------------------------

def embed(tokens: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x = E[token]  (core/model.cpp:358, 550-558)."""
    return table[tokens]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """s = 1/sqrt(mean(x^2) + eps); y = (x * s) * w  (core/ops.cpp:189-194)."""
    ss = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    s = 1.0 / torch.sqrt(ss + eps)
    return (x * s) * weight


def rope_inv_freq(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """f_i = theta^(-2i/head_dim), i < head_dim/2  (core/ops.cpp:461-463).

    With rope_scaling of type llama3 (absent from the reference; from config.json):
    wavelength l_i = 2*pi/f_i; l_i < orig/high keeps f_i; l_i > orig/low gives f_i/factor;
    between them s = (orig/l_i - low)/(high - low), f_i' = (1-s)*f_i/factor + s*f_i."""
    half = head_dim // 2
    i = torch.arange(half, dtype=torch.float64)
    f = theta ** (-(2.0 * i) / head_dim)
    if scaling is None:
        return f
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return f
    assert kind == "llama3", kind
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    out = f.clone()
    for j in range(half):
        wavelen = 2.0 * math.pi / f[j].item()
        if wavelen < orig / high:
            continue
        if wavelen > orig / low:
            out[j] = f[j] / factor
        else:
            s = (orig / wavelen - low) / (high - low)
            out[j] = (1.0 - s) * f[j] / factor + s * f[j]
    return out


def rope_rotate(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """Rotate-half pairing (i, i+half) on x [n, heads, head_dim] at absolute positions:
    x'_i = x_i cos - x_{i+half} sin;  x'_{i+half} = x_i sin + x_{i+half} cos
    (core/ops.cpp:467-474)."""
    half = x.shape[-1] // 2
    ang = positions.to(device=x.device, dtype=torch.float64)[:, None] * inv_freq.to(x.device)[None, :]      # [n, half]
    cos = torch.cos(ang)[:, None, :].to(x.dtype)
    sin = torch.sin(ang)[:, None, :].to(x.dtype)
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1)


def softmax_rows(s: torch.Tensor) -> torch.Tensor:
    """Subtract the maximum, exponentiate, divide by the sum  (core/ops.cpp:386-435)."""
    m = s.max(dim=-1, keepdim=True).values
    e = torch.exp(s - m)
    return e / e.sum(dim=-1, keepdim=True)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     window: int | None = None) -> torch.Tensor:
    """q [n, H, hd], k/v [n, KVH, hd] of one whole sequence -> [n, H*hd].

    Query head h reads KV head h // (H/KVH); s_t = q.k_t / sqrt(hd) for keys t <= p;
    softmax; o = sum_t s_t v_t  (core/model.cpp:411-435, 605-626).  `window` keeps only
    keys p-window < t <= p (not used by the reference; for toy parts in tests)."""
    n, H, hd = q.shape
    KVH = k.shape[1]
    group = H // KVH
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros(n, H, hd, dtype=q.dtype, device=q.device)
    pos = torch.arange(n, device=q.device)
    allowed = pos[None, :] <= pos[:, None]
    if window is not None:
        allowed &= pos[None, :] > pos[:, None] - window
    for h in range(H):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        out[:, h, :] = softmax_rows(s) @ v[:, kh, :]
    return out.reshape(n, H * hd)


def swiglu_ffn(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
               w_down: torch.Tensor) -> torch.Tensor:
    """g = Wg x; u = Wu x; a = g/(1+exp(-g)) * u; y = Wd a  (core/model.cpp:636-642)."""
    g = x @ w_gate.T
    u = x @ w_up.T
    a = (g / (1.0 + torch.exp(-g))) * u
    return a @ w_down.T


def lm_head(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """logits = W x, W the separate head if it exists, else the embedding table
    (core/model.cpp:482-492)."""
    return x @ w.T


# ----------------------------------------------------------------------------------------
# whole model
# ----------------------------------------------------------------------------------------

class PlainLlama:
    """config.json + model.safetensors -> logits of a whole sequence."""

    def __init__(self, folder, dtype=torch.float64, device="cpu"):
        self.cfg = read_config(folder)
        self.dtype = dtype
        self.device = device
        self.w = {k: (v.to(dtype) if v.dtype.is_floating_point else v).to(device)
                  for k, v in read_safetensors(Path(folder) / "model.safetensors").items()}
        c = self.cfg
        self.n_layers = c["num_hidden_layers"]
        self.H = c["num_attention_heads"]
        self.KVH = c.get("num_key_value_heads", self.H)
        self.D = c["hidden_size"]
        self.hd = c.get("head_dim") or self.D // self.H
        self.eps = c["rms_norm_eps"]
        self.inv_freq = rope_inv_freq(self.hd, float(c.get("rope_theta", 10000.0)),
                                      c.get("rope_scaling"))
        self.tied = bool(c.get("tie_word_embeddings", False))

    def hidden(self, tokens) -> torch.Tensor:
        """Residual stream after the last layer, [n, D]  (core/model.cpp:361-474)."""
        w = self.w
        tokens = torch.as_tensor(tokens, dtype=torch.int64).to(self.device)
        n = tokens.numel()
        pos = torch.arange(n, device=self.device)
        x = embed(tokens, w["model.embed_tokens.weight"])
        for l in range(self.n_layers):
            p = f"model.layers.{l}."
            h = rms_norm(x, w[p + "input_layernorm.weight"], self.eps)
            q = (h @ w[p + "self_attn.q_proj.weight"].T).reshape(n, self.H, self.hd)
            k = (h @ w[p + "self_attn.k_proj.weight"].T).reshape(n, self.KVH, self.hd)
            v = (h @ w[p + "self_attn.v_proj.weight"].T).reshape(n, self.KVH, self.hd)
            q = rope_rotate(q, pos, self.inv_freq)
            k = rope_rotate(k, pos, self.inv_freq)
            o = causal_attention(q, k, v)
            x = x + o @ w[p + "self_attn.o_proj.weight"].T
            h = rms_norm(x, w[p + "post_attention_layernorm.weight"], self.eps)
            x = x + swiglu_ffn(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                               w[p + "mlp.down_proj.weight"])
        return x

    def logits(self, tokens) -> torch.Tensor:
        """Logits at every position of one whole sequence, [n, V]
        (core/model.cpp:477-492, 647-673)."""
        x = rms_norm(self.hidden(tokens), self.w["model.norm.weight"], self.eps)
        head = self.w["model.embed_tokens.weight"] if self.tied else self.w["lm_head.weight"]
        return lm_head(x, head)


# ----------------------------------------------------------------------------------------
# sampling
# ----------------------------------------------------------------------------------------

_MASK64 = (1 << 64) - 1


def uniform_from_counter(seed: int, counter: int) -> float:
    """One uniform in [0, 1) per (sequence seed, draw number): the splitmix64 finaliser of
    seed + (counter+1) * 0x9E3779B97F4A7C15, top 24 bits.  The reference draws from
    std::mt19937 seeded by the clock (core/engine.cpp:109-111), which cannot be replayed;
    this counter form is the library's own definition."""
    z = (seed + (counter + 1) * 0x9E3779B97F4A7C15) & _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


def greedy(logits: torch.Tensor) -> int:
    """First maximum (strict >)  (core/ops.cpp:490-497)."""
    best, val = 0, logits[0].item()
    for i in range(1, logits.numel()):
        if logits[i].item() > val:
            best, val = i, logits[i].item()
    return best


def repeat_penalty(logits: torch.Tensor, history: list[int], penalty: float,
                   last_n: int) -> torch.Tensor:
    """For each of the last `last_n` recorded tokens, in order (a token recorded twice is
    penalised twice): positive logit divided by the penalty, else multiplied
    (core/sampler.cpp:15-27)."""
    out = logits.clone()
    if penalty <= 1.0 or not history:
        return out
    for tok in history[-last_n:]:
        if 0 <= tok < out.numel():
            out[tok] = out[tok] / penalty if out[tok] > 0 else out[tok] * penalty
    return out


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, u: float,
           history: list[int] | None = None, penalty: float = 1.0, last_n: int = 64) -> int:
    """Repeat penalty -> logits/T (skipped for T <= 0 and T == 1) -> T <= 0: first max ->
    softmax -> the top_k most probable (0 = all), ties by lower index -> cut where the
    running sum reaches top_p -> r = u * kept mass; walk the kept tokens in index order
    and return the first whose running sum exceeds r  (core/sampler.cpp:35-39, 48-97).

    The reference walks them in order of probability; the distribution is the same, and
    index order makes the draw independent of how ties are sorted."""
    x = repeat_penalty(logits.to(torch.float64), history or [], penalty, last_n)
    if temperature <= 0.0:
        return greedy(x)
    if temperature != 1.0:
        x = x * (1.0 / temperature)
    p = softmax_rows(x)
    V = p.numel()
    order = sorted(range(V), key=lambda i: (-p[i].item(), i))
    k = min(top_k, V) if top_k > 0 else V
    kept = order[:k]
    cum, cut = 0.0, k
    for j, i in enumerate(kept):
        cum += p[i].item()
        if cum >= top_p:
            cut = j + 1
            break
    kept = sorted(kept[:cut])
    total = sum(p[i].item() for i in kept)
    r = u * total
    run = 0.0
    for i in kept:
        run += p[i].item()
        if run > r:
            return i
    return kept[-1]


def generate(model: PlainLlama, prompt: list[int], max_new_tokens: int, temperature: float = 0.0,
             top_k: int = 0, top_p: float = 1.0, seed: int = 0, stop_ids=(),
             penalty: float = 1.0, last_n: int = 64) -> list[int]:
    """Whole-sequence generation: every step runs the full sequence again.  The loop is
    the reference's (core/engine.cpp:136-148): sample, stop on a stop id without emitting
    it, else append.  The prompt without its last token, then every sampled token, is the
    history of the repeat penalty (core/engine.cpp:118-122, core/sampler.cpp:95)."""
    seq = list(prompt)
    out: list[int] = []
    for step in range(max_new_tokens):
        lg = model.logits(seq)[-1]
        tok = sample(lg, temperature, top_k, top_p, uniform_from_counter(seed, step),
                     history=list(prompt[:-1]) + out, penalty=penalty, last_n=last_n)
        if tok in stop_ids:
            break
        out.append(tok)
        seq.append(tok)
    return out
