"""Seeded random weights: a source of tensors by name, and a writer of model folders.

Values are a pure function of (seed, tensor name, element index): a splitmix64 hash gives
two 32-bit uniforms per element, Box-Muller (in double precision) turns them into a
normal deviate, and the result is rounded to the stored dtype.  The same numbers come out
on the CPU and on a GPU, so a folder written on one machine equals the tensors generated
directly on the device of another.  Matrices and embeddings are N(0, std); norm weights
are 1 + N(0, norm_std).

The reference has no random-weights mode (it always needs a model file; only
benchmark/micro_gemm.cpp:88-91 randomises activations).
"""
from __future__ import annotations

import hashlib
import json
import math
from dataclasses import dataclass
from pathlib import Path

import torch

from .safetensors_io import write_safetensors

_GOLDEN = -7046029254386353131          # 0x9E3779B97F4A7C15 as a signed 64-bit integer
_M1 = -4658895280553007687              # 0xBF58476D1CE4E5B9
_M2 = -7723592293110705685              # 0x94D049BB133111EB
_CHUNK = 1 << 24


def _lsr(z: torch.Tensor, n: int) -> torch.Tensor:
    """Logical shift right of int64 values."""
    return (z >> n) & ((1 << (64 - n)) - 1)


def _splitmix(z: torch.Tensor) -> torch.Tensor:
    z = (z ^ _lsr(z, 30)) * _M1
    z = (z ^ _lsr(z, 27)) * _M2
    return z ^ _lsr(z, 31)


def _key(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little", signed=True)


def normal_tensor(seed: int, name: str, shape, mean: float, std: float, dtype, device) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= int(s)
    out = torch.empty(n, dtype=dtype, device=device)
    key = _key(seed, name)
    for start in range(0, n, _CHUNK):
        stop = min(n, start + _CHUNK)
        idx = torch.arange(start, stop, dtype=torch.int64, device=device)
        z = _splitmix(idx * _GOLDEN + key)
        u1 = (_lsr(z, 32).to(torch.float64) + 1.0) * (1.0 / 4294967296.0)          # (0, 1]
        u2 = (z & 0xFFFFFFFF).to(torch.float64) * (1.0 / 4294967296.0)              # [0, 1)
        g = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos((2.0 * math.pi) * u2)
        out[start:stop] = (mean + std * g).to(dtype)
    return out.reshape(tuple(shape))


@dataclass(frozen=True)
class _Info:
    dtype: torch.dtype
    shape: tuple


class RandomSource:
    """Offers the tensors of `decls` (TensorDecl list) with seeded random values."""

    def __init__(self, decls, seed: int, dtype=torch.bfloat16, device="cpu", std: float = 0.02,
                 norm_std: float = 0.1):
        self.decls = {d.name: d for d in decls}
        self.seed, self.dtype, self.device = int(seed), dtype, torch.device(device)
        self.std, self.norm_std = float(std), float(norm_std)

    def names(self):
        return self.decls.keys()

    def info(self, name):
        return _Info(self.dtype, tuple(self.decls[name].shape))

    def read(self, name) -> torch.Tensor:
        d = self.decls[name]
        if d.init == "ones_normal":
            return normal_tensor(self.seed, name, d.shape, 1.0, self.norm_std, self.dtype, self.device)
        if d.init == "normal":
            return normal_tensor(self.seed, name, d.shape, 0.0, self.std, self.dtype, self.device)
        raise ValueError(f"{name}: unknown init {d.init!r}")


def write_model_folder(folder, config, seed: int, dtype=torch.bfloat16, std: float = 0.02,
                       norm_std: float = 0.1, device="cpu") -> Path:
    """Writes config.json and model.safetensors for `config` (a typed configuration of a
    registered architecture) with random weights from `seed`."""
    from ..config.base import get_architecture
    from ..engine.runtime import Runtime
    from ..parts.model import DecoderModel

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    arch = get_architecture(config.architecture)
    spec = arch.build_spec(config)
    # the parts are only asked for their tensor declarations here; nothing runs
    model = DecoderModel(spec, Runtime(dtype if dtype != torch.float16 else torch.bfloat16, torch.device("cpu")))
    src = RandomSource(model.tensors(), seed, dtype, device, std, norm_std)
    cfg = config.to_dict()
    cfg["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    (folder / "config.json").write_text(json.dumps(cfg, indent=2) + "\n")
    items = [(d.name, tuple(d.shape), dtype, (lambda n=d.name: src.read(n))) for d in model.tensors()]
    write_safetensors(folder / "model.safetensors", items, metadata={"format": "pt", "seed": seed})
    return folder
