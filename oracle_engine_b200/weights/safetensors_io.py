"""Reading and writing safetensors files, by tensor name.

File layout: 8 bytes little-endian header length, a JSON header
{name: {"dtype", "shape", "data_offsets": [begin, end]}} (plus an optional
"__metadata__"), then the raw little-endian tensor bytes.  A model folder holds either one
`model.safetensors` or shards listed by `model.safetensors.index.json` ("weight_map").

Takes the place of the reference's GGUF container (core/gguf_parser.cpp:164-198,
307-324: header, tensor infos, data section) and of its mmap access
(core/platform.cpp:312-327); like the parser it refuses a file whose header or offsets do
not fit the file (core/gguf_parser.cpp:237-240, 296-300, 311-317).

Tensors come back in the precision the engine keeps them in: 16-bit floats as bfloat16,
32-bit floats as float32, integers as int32.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import torch


class WeightError(RuntimeError):
    """A model file that cannot be used; the message lists everything that is wrong."""


_DTYPES = {  # name -> (torch dtype as stored, bytes per element)
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "I32": (torch.int32, 4), "I64": (torch.int64, 8), "F64": (torch.float64, 8),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16", torch.int32: "I32",
          torch.int64: "I64", torch.float64: "F64"}


def kept_dtype(stored: torch.dtype) -> torch.dtype:
    """The dtype a stored tensor is kept in: bf16 for 16-bit floats, float32 for 32-bit
    (and 64-bit) floats, int32 for integer tables."""
    if stored in (torch.bfloat16, torch.float16):
        return torch.bfloat16
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.int32


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: torch.dtype          # as stored
    shape: tuple[int, ...]
    begin: int                  # absolute byte offsets in the file
    end: int
    file: Path


class SafetensorsFile:
    """One safetensors file, memory-mapped; tensors are read lazily by name."""

    def __init__(self, path):
        self.path = Path(path)
        if not self.path.is_file():
            raise WeightError(f"{self.path}: no such file")
        size = self.path.stat().st_size
        if size < 8:
            raise WeightError(f"{self.path}: truncated (no header length)")
        self._fh = open(self.path, "rb")
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_COPY)
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if hlen > size - 8:
            raise WeightError(f"{self.path}: truncated header ({hlen} bytes announced, file has {size - 8})")
        try:
            header = json.loads(bytes(self._mm[8:8 + hlen]))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise WeightError(f"{self.path}: header is not valid JSON ({e})") from None
        base = 8 + hlen
        self.metadata = header.pop("__metadata__", {}) if isinstance(header, dict) else {}
        self.infos: dict[str, TensorInfo] = {}
        problems = []
        for name, info in header.items():
            try:
                dt, width = _DTYPES[info["dtype"]]
                shape = tuple(int(s) for s in info["shape"])
                b, e = (int(v) for v in info["data_offsets"])
            except (KeyError, TypeError, ValueError):
                problems.append(f"{name}: malformed entry {info!r}")
                continue
            n = 1
            for s in shape:
                n *= s
            if e - b != n * width:
                problems.append(f"{name}: {e - b} bytes stored for shape {list(shape)} of {info['dtype']}")
            elif b < 0 or base + e > size:
                problems.append(f"{name}: data [{b}, {e}) lies outside the file (truncated?)")
            else:
                self.infos[name] = TensorInfo(name, dt, shape, base + b, base + e, self.path)
        if problems:
            raise WeightError(f"{self.path}: " + "; ".join(problems))

    def names(self):
        return self.infos.keys()

    def read(self, name: str) -> torch.Tensor:
        """The tensor as stored (a CPU tensor viewing the mapping; copy before closing)."""
        i = self.infos[name]
        n = 1
        for s in i.shape:
            n *= s
        if n == 0:
            return torch.empty(i.shape, dtype=i.dtype)
        return torch.frombuffer(self._mm, dtype=i.dtype, count=n, offset=i.begin).reshape(i.shape)

    def close(self):
        try:
            self._mm.close()
        except (BufferError, ValueError):
            pass                          # tensors still view the mapping; the OS unmaps at exit
        self._fh.close()


class ModelFiles:
    """All tensors of a model folder (one file or shards), by name."""

    def __init__(self, folder):
        self.folder = Path(folder)
        index = self.folder / "model.safetensors.index.json"
        single = self.folder / "model.safetensors"
        self.files: list[SafetensorsFile] = []
        self.where: dict[str, SafetensorsFile] = {}
        if index.is_file():
            try:
                weight_map = json.loads(index.read_text())["weight_map"]
            except (json.JSONDecodeError, KeyError) as e:
                raise WeightError(f"{index}: no usable weight_map ({e})") from None
            opened: dict[str, SafetensorsFile] = {}
            missing = []
            for name, fname in weight_map.items():
                if fname not in opened:
                    opened[fname] = SafetensorsFile(self.folder / fname)
                if name not in opened[fname].infos:
                    missing.append(f"{name} (index says {fname})")
                self.where[name] = opened[fname]
            if missing:
                raise WeightError(f"{index}: tensors not found in their shard: " + ", ".join(missing))
            self.files = list(opened.values())
        elif single.is_file():
            f = SafetensorsFile(single)
            self.files = [f]
            self.where = {n: f for n in f.names()}
        else:
            raise WeightError(f"{self.folder}: neither model.safetensors nor model.safetensors.index.json")

    def names(self):
        return self.where.keys()

    def info(self, name: str) -> TensorInfo:
        return self.where[name].infos[name]

    def read(self, name: str) -> torch.Tensor:
        return self.where[name].read(name)

    def close(self):
        for f in self.files:
            f.close()


def write_safetensors(path, tensors, metadata: dict | None = None) -> None:
    """Writes `tensors` (a dict name -> CPU/CUDA tensor, or an iterable of (name, shape,
    dtype, make) with `make()` returning the tensor) as one safetensors file, streaming
    tensor by tensor so that a large model never sits in host memory twice."""
    if isinstance(tensors, dict):
        items = [(n, tuple(t.shape), t.dtype, (lambda t=t: t)) for n, t in tensors.items()]
    else:
        items = list(tensors)
    header = {}
    offset = 0
    for name, shape, dtype, _ in items:
        if dtype not in _NAMES:
            raise WeightError(f"{name}: dtype {dtype} cannot be written")
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * _DTYPES[_NAMES[dtype]][1]
        header[name] = {"dtype": _NAMES[dtype], "shape": [int(s) for s in shape],
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name, shape, dtype, make in items:
            t = make().detach().to("cpu").contiguous()
            if tuple(t.shape) != tuple(shape) or t.dtype != dtype:
                raise WeightError(f"{name}: generator returned {tuple(t.shape)} {t.dtype}, "
                                  f"declared {tuple(shape)} {dtype}")
            fh.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
