"""Binding a model's weights by tensor name, with one error for everything that is wrong.

The model declares the tensors it reads (`DecoderModel.tensors()`: name, shape); a source
offers tensors by name (a model folder, `ModelFiles`, or seeded random weights,
`RandomSource`).  `load_weights` first compares the two completely and raises a single
`WeightError` listing missing tensors, unexpected tensors and wrong shapes; only then are
tensors copied to the device, each kept in the precision it is stored in (16-bit floats
as bfloat16, 32-bit floats as float32, integer tables as int32).

The reference binds by name through `GGUFParser::tensor_info / tensor_raw`
(core/gguf_parser.cpp:396-410) and silently skips a missing norm tensor
(core/model.cpp:317-320); here a missing tensor is an error.
"""
from __future__ import annotations

import torch

from .safetensors_io import WeightError, kept_dtype


def check_tensors(available: dict, decls, ignored_suffixes=()) -> None:
    """available: name -> (dtype, shape).  Raises WeightError naming every problem."""
    wanted = {d.name: tuple(d.shape) for d in decls}
    missing = sorted(n for n in wanted if n not in available)
    unexpected = sorted(n for n in available if n not in wanted
                        and not any(n.endswith(s) for s in ignored_suffixes))
    wrong = []
    for n, shape in sorted(wanted.items()):
        if n in available:
            dt, have = available[n]
            if tuple(have) != shape:
                wrong.append(f"{n}: file has {list(have)}, model needs {list(shape)}")
            elif not (dt.is_floating_point):
                wrong.append(f"{n}: stored as {dt}, a floating-point tensor is needed")
    if missing or unexpected or wrong:
        parts = []
        if missing:
            parts.append(f"{len(missing)} missing: " + ", ".join(missing))
        if unexpected:
            parts.append(f"{len(unexpected)} unexpected: " + ", ".join(unexpected))
        if wrong:
            parts.append(f"{len(wrong)} wrong shape or type: " + "; ".join(wrong))
        raise WeightError("weights do not match the model: " + " | ".join(parts))


def load_weights(model, source, ignored_suffixes=None) -> None:
    """Checks `source` against `model.tensors()`, then hands every part its tensors."""
    decls = model.tensors()
    if ignored_suffixes is None:
        ignored_suffixes = getattr(model.spec, "ignored_tensors", ())
    available = {}
    for n in source.names():
        info = source.info(n)
        available[n] = (info.dtype, tuple(info.shape))
    check_tensors(available, decls, ignored_suffixes)
    device = model.rt.device

    def get(name: str) -> torch.Tensor:
        t = source.read(name)
        keep = kept_dtype(t.dtype)
        if t.device != device:
            t = t.to(device, non_blocking=False)
        return t if t.dtype == keep else t.to(keep)

    model.load(get)
