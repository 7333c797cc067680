"""Binding checkpoint tensors to a model by tensor name.

The reference takes tensors out of its weight map one by one and stops at the
first problem: ``"Missing weight: <name>"``, ``"Wrong shape/storage: <name>"``,
and any tensor left over is ``"Unexpected weight: <name>"``
(``src/generation/generator.cpp:265-289, 507-508``).  Here all problems of a
checkpoint are collected into one ``WeightError`` that lists missing tensors,
unexpected tensors, wrong shapes and tensors that hold a NaN or an infinity
(``"Non-finite weight: <name>"``, ``src/generation/generator.cpp:274-285``) together.

Tensors keep their stored dtype on the host: bfloat16 stays bfloat16, a tensor
stored in 32 bits stays 32-bit, integer tables become int32.  Parts choose the
device dtype when they upload (``Runtime.upload``).
"""
from __future__ import annotations

import fnmatch
import json
from pathlib import Path
from typing import Dict, Iterable, Mapping, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile

_INTEGER = (torch.int64, torch.int16, torch.int8, torch.uint8, torch.bool)


class WeightError(ValueError):
    """The checkpoint does not fit the model.  ``missing``, ``unexpected``,
    ``wrong_shape`` (name -> (expected, found)) and ``non_finite`` (names of
    tensors with a NaN or an infinity in them) hold the details."""

    def __init__(self, source, missing, unexpected, wrong_shape, wrong_dtype=(), non_finite=()):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = dict(wrong_shape)
        self.wrong_dtype = dict(wrong_dtype)
        self.non_finite = sorted(non_finite)
        lines = [f"checkpoint {source} does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} expected {list(e)} found {list(f)}" for n, (e, f) in sorted(self.wrong_shape.items())))
        if self.wrong_dtype:
            lines.append(f"  unusable dtypes ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n} is {d}" for n, d in sorted(self.wrong_dtype.items())))
        if self.non_finite:
            lines.append(f"  non-finite weights ({len(self.non_finite)}): " + ", ".join(self.non_finite))
        super().__init__("\n".join(lines))


def checkpoint_files(model_dir) -> Sequence[Path]:
    """``model.safetensors``, or the shards ``model.safetensors.index.json`` names."""
    model_dir = Path(model_dir)
    if model_dir.is_file():
        return [model_dir]
    single = model_dir / "model.safetensors"
    if single.is_file():
        return [single]
    index = model_dir / "model.safetensors.index.json"
    if index.is_file():
        weight_map = json.loads(index.read_text()).get("weight_map", {})
        return [model_dir / name for name in sorted(set(weight_map.values()))]
    raise SafetensorsError(f"no model.safetensors (or index) in {model_dir}")


def read_checkpoint(model_dir) -> Dict[str, torch.Tensor]:
    """Every tensor of the checkpoint as a host view with its stored dtype."""
    tensors: Dict[str, torch.Tensor] = {}
    for path in checkpoint_files(model_dir):
        handle = SafetensorsFile(path)
        for name in handle.names():
            if name in tensors:
                raise SafetensorsError(f"tensor {name!r} appears in more than one shard")
            tensors[name] = handle.tensor(name)
    return tensors


def check_and_select(source, tensors: Mapping[str, torch.Tensor],
                     expected: Mapping[str, Tuple[int, ...]],
                     ignorable: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """Return the expected tensors, or raise one ``WeightError`` listing every mismatch."""
    ignorable = tuple(ignorable)
    missing = [n for n in expected if n not in tensors]
    unexpected = [n for n in tensors if n not in expected
                  and not any(fnmatch.fnmatchcase(n, pattern) for pattern in ignorable)]
    wrong_shape = {n: (tuple(expected[n]), tuple(tensors[n].shape)) for n in expected
                   if n in tensors and tuple(tensors[n].shape) != tuple(expected[n])}
    wrong_dtype = {}
    non_finite = []
    selected = {}
    for name in expected:
        if name not in tensors or name in wrong_shape:
            continue
        tensor = tensors[name]
        if tensor.dtype in _INTEGER:
            tensor = tensor.to(torch.int32)
        elif tensor.dtype == torch.float64:
            wrong_dtype[name] = "F64"
            continue
        elif not bool(torch.isfinite(tensor).all()):
            non_finite.append(name)
            continue
        selected[name] = tensor
    if missing or unexpected or wrong_shape or wrong_dtype or non_finite:
        raise WeightError(source, missing, unexpected, wrong_shape, wrong_dtype, non_finite)
    return selected


def load_checkpoint(model_dir, expected: Mapping[str, Tuple[int, ...]],
                    ignorable: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    return check_and_select(str(model_dir), read_checkpoint(model_dir), expected, ignorable)
