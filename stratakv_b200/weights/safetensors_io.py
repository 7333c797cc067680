"""Reader and writer for the safetensors container, over a memory mapping.

File layout: an 8-byte little-endian header length, a JSON header that maps
tensor names to ``{"dtype", "shape", "data_offsets"}``, then the payload.  The
checks are the ones the reference's loader makes (``src/io/safetensors.cpp:
485-516, 525-608``): header length within the file and under 100 MiB, byte
range equal to element count times width, ranges inside the payload, no
overlap and no hole.  Unlike the reference, which widens every tensor to FP32
on the host (``src/io/safetensors.cpp:573-602``), tensors keep the dtype they
are stored in: a BF16 checkpoint is read as BF16 views of the mapping.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Mapping, Tuple

import torch

MAX_HEADER_BYTES = 100 * 1024 * 1024  # src/io/safetensors.cpp:536-539


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors container."""


_DTYPES = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "bfloat16": (torch.bfloat16, 2),  # alias the reference accepts, tests/phase7_smoke.cpp:57-62
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
          torch.float64: "F64", torch.int64: "I64", torch.int32: "I32",
          torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8", torch.bool: "BOOL"}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int  # byte offsets within the payload
    end: int


def _reject_duplicates(pairs):
    seen = {}
    for key, value in pairs:
        if key in seen:
            raise SafetensorsError(f"duplicate key in header: {key!r}")
        seen[key] = value
    return seen


class SafetensorsFile:
    """An open, memory-mapped safetensors file; tensors are views of the mapping."""

    def __init__(self, path):
        self.path = Path(path)
        try:
            self._handle = open(self.path, "rb")
        except OSError as error:
            raise SafetensorsError(f"{self.path}: cannot open ({error.strerror})") from None
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: file is shorter than the 8-byte header length")
        # ACCESS_COPY is a private copy-on-write mapping, as the reference's
        # MAP_PRIVATE (src/io/safetensors.cpp:164-203): writes never reach the file.
        self._map = mmap.mmap(self._handle.fileno(), 0, access=mmap.ACCESS_COPY)
        (header_len,) = struct.unpack("<Q", self._map[:8])
        if header_len > MAX_HEADER_BYTES:
            raise SafetensorsError(f"{self.path}: header length {header_len} exceeds {MAX_HEADER_BYTES}")
        if 8 + header_len > size:
            raise SafetensorsError(f"{self.path}: header length {header_len} runs past the end of the file")
        try:
            text = self._map[8:8 + header_len].decode("utf-8")
            header = json.loads(text, object_pairs_hook=_reject_duplicates)
        except UnicodeDecodeError:
            raise SafetensorsError(f"{self.path}: header is not valid UTF-8") from None
        except json.JSONDecodeError as error:
            raise SafetensorsError(f"{self.path}: header is not valid JSON ({error})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{self.path}: header must be a JSON object")
        self.payload_offset = 8 + header_len
        self.payload_size = size - self.payload_offset
        self.metadata = header.pop("__metadata__", None)
        if self.metadata is not None and not (
                isinstance(self.metadata, dict)
                and all(isinstance(v, str) for v in self.metadata.values())):
            raise SafetensorsError(f"{self.path}: __metadata__ must map strings to strings")
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            self.entries[name] = self._entry(name, info)
        self._check_coverage()

    def _entry(self, name, info) -> TensorEntry:
        where = f"{self.path}: tensor {name!r}"
        if not isinstance(info, dict):
            raise SafetensorsError(f"{where}: entry must be an object")
        unknown = set(info) - {"dtype", "shape", "data_offsets"}
        if unknown:
            raise SafetensorsError(f"{where}: unknown field(s) {sorted(unknown)}")
        for key in ("dtype", "shape", "data_offsets"):
            if key not in info:
                raise SafetensorsError(f"{where}: missing '{key}'")
        if info["dtype"] not in _DTYPES:
            raise SafetensorsError(f"{where}: unsupported dtype {info['dtype']!r}")
        dtype, width = _DTYPES[info["dtype"]]
        shape = info["shape"]
        if not isinstance(shape, list) or not all(
                isinstance(d, int) and not isinstance(d, bool) and d >= 0 for d in shape):
            raise SafetensorsError(f"{where}: shape must be a list of non-negative integers")
        offsets = info["data_offsets"]
        if (not isinstance(offsets, list) or len(offsets) != 2 or not all(
                isinstance(o, int) and not isinstance(o, bool) and o >= 0 for o in offsets)):
            raise SafetensorsError(f"{where}: data_offsets must be two non-negative integers")
        begin, end = offsets
        count = 1
        for d in shape:
            count *= d
        if end < begin or end - begin != count * width:
            raise SafetensorsError(
                f"{where}: byte range [{begin}, {end}) does not hold {count} elements of {width} bytes")
        if end > self.payload_size:
            raise SafetensorsError(f"{where}: byte range ends at {end}, payload has {self.payload_size} bytes")
        return TensorEntry(name, dtype, tuple(shape), begin, end)

    def _check_coverage(self) -> None:
        cursor = 0
        for entry in sorted(self.entries.values(), key=lambda e: (e.begin, e.end)):
            if entry.begin < cursor:
                raise SafetensorsError(f"{self.path}: tensor {entry.name!r} overlaps another tensor")
            if entry.begin > cursor:
                raise SafetensorsError(
                    f"{self.path}: payload bytes [{cursor}, {entry.begin}) belong to no tensor")
            cursor = entry.end
        if cursor != self.payload_size:
            raise SafetensorsError(
                f"{self.path}: payload bytes [{cursor}, {self.payload_size}) belong to no tensor")

    def names(self):
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        """A view of the mapping (no copy) with the stored dtype and shape."""
        entry = self.entries[name]
        count = 1
        for d in entry.shape:
            count *= d
        if count == 0:
            return torch.empty(entry.shape, dtype=entry.dtype)
        flat = torch.frombuffer(self._map, dtype=entry.dtype, count=count,
                                offset=self.payload_offset + entry.begin)
        return flat.reshape(entry.shape)

    def close(self) -> None:
        # Views handed out keep the mapping alive through the buffer protocol;
        # closing is best effort and only drops this object's references.
        try:
            self._map.close()
        except BufferError:
            pass
        self._handle.close()


def write_safetensors(path, tensors: Mapping[str, torch.Tensor], metadata=None) -> None:
    """Write ``tensors`` (CPU, any supported dtype) as one safetensors file."""
    header = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    cursor = 0
    order = list(tensors)
    for name in order:
        tensor = tensors[name]
        if tensor.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {tensor.dtype} cannot be stored")
        nbytes = tensor.numel() * tensor.element_size()
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [cursor, cursor + nbytes]}
        cursor += nbytes
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)  # keeps the payload 8-byte aligned
    # Written beside the target and renamed over it: a file that is mapped
    # somewhere (even by the tensors being written) is never truncated.
    path = Path(path)
    staged = path.with_name(path.name + f".tmp{os.getpid()}")
    with open(staged, "wb") as out:
        out.write(struct.pack("<Q", len(text)))
        out.write(text)
        for name in order:
            tensor = tensors[name].detach().cpu().contiguous()
            out.write(tensor.reshape(-1).view(torch.uint8).numpy().tobytes())
    os.replace(staged, path)
