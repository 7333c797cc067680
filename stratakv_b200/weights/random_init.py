"""Random weights for a model description, and a model folder made from them.

The reference has no such mode; its tests build identity and zero models by
hand (``tests/phase6_smoke.cpp:149-180``).  Matrices and the embedding are
N(0, std), norm weights are 1 + N(0, std), drawn in float32 from a generator
seeded by ``(seed, tensor name)`` so that a tensor's values do not depend on
which other tensors exist, then cast to the stored dtype.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Dict, Mapping

import torch

from ..parts.base import TensorRequest
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, request: TensorRequest, seed: int, std: float,
                  dtype: torch.dtype, device="cpu") -> torch.Tensor:
    generator = torch.Generator(device=device)
    generator.manual_seed(_tensor_seed(seed, name))
    values = torch.randn(request.shape, generator=generator, dtype=torch.float32, device=device) * std
    if request.init == "around_one":
        values += 1.0
    elif request.init != "normal":
        raise ValueError(f"unknown init '{request.init}' for tensor {name}")
    return values.to(dtype)


def random_tensors(expected: Mapping[str, TensorRequest], seed: int, std: float = 0.02,
                   dtype: torch.dtype = torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    return {name: random_tensor(name, request, seed, std, dtype, device)
            for name, request in expected.items()}


def write_random_model(folder, config, seed: int, dtype: torch.dtype = torch.bfloat16,
                       std: float = 0.02) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a typed
    configuration of a registered architecture) with random weights."""
    from ..config.registry import resolve_architecture
    from ..engine.model import expected_tensors

    arch = resolve_architecture(config.architecture)
    spec = arch.build_spec(config)
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    raw = config.to_dict()
    raw["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32",
                          torch.float16: "float16"}[dtype]
    (folder / "config.json").write_text(json.dumps(raw, indent=2) + "\n")
    tensors = random_tensors(expected_tensors(spec), seed, std, dtype)
    write_safetensors(folder / "model.safetensors", tensors, metadata={"format": "pt"})
    return folder


def main(argv=None) -> int:
    """``python -m stratakv_b200.weights.random_init CONFIG.json OUT_DIR [--seed S] [--dtype bfloat16|float32]``:
    write a model folder (config.json, model.safetensors) with random weights for a configuration."""
    import argparse
    from ..config import load_config
    parser = argparse.ArgumentParser(prog="stratakv_b200.weights.random_init", description=main.__doc__)
    parser.add_argument("config", help="a config.json (or a folder that holds one)")
    parser.add_argument("out", help="folder to write")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "float16"])
    args = parser.parse_args(argv)
    _, config = load_config(args.config)
    folder = write_random_model(args.out, config, args.seed, getattr(torch, args.dtype))
    print(folder)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
