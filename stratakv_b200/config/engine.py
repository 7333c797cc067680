"""Sizing of one engine instance: the cache, the batch, the compute dtype.

Counterpart of the cache and device fields of the reference's
``GeneratorConfig`` (``include/stratakv/generation/generator.h:10-27``), whose
values the reference CLI fixes at 1024 blocks of 16 tokens (``src/cli.cpp:
276-277``).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .llama import ConfigError

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ConfigError(f"compute dtype must be bfloat16 or float32, got {name}")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ConfigError(f"compute dtype must be bfloat16 or float32, got {name!r}") from None


@dataclass(frozen=True)
class EngineConfig:
    """``max_tokens``: most tokens live requests hold at once, each request's
    count rounded up to a whole number of blocks.  ``block_size`` tokens per
    cache block.  ``max_batch``: most sequences in one step (0: as many as the
    cache could hold at one block each).  ``max_context``: most positions one
    sequence may reach (prompt plus generated tokens); 0 takes the model's
    ``max_position_embeddings``, a positive value replaces it (the rotary
    encoding is defined at any position; what lies beyond the model's own limit
    is the caller's decision).  The reference's only such limit is its cache
    capacity (``src/generation/generator.cpp:628-632``)."""
    max_tokens: int
    dtype: torch.dtype = torch.bfloat16
    block_size: int = 64
    max_batch: int = 0
    device: str = "cuda:0"
    use_cuda_graphs: bool = True
    max_context: int = 0

    def __post_init__(self):
        if self.max_tokens <= 0:
            raise ConfigError("max_tokens must be positive")
        if self.block_size <= 0 or self.block_size % 16 != 0:
            raise ConfigError("block_size must be a positive multiple of 16")
        if self.max_batch < 0:
            raise ConfigError("max_batch must be non-negative")
        if self.max_context < 0:
            raise ConfigError("max_context must be non-negative")
        object.__setattr__(self, "dtype", parse_dtype(self.dtype))

    @property
    def num_blocks(self) -> int:
        return -(-self.max_tokens // self.block_size)

    @property
    def slots(self) -> int:
        return self.max_batch if self.max_batch else self.num_blocks
