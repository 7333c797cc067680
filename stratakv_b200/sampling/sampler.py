"""Choosing the next token: greedy, temperature, top-k, top-p, seeded draws.

Names and meanings are the reference's ``SamplerConfig``
(``include/stratakv/generation/sampler.h:8-17``, ``src/generation/sampler.cpp:
12-22, 43-148``): ``temperature == 0`` is greedy argmax (lowest index among
equals); ``top_k == 0`` disables top-k and ``top_k >= vocab`` keeps everything;
``top_p`` lies in (0, 1] and 1 disables it; the token that crosses ``top_p`` is
kept.  The reference draws with ``std::mt19937`` seeded from ``random_device``;
here every draw is Philox4x32-10 of ``(seed, stream, position)``: a request's
tokens depend on its own stream and how many tokens it has drawn, not on what
else is in the batch.  The choice is made on the device; only token ids come
back to the host.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Optional

import torch


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0

    def __post_init__(self):
        if not math.isfinite(self.temperature) or self.temperature < 0.0:
            raise ValueError("sampler: temperature must be finite and nonnegative")
        if self.top_k < 0:
            raise ValueError("sampler: top_k must be nonnegative")
        if not math.isfinite(self.top_p) or self.top_p <= 0.0 or self.top_p > 1.0:
            raise ValueError("sampler: top_p must be in (0, 1]")
        if not (0 <= self.seed < 2 ** 64):
            raise ValueError("sampler: seed must fit in 64 bits")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0


class Sampler:
    """Runs the sampling kernels for one engine."""

    def __init__(self, kernels, params: SamplingParams, flags: Optional[torch.Tensor] = None):
        self.kernels = kernels
        self.params = params
        self.flags = flags

    def sample(self, logits: torch.Tensor, streams: torch.Tensor, counters: torch.Tensor,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One token id per row of ``logits`` (int32, on the device).  ``streams``
        and ``counters`` (int32 per row) select each row's random number."""
        rows = logits.shape[0]
        if out is None:
            out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        if self.params.greedy:
            self.kernels.argmax(logits, out, self.flags)
        else:
            self.kernels.sample(logits, out, self.params.temperature, self.params.top_k, self.params.top_p,
                                self.params.seed, streams, counters, self.flags)
        return out
