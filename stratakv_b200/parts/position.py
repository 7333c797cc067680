"""Rotary position encoding with split-half pairs.

For pair ``i`` of a head: ``f_i = theta^(-2i/d)`` computed in double and stored
as float; ``angle = position * f_i`` in double; cos and sin in double, then
rounded to float; ``x[i], x[i+d/2] = x1*cos - x2*sin, x1*sin + x2*cos``
(``src/layers/attention.cpp:63-69, 96-135``).  The table of (cos, sin) is built
on the host with exactly those steps and grows when a longer position is asked
for; the kernel that applies it also writes keys and values into the cache.
"""
from __future__ import annotations

import numpy as np
import torch

from .registry import register_position


def rope_table(head_dim: int, theta: float, positions: int) -> np.ndarray:
    """``[positions, head_dim/2, 2]`` float32 of (cos, sin)."""
    half = head_dim // 2
    exponent = -2.0 * np.arange(half, dtype=np.float64) / float(head_dim)
    inv_freq = np.power(np.float64(theta), exponent).astype(np.float32)
    angle = np.arange(positions, dtype=np.float64)[:, None] * inv_freq.astype(np.float64)[None, :]
    return np.stack([np.cos(angle), np.sin(angle)], axis=-1).astype(np.float32)


class RopeHalf:
    role = "position"

    def __init__(self, spec, runtime):
        self.spec = spec
        self.rt = runtime
        self.table = None
        self.length = 0
        self._retired = []          # earlier tables stay alive: captured graphs may still read them

    def ensure(self, positions: int) -> None:
        """Make the table cover positions ``0 .. positions-1`` (never inside a graph capture)."""
        if positions <= self.length:
            return
        length = max(positions, 2 * self.length, 256)
        if self.table is not None:
            self._retired.append(self.table)
        host = torch.from_numpy(rope_table(self.spec.head_dim, self.spec.theta, length))
        self.table = host.to(self.rt.device).contiguous()
        self.length = length

    def fusion_table(self, max_positions: int):
        """The (cos, sin) table for kernels that rotate queries and keys themselves."""
        self.ensure(max_positions)
        return self.table

    def rotate_and_store(self, step, qkv, q_out, k_cache, v_cache, block_table, num_heads, num_kv_heads,
                         head_dim, block_size, write_kv):
        if head_dim != self.spec.head_dim:
            raise ValueError("rotary table was built for another head size")
        self.ensure(step.max_ctx)
        self.rt.kernels(head_dim).rope_kv_write(
            qkv, self.table, step.positions, step.token_seq, block_table, q_out, k_cache, v_cache,
            num_heads, num_kv_heads, head_dim, block_size, write_kv)


class NoPosition:
    """No position encoding: queries and keys pass unrotated into the cache."""
    role = "position"

    def __init__(self, spec, runtime):
        self.spec = spec
        self.rt = runtime

    def ensure(self, positions: int) -> None:
        pass

    def fusion_table(self, max_positions: int):
        return None

    def rotate_and_store(self, step, qkv, q_out, k_cache, v_cache, block_table, num_heads, num_kv_heads,
                         head_dim, block_size, write_kv):
        self.rt.kernels(head_dim).rope_kv_write(
            qkv, None, step.positions, step.token_seq, block_table, q_out, k_cache, v_cache,
            num_heads, num_kv_heads, head_dim, block_size, write_kv)


register_position("rope_half", RopeHalf)
register_position("none", NoPosition)
