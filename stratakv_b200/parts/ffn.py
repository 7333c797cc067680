"""Gated feed-forward: ``x += down(act(gate(h)) * up(h))``, no bias, dense
(``src/models/transformer_block.cpp:312-329``).

Gate and up rows are packed into one matrix in tiles of 16 rows (8 gate rows,
then the 8 up rows that go with them), which lets the projection's epilogue
apply the activation and the product before anything is written; the residual
sum is the epilogue of the down projection.
"""
from __future__ import annotations

import torch

from .. import ops as _ops
from .base import FeedForward, TensorRequest
from .registry import register_ffn


def pack_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``[F, H]`` gate and up -> ``[2F', H]`` with rows (gate 8t..8t+7, up 8t..8t+7) per tile ``t``.
    ``F'`` is ``F`` rounded up to a multiple of 8; the added rows are zero (they produce
    ``act(0) * 0 = 0`` and meet zero columns of the down projection)."""
    rows, cols = gate.shape
    if rows % 8 != 0:
        pad = 8 - rows % 8
        gate = torch.cat([gate, gate.new_zeros(pad, cols)])
        up = torch.cat([up, up.new_zeros(pad, cols)])
        rows += pad
    tiles = torch.stack([gate.view(rows // 8, 8, cols), up.view(rows // 8, 8, cols)], dim=1)
    return tiles.reshape(2 * rows, cols).contiguous()


class GatedMlp(FeedForward):
    graph_safe = True
    folds_norm = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.activation not in _ops.ACTIVATIONS:
            raise ValueError(f"gated feed-forward: activation '{spec.activation}' is not supported")
        if runtime.dtype == torch.bfloat16 and spec.hidden_size % 8 != 0:
            raise ValueError(f"gated feed-forward: hidden size {spec.hidden_size} is not supported in bfloat16 "
                             "(rows of 16 bytes are needed: a multiple of 8); float32 takes any size")
        self.padded = -(-spec.intermediate_size // 8) * 8      # the kernels' tiles hold 8 gate and 8 up rows

    @classmethod
    def expected_tensors(cls, spec):
        return {spec.gate_weight: TensorRequest((spec.intermediate_size, spec.hidden_size)),
                spec.up_weight: TensorRequest((spec.intermediate_size, spec.hidden_size)),
                spec.down_weight: TensorRequest((spec.hidden_size, spec.intermediate_size))}

    def bind(self, tensors):
        s = self.spec
        gate = self.rt.upload(tensors[s.gate_weight])
        up = self.rt.upload(tensors[s.up_weight])
        self.w_gate_up = pack_gate_up(gate, up)
        del gate, up
        down = self.rt.upload(tensors[s.down_weight])
        if self.padded != s.intermediate_size:
            down = torch.cat([down, down.new_zeros(down.shape[0], self.padded - s.intermediate_size)], dim=1)
        self.w_down = down.contiguous()

    def forward(self, step, h, x):
        s, rt = self.spec, self.rt
        ops = rt.kernels()
        z = rt.workspace.get("ffn_hidden", (h.shape[0], self.padded), rt.dtype)
        ops.linear(h, self.w_gate_up, z, _ops.MODE_GATED, s.activation)
        ops.linear(z, self.w_down, x, _ops.MODE_ADD_F32, stats=getattr(step, "residual_stats", None))


register_ffn("gated_mlp", GatedMlp)
