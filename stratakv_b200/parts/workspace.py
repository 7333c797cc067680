"""Named scratch buffers that live across steps, so a step allocates nothing
once its sizes have been seen (the reference keeps eleven fixed workspaces per
layer for its one-token step, ``src/models/transformer_block.cpp:230-258``)."""
from __future__ import annotations

from typing import Dict, Tuple

import torch


class Workspace:
    def __init__(self, device):
        self.device = torch.device(device)
        self._buffers: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self.generation = 0          # bumped whenever a buffer is reallocated

    def get(self, name: str, shape, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """``zero``: the buffer is zero when it is first handed out (and after it had to grow)."""
        count = 1
        for d in shape:
            count *= int(d)
        key = (name, dtype)
        buffer = self._buffers.get(key)
        if buffer is None or buffer.numel() < count:
            capacity = max(count, 1)
            if buffer is not None:
                capacity = max(capacity, 2 * buffer.numel())
            buffer = (torch.zeros if zero else torch.empty)(capacity, dtype=dtype, device=self.device)
            self._buffers[key] = buffer
            self.generation += 1
        return buffer[:count].view(*shape)
