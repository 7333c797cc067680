"""Bookkeeping that lets a norm be folded into the projections around it.

At decode the float residual stream is a few rows; an RMSNorm kernel of its own
costs a launch and a round trip through memory for almost no work.  RMSNorm is
``x * weight`` times one factor per row, ``1 / sqrt(mean(x^2) + eps)``, and a
factor per row commutes with the projection that follows.  So the kernel that
writes the stream (the embedding, a residual-add projection) also leaves, in a
``ResidualStats``, each row times the weight of the norm that reads the stream
next (in the compute dtype) and what gives the row's factor; that norm then
hands over ``NormedRows`` instead of running, and its consumer's first
projection multiplies its result by the factor.  With few rows the writer only
leaves partial sums of squares (one per block of the kernel) and the consumer
adds them up while it loads its weights; with more, that would be much traffic
for every block of the consumer, and the writer's last block makes the factor.  All of the norm's arithmetic stays in
float32 and the activations are rounded once, as with the separate kernel; only
the place of that rounding (before the factor instead of after it) differs.

Who does what: the model and the arrangement call ``expect(norm)`` before a part
that may write the stream, naming the norm that reads it next (None: nobody who
can use it).  The writing kernel's wrapper fills the buffers and calls
``filled()``, or ``invalidate()`` where it cannot.  A norm asks ``ready_for(self)``.
A norm that folds has ``gamma`` (float32 weight) and ``spec.eps``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

import torch

KERNEL_FOLD_ROWS = 64      # the small-step projection kernel folds norms for at most this many tokens
MAX_FUSED_ROWS = 16        # the engine asks for it up to here: larger steps run on the tensor-memory kernels, which do not fold
CONSUMER_SUMS_ROWS = 16    # up to here the consumer adds the partial sums up, beyond (up to 64 rows) the writer does
COLUMNS_PER_PARTIAL = 16   # a residual-add projection sums squares over 16 columns per block


class ResidualStats:
    """While ``prepared_for`` is not None: ``scaled[row]`` is the stream's row times
    ``prepared_for.gamma``, and that norm's factor for the row is ``row_scale[row]`` if
    ``n_partials`` is 0, else ``1 / sqrt(sum(partials[row, :n_partials]) / width + eps)``."""

    def __init__(self, scaled: torch.Tensor, row_scale: torch.Tensor, partials: torch.Tensor, counter: torch.Tensor):
        self.scaled = scaled
        self.row_scale = row_scale
        self.partials = partials       # [rows, >= width / 16]
        self.counter = counter         # one int32, zero between kernels
        self.n_partials = 0
        self.next_norm: Any = None
        self.prepared_for: Any = None

    @classmethod
    def allocate(cls, get, rows: int, width: int, dtype):
        """Buffers from ``get(name, shape, dtype, zero=False)`` (a workspace's)."""
        partial_width = (width + COLUMNS_PER_PARTIAL - 1) // COLUMNS_PER_PARTIAL
        partial_width = (partial_width + 3) // 4 * 4      # rows of whole 16 bytes: the consumer copies them so
        return cls(get("residual_scaled", (rows, width), dtype), get("residual_row_scale", (rows,), torch.float32),
                   get("residual_partials", (rows, partial_width), torch.float32),
                   get("residual_counter", (1,), torch.int32, zero=True))

    def expect(self, norm) -> None:
        self.next_norm = norm

    @property
    def consumer_sums(self) -> bool:
        # (the consumer stages rows x partial sums in shared memory beside its reduction area: 24 KB at most)
        rows, width = self.partials.shape
        return rows <= CONSUMER_SUMS_ROWS and rows * width <= 6144

    def filled(self, n_partials: int = 0) -> None:
        self.prepared_for = self.next_norm
        self.n_partials = n_partials

    def invalidate(self) -> None:
        self.prepared_for = None

    def ready_for(self, norm) -> bool:
        return norm is not None and self.prepared_for is norm


@dataclass
class NormedRows:
    """A norm not yet finished: ``scaled[rows]`` still lacks the factor per row, which the consuming
    projection applies to its result: ``row_scale[rows]``, or (``n_partials`` > 0) made from the
    rows' partial sums of squares and ``eps``."""
    scaled: torch.Tensor
    row_scale: torch.Tensor
    rows: Optional[torch.Tensor] = None
    partials: Optional[torch.Tensor] = None
    n_partials: int = 0
    eps: float = 0.0

    @property
    def shape(self):
        return (self.scaled.shape[0] if self.rows is None else self.rows.numel(), self.scaled.shape[1])
