"""RMSNorm part: ``y = x * (1 / sqrt(mean(x^2) + eps)) * weight``
(``src/layers/rmsnorm.cpp:63-97``; eps is the spec's, where the reference's
generator always uses the class default ``1e-5``, ``include/stratakv/layers/rmsnorm.h:13-16``).
The weight is kept in float32 whatever the compute dtype, as the reference does
(``src/layers/rmsnorm.cpp:44-61``)."""
from __future__ import annotations

import torch

from .base import Norm, TensorRequest
from .registry import register_norm
from ..residual import NormedRows


class RMSNorm(Norm):
    graph_safe = True
    folds_norm = True

    @classmethod
    def expected_tensors(cls, spec):
        return {spec.weight: TensorRequest((spec.size,), "around_one")}

    def bind(self, tensors):
        self.gamma = self.rt.upload(tensors[self.spec.weight], torch.float32)

    def forward(self, x, rows=None, out=None, name="normed", stats=None):
        """``stats`` prepared for this norm: leave the rest of the work to the consumer's projection."""
        if stats is not None and out is None and stats.ready_for(self):
            return NormedRows(stats.scaled, stats.row_scale, rows, stats.partials, stats.n_partials, self.spec.eps)
        n_rows = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = self.rt.workspace.get(name, (n_rows, self.spec.size), self.rt.dtype)
        self.rt.kernels().rmsnorm(x, self.gamma, self.spec.eps, out, rows)
        return out


register_norm("rmsnorm", RMSNorm)
