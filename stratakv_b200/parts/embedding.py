"""The two ends of a model as parts: token embedding and output head.

``TokenEmbedding``: row ``ids[t]`` of the table becomes row ``t`` of the float32
residual stream (``src/generation/generator.cpp:520-529``).  ``LinearHead``:
``logits = y . W^T`` on the rows that the final norm was asked for, in float32
(``src/generation/generator.cpp:773-774``); its weight may be the embedding
table (tied), in which case both parts share one copy on the device.

Both are looked up by their spec's ``kind`` like every other part, so an
embedding with a scale factor or a head that caps its logits is another class
registered under another kind; the model only calls ``forward``.
"""
from __future__ import annotations

import torch

from .. import ops as _ops
from .base import Part, TensorRequest
from .registry import register_embedding, register_head


class TokenEmbedding(Part):
    role = "embedding"
    graph_safe = True

    @classmethod
    def expected_tensors(cls, spec):
        return {spec.weight: TensorRequest((spec.vocab_size, spec.hidden_size))}

    def bind(self, tensors):
        self.table = self.rt.upload_shared(self.spec.weight, tensors[self.spec.weight])

    def forward(self, step, x, flags, stats=None) -> None:
        """Fill the stream ``x`` [tokens, hidden] for ``step.token_ids``; an id outside the table raises
        bit 0 of ``flags``.  ``stats``: see ``residual.ResidualStats`` (the kernel fills it where it can)."""
        self.rt.kernels().embed(self.table, step.token_ids, x, flags, stats=stats)


class LinearHead(Part):
    role = "head"
    graph_safe = True
    folds_norm = True

    @classmethod
    def expected_tensors(cls, spec):
        return {spec.weight: TensorRequest((spec.vocab_size, spec.hidden_size))}

    def bind(self, tensors):
        self.weight = self.rt.upload_shared(self.spec.weight, tensors[self.spec.weight])

    def forward(self, y, n_rows: int) -> torch.Tensor:
        """``y``: the normalised rows (or ``residual.NormedRows``); returns float32 ``[n_rows, vocab]``
        in scratch memory that the next step overwrites."""
        logits = self.rt.workspace.get("logits", (n_rows, self.spec.vocab_size), torch.float32)
        self.rt.kernels().linear(y, self.weight, logits, _ops.MODE_STORE_F32)
        return logits


register_embedding("embedding", TokenEmbedding)
register_head("linear_head", LinearHead)
