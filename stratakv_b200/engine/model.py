"""A model built from a ``ModelSpec``: embedding, layers in schedule order, final norm, head.

One forward pass of a step: gather embeddings into the float32 residual stream,
run every schedule entry's layer, then normalise only the rows whose logits are
wanted and multiply them with the head (the reference likewise computes the
final norm and the head on the last position only, ``src/generation/generator.cpp:
691-715``).
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from .. import ops as _ops
from ..parts.base import CacheRequest, Runtime, StepBatch, TensorRequest
from ..parts.block import Layer
from ..parts.registry import part_class
from ..parts.spec import ModelSpec
from ..residual import MAX_FUSED_ROWS, ResidualStats


def expected_tensors(spec: ModelSpec) -> Dict[str, TensorRequest]:
    """Every checkpoint tensor the model needs, by name, with its shape."""
    found: Dict[str, TensorRequest] = {}

    def add(requests: Mapping[str, TensorRequest]):
        for name, request in requests.items():
            if name in found and tuple(found[name].shape) != tuple(request.shape):
                raise ValueError(f"tensor {name} is requested with two shapes: "
                                 f"{found[name].shape} and {request.shape}")
            found.setdefault(name, request)

    add(part_class("embedding", spec.embedding.kind).expected_tensors(spec.embedding))
    for layer in spec.layers:
        for _, role, part_spec in layer.named_parts():
            add(part_class(role, part_spec.kind).expected_tensors(part_spec))
    add(part_class("norm", spec.final_norm.kind).expected_tensors(spec.final_norm))
    add(part_class("head", spec.head.kind).expected_tensors(spec.head))
    return found


def cache_requests(spec: ModelSpec) -> List[CacheRequest]:
    """What each cache entry must hold, from the mixer of the run that writes it."""
    requests: List[Optional[CacheRequest]] = [None] * spec.num_cache_entries()
    for entry in spec.schedule:
        if not (0 <= entry.layer < len(spec.layers)):
            raise ValueError(f"schedule names layer {entry.layer}; the model has {len(spec.layers)}")
        if entry.writes_cache:
            if requests[entry.cache] is not None:
                raise ValueError(f"cache entry {entry.cache} is written by two runs")
            mixer = spec.layers[entry.layer].mixer
            requests[entry.cache] = (part_class("mixer", mixer.kind).cache_request(mixer) if mixer is not None
                                     else CacheRequest())
    for index, request in enumerate(requests):
        if request is None:
            raise ValueError(f"cache entry {index} is read but no run writes it")
    return requests


def default_head_dim(spec: ModelSpec) -> int:
    for layer in spec.layers:
        head_dim = getattr(layer.mixer, "head_dim", None)
        if head_dim:
            return head_dim
    return 64       # no part needs a head size: any build of the library will do


class Model:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec = spec
        self.rt = runtime
        self.layers = [Layer(layer_spec, runtime) for layer_spec in spec.layers]
        self.final_norm = part_class("norm", spec.final_norm.kind)(spec.final_norm, runtime)
        self.embedding = part_class("embedding", spec.embedding.kind)(spec.embedding, runtime)
        self.head = part_class("head", spec.head.kind)(spec.head, runtime)
        # Raised by kernels: bit 0 = token id outside the vocabulary.
        self.flags = torch.zeros(1, dtype=torch.int32, device=runtime.device)

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.embedding.bind(tensors)
        self.head.bind(tensors)                            # the same device tensor when tied
        for layer in self.layers:
            for part in layer.parts():
                part.bind(tensors)
        self.final_norm.bind(tensors)

    def graph_safe(self) -> bool:
        return (all(part.graph_safe for layer in self.layers for part in layer.parts())
                and self.final_norm.graph_safe and self.embedding.graph_safe and self.head.graph_safe)

    def prepare_positions(self, max_positions: int) -> None:
        """Let position encodings build their tables up to ``max_positions`` (before a graph capture)."""
        for layer in self.layers:
            position = getattr(layer.mixer, "position", None)
            if position is not None:
                position.ensure(max_positions)

    def weight_bytes(self) -> int:
        """Bytes of weights one decode step reads (each matrix once; one embedding row per token is left out)."""
        seen, total = set(), 0
        tensors = []
        parts = [self.head, self.final_norm] + [part for layer in self.layers for part in layer.parts()]
        for part in parts:
            for value in vars(part).values():
                if isinstance(value, torch.Tensor):
                    tensors.append(value)
        for tensor in tensors:
            if tensor.data_ptr() not in seen:
                seen.add(tensor.data_ptr())
                total += tensor.numel() * tensor.element_size()
        return total

    def forward(self, step: StepBatch, want_rows: Optional[torch.Tensor], n_want: int):
        """Run the step's tokens; return float32 logits ``[n_want, vocab]`` (a view
        of scratch memory that the next step overwrites) or ``None``."""
        with _ops.stream_scope():
            return self._forward(step, want_rows, n_want)

    def _forward(self, step: StepBatch, want_rows: Optional[torch.Tensor], n_want: int):
        rt, spec = self.rt, self.spec
        x = rt.workspace.get("residual", (step.n_tokens, spec.hidden_size), torch.float32)
        stats = None
        if step.is_decode and rt.dtype == torch.bfloat16 and step.n_tokens <= MAX_FUSED_ROWS:
            # few rows: norms are folded into the projections after them (residual.py)
            stats = ResidualStats.allocate(rt.workspace.get, step.n_tokens, spec.hidden_size, rt.dtype)
        step.residual_stats = stats
        final = self.final_norm if self.final_norm.folds_norm and self.head.folds_norm else None
        readers = [self.layers[entry.layer].first_norm for entry in spec.schedule] + [final]
        if stats is not None:
            stats.expect(readers[0])
        self.embedding.forward(step, x, self.flags, stats=stats)
        for index, entry in enumerate(spec.schedule):
            step.norm_after_layer = readers[index + 1]
            self.layers[entry.layer].forward(step, x, entry)
        if n_want == 0:
            return None
        if stats is not None and final is not None:
            y = self.final_norm.forward(x, rows=want_rows, name="final_normed", stats=stats)
        else:
            y = self.final_norm.forward(x, rows=want_rows, name="final_normed")
        return self.head.forward(y, n_want)
