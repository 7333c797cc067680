"""Descriptions of a model as data: parts, layers, their order, and the head.

An architecture turns its typed configuration into one ``ModelSpec``.  Every
size and constant a part needs is a field of that part's spec; no part reads
the model's configuration or knows which model it is in.  Layers may differ
from one another (each ``LayerSpec`` names its own mixer and feed-forward),
and the order in which layers run is a list of ``ScheduleEntry`` which may
name a layer twice or let a layer read the cache another run wrote.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """RMSNorm: ``y = x / sqrt(mean(x^2) + eps) * weight`` (``src/layers/rmsnorm.cpp:63-97``)."""
    size: int
    eps: float
    weight: str                      # tensor name
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding with split-half pairing (``src/layers/attention.cpp:96-135``)."""
    head_dim: int
    theta: float
    kind: str = "rope_half"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a paged cache (``src/layers/attention.cpp:153-342``)."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float                     # multiplies q.k after the dot product
    position: Optional[RopeSpec]
    q_weight: str
    k_weight: str
    v_weight: str
    o_weight: str
    window: int = 0                  # 0: every earlier key; w > 0: the last w keys only
    kind: str = "attention"


@dataclass(frozen=True)
class GatedMlpSpec:
    """``down(act(gate(x)) * up(x))`` (``src/models/transformer_block.cpp:312-325``)."""
    hidden_size: int
    intermediate_size: int
    activation: str                  # "silu"
    gate_weight: str
    up_weight: str
    down_weight: str
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class LayerSpec:
    """One block: which norm, mixer and feed-forward, and how they are arranged.

    ``pre_norm``: ``x += mixer(norm1(x)); x += ffn(norm2(x))``
    (``src/models/transformer_block.cpp:301-331``).

    The four named places are what that arrangement uses; another arrangement may leave
    some of them ``None`` (a block without a feed-forward, one norm for two branches) and
    may name further parts in ``extras`` as ``(name, role, spec)``, which the layer builds
    and hands to the arrangement as ``layer.extra[name]``.
    """
    mixer_norm: Any
    mixer: Any
    ffn_norm: Any = None
    ffn: Any = None
    arrangement: str = "pre_norm"
    extras: Tuple[Tuple[str, str, Any], ...] = ()

    def named_parts(self):
        """``(name, role, spec)`` of every part this layer has, in a fixed order."""
        places = (("mixer_norm", "norm", self.mixer_norm), ("mixer", "mixer", self.mixer),
                  ("ffn_norm", "norm", self.ffn_norm), ("ffn", "ffn", self.ffn))
        return tuple(place for place in places if place[2] is not None) + tuple(self.extras)


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``cache`` is the index of the cache entry the run's
    mixer uses; ``writes_cache`` false means it only reads what another run wrote."""
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class EmbeddingSpec:
    vocab_size: int
    hidden_size: int
    weight: str
    kind: str = "embedding"


@dataclass(frozen=True)
class HeadSpec:
    """Final norm on the wanted rows, then ``logits = y . W^T`` (``src/generation/generator.cpp:773-774``).
    ``weight`` may be the embedding table's name (tied)."""
    vocab_size: int
    hidden_size: int
    weight: str
    kind: str = "linear_head"


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: EmbeddingSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: Any
    head: HeadSpec
    stop_token_ids: Tuple[int, ...] = ()
    max_positions: int = 0
    # Tensor names a checkpoint may carry that the model does not use.
    ignorable: Tuple[str, ...] = ()

    def num_cache_entries(self) -> int:
        return 1 + max((e.cache for e in self.schedule), default=-1)
