"""Arrangements: how a layer's norms, mixer and feed-forward are strung together.

``pre_norm`` is the Llama block, ``x += mixer(norm(x)); x += ffn(norm(x))``
(``src/models/transformer_block.cpp:301-331``).  Another arrangement is one more
function registered under its name.
"""
from __future__ import annotations

from .registry import part_class, register_arrangement


class Layer:
    """The built parts of one ``LayerSpec``."""
    # the norm that reads the stream first, and the part it feeds (for the layer or embedding before)
    first_norm = property(lambda self: foldable(self.mixer_norm, self.mixer))

    def __init__(self, spec, runtime):
        self.spec = spec
        self.mixer_norm = part_class("norm", spec.mixer_norm.kind)(spec.mixer_norm, runtime)
        self.mixer = part_class("mixer", spec.mixer.kind)(spec.mixer, runtime)
        self.ffn_norm = part_class("norm", spec.ffn_norm.kind)(spec.ffn_norm, runtime)
        self.ffn = part_class("ffn", spec.ffn.kind)(spec.ffn, runtime)
        self.run = part_class("arrangement", spec.arrangement)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    def forward(self, step, x, entry):
        self.run(self, step, x, entry)


def _normed(norm, consumer, step, x):
    stats = step.residual_stats
    if stats is not None and norm.folds_norm and consumer.folds_norm:
        return norm.forward(x, stats=stats)
    return norm.forward(x)


def foldable(norm, consumer):
    """The norm, if it can be folded into its consumer's first projection, else None."""
    return norm if norm is not None and norm.folds_norm and consumer.folds_norm else None


def pre_norm(layer: Layer, step, x, entry) -> None:
    stats = step.residual_stats
    h = _normed(layer.mixer_norm, layer.mixer, step, x)
    if stats is not None:
        stats.expect(foldable(layer.ffn_norm, layer.ffn))
    layer.mixer.forward(step, h, x, entry.cache, entry.writes_cache)
    if stats is not None and not layer.mixer.folds_norm:
        stats.invalidate()
    h = _normed(layer.ffn_norm, layer.ffn, step, x)
    if stats is not None:
        stats.expect(step.norm_after_layer)
    layer.ffn.forward(step, h, x)
    if stats is not None and not layer.ffn.folds_norm:
        stats.invalidate()


register_arrangement("pre_norm", pre_norm)
