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
        self.mixer_norm = self.mixer = self.ffn_norm = self.ffn = None
        self.extra = {}
        self._parts = []
        named = {"mixer_norm", "mixer", "ffn_norm", "ffn"}
        for name, role, part_spec in spec.named_parts():
            part = part_class(role, part_spec.kind)(part_spec, runtime)
            if name in named:
                setattr(self, name, part)
            else:
                self.extra[name] = part
            self._parts.append(part)
        self.run = part_class("arrangement", spec.arrangement)

    def parts(self):
        return tuple(self._parts)

    def forward(self, step, x, entry):
        self.run(self, step, x, entry)


def _normed(norm, consumer, step, x):
    stats = step.residual_stats
    if stats is not None and norm.folds_norm and consumer.folds_norm:
        return norm.forward(x, stats=stats)
    return norm.forward(x)


def foldable(norm, consumer):
    """The norm, if it can be folded into its consumer's first projection, else None."""
    return norm if norm is not None and consumer is not None and norm.folds_norm and consumer.folds_norm else None


def pre_norm(layer: Layer, step, x, entry) -> None:
    if layer.mixer_norm is None or layer.mixer is None or layer.ffn_norm is None or layer.ffn is None:
        raise ValueError("the pre_norm arrangement needs a norm and a mixer, and a norm and a feed-forward")
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
