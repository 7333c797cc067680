"""Arrangements: how a layer's norms, mixer and feed-forward are strung together.

``pre_norm`` is the Llama block, ``x += mixer(norm(x)); x += ffn(norm(x))``
(``src/models/transformer_block.cpp:301-331``).  Another arrangement is one more
function registered under its name.
"""
from __future__ import annotations

from .registry import part_class, register_arrangement


class Layer:
    """The built parts of one ``LayerSpec``."""

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


def pre_norm(layer: Layer, step, x, entry) -> None:
    h = layer.mixer_norm.forward(x)
    layer.mixer.forward(step, h, x, entry.cache, entry.writes_cache)
    h = layer.ffn_norm.forward(x)
    layer.ffn.forward(step, h, x)


register_arrangement("pre_norm", pre_norm)
