"""Registries of part kinds: a spec's ``kind`` string chooses the class that runs it.

A new mixer, feed-forward, norm, position encoding, embedding or output head is added by registering
its class under a new kind; the model builder, the cache and the step function
only see the interfaces in ``parts/base.py``.
"""
from __future__ import annotations

from typing import Dict

_KINDS: Dict[str, Dict[str, type]] = {"mixer": {}, "ffn": {}, "norm": {}, "position": {},
                                      "arrangement": {}, "embedding": {}, "head": {}}


def register_part(role: str, kind: str, cls) -> None:
    if role not in _KINDS:
        raise KeyError(f"unknown part role '{role}'; roles: {sorted(_KINDS)}")
    _KINDS[role][kind] = cls


def register_mixer(kind, cls): register_part("mixer", kind, cls)
def register_ffn(kind, cls): register_part("ffn", kind, cls)
def register_norm(kind, cls): register_part("norm", kind, cls)
def register_position(kind, cls): register_part("position", kind, cls)
def register_arrangement(kind, fn): register_part("arrangement", kind, fn)
def register_embedding(kind, cls): register_part("embedding", kind, cls)
def register_head(kind, cls): register_part("head", kind, cls)


def part_class(role: str, kind: str):
    try:
        return _KINDS[role][kind]
    except KeyError:
        raise KeyError(f"no {role} registered under kind '{kind}'; "
                       f"known: {sorted(_KINDS.get(role, {}))}") from None
