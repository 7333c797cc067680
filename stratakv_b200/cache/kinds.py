"""Kinds of cache storage, by name.

A mixer asks for cache through a ``CacheRequest`` whose ``kind`` names one of
these.  A kind says whether it keeps blocks of positions at all, whether old
blocks may be given back once a window has passed them, and which tensors one
block holds for one cache entry.  ``KVCache`` allocates what the kind says and
knows nothing of keys or values itself; a mixer that caches something else (a
compressed latent per position, keys and values of unequal widths) registers a
kind of its own beside these and finds its tensors by name.

The reference has one kind only: per layer, keys and values of equal width in
token-major blocks (``include/stratakv/layers/attention.h:88-91``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Tuple

Shapes = Dict[str, Tuple[int, ...]]


@dataclass(frozen=True)
class CacheKind:
    """``block_tensors(request, block_size)`` returns, by tensor name, the shape of ONE block of ONE cache
    entry; the cache puts ``[entries, blocks + 1]`` in front.  ``paged`` false: nothing is kept per
    position (fixed-size state only).  ``windowed``: blocks behind ``request.window`` are given back."""
    name: str
    paged: bool
    windowed: bool
    block_tensors: Callable[..., Shapes]


_KINDS: Dict[str, CacheKind] = {}


def register_cache_kind(kind: CacheKind) -> None:
    _KINDS[kind.name] = kind


def cache_kind(name: str) -> CacheKind:
    try:
        return _KINDS[name]
    except KeyError:
        raise ValueError(f"unknown cache kind '{name}'; known: {sorted(_KINDS)}") from None


def _keys_and_values(request, block_size: int) -> Shapes:
    """Head-major blocks: one KV head's share of a block is a contiguous ``block_size x width`` tile.
    Values may be narrower or wider than keys (``v_head_dim``); 0 means the same width."""
    value_dim = request.v_head_dim or request.head_dim
    return {"k": (request.num_kv_heads, block_size, request.head_dim),
            "v": (request.num_kv_heads, block_size, value_dim)}


register_cache_kind(CacheKind("kv", paged=True, windowed=False, block_tensors=_keys_and_values))
register_cache_kind(CacheKind("kv_window", paged=True, windowed=True, block_tensors=_keys_and_values))
register_cache_kind(CacheKind("none", paged=False, windowed=False, block_tensors=lambda request, block_size: {}))
