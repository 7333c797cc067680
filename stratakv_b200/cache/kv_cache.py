"""The cache: a slot per sequence, keys and values per cache entry, per-sequence state.

Layout.  Cache entries (one per run of a layer that writes keys) whose mixers
ask for the same thing form a *group*; each group has storage and a block
allocator of its own, so layers that keep every key and layers that keep a
window do not share blocks.  A group's keys are one tensor
``[entries, blocks, kv_heads, block_size, head_dim]`` (values likewise): one KV
head's share of a block is a contiguous ``block_size x head_dim`` tile.  A block
id addresses the same block in every entry of its group; the reference instead
gives each layer a pool and a page table of its own (``src/generation/generator.cpp:
213-224``) with token-major blocks ``[blocks, block_size, kv_heads * head_dim]``
(``include/stratakv/layers/attention.h:88-91``).

A sequence holds one slot from its first step until it is released; the slot
indexes its length, its block lists and its row of the fixed-size state area
(zeroed when the slot is taken).  ``reserve`` takes every block a step needs
before anything runs, or raises ``CacheFull`` and takes nothing, the way the
reference checks capacity before it mutates (``src/layers/attention.cpp:197-212``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Sequence, Tuple

import torch

from ..parts.base import CacheRequest
from .allocator import CacheFull, IdAllocator
from .kinds import CacheKind, cache_kind


@dataclass
class CacheGroup:
    index: int
    request: CacheRequest
    kind: CacheKind
    entries: List[int]                    # cache entry ids, in local order
    blocks: IdAllocator
    # what the kind keeps, by tensor name: [entries, blocks + 1, *the kind's shape of one block]
    storage: Dict[str, torch.Tensor] = field(default_factory=dict)

    @property
    def keys(self) -> torch.Tensor:       # [entries, blocks, kv_heads, block_size, head_dim] for the "kv" kinds
        return self.storage["k"]

    @property
    def values(self) -> torch.Tensor:
        return self.storage["v"]


@dataclass
class SequenceRecord:
    serial: int = 0                       # distinguishes successive users of one slot
    length: int = 0
    blocks: Dict[int, List[int]] = field(default_factory=dict)    # group -> block ids by logical block
    dropped: Dict[int, int] = field(default_factory=dict)          # group -> leading logical blocks freed


class KVCache:
    def __init__(self, requests: Sequence[CacheRequest], num_blocks: int, block_size: int,
                 max_slots: int, dtype: torch.dtype, device):
        self.block_size = block_size
        self.num_blocks = num_blocks
        self.max_slots = max_slots
        self.dtype = dtype
        self.device = torch.device(device)
        self.slots = IdAllocator(max_slots, "slot")
        self.groups: List[CacheGroup] = []
        self.entry_group: List[Tuple[int, int]] = []        # entry -> (group, local index); (-1, -1): none
        by_key: Dict[tuple, CacheGroup] = {}
        for entry, request in enumerate(requests):
            try:
                kind = cache_kind(request.kind)
            except ValueError as error:
                raise ValueError(f"cache entry {entry}: {error}") from None
            if not kind.paged:
                self.entry_group.append((-1, -1))
                continue
            if kind.windowed and request.window <= 0:
                raise ValueError(f"cache entry {entry}: a window group needs a positive window")
            group = by_key.get(request.group_key())
            if group is None:
                group = CacheGroup(len(self.groups), request, kind, [], IdAllocator(num_blocks, "block"))
                by_key[request.group_key()] = group
                self.groups.append(group)
            self.entry_group.append((group.index, len(group.entries)))
            group.entries.append(entry)
        for group in self.groups:
            # one block more than the allocator hands out: padding rows of a step write there
            for name, shape in group.kind.block_tensors(group.request, block_size).items():
                group.storage[name] = torch.zeros((len(group.entries), num_blocks + 1) + tuple(shape), dtype=dtype,
                                                  device=self.device)
        # Fixed-size per-sequence state, one row per slot for each entry that asks for some.
        self.state_bytes = [r.state_bytes for r in requests]
        self._state = {entry: torch.zeros((max_slots, r.state_bytes), dtype=torch.uint8, device=self.device)
                       for entry, r in enumerate(requests) if r.state_bytes > 0}
        self.sequences: Dict[int, SequenceRecord] = {}
        self.trash_block = num_blocks         # owned by no sequence
        self._serial = 0

    # ---- storage views ---------------------------------------------------
    def entry_kv(self, entry: int):
        group, local = self.entry_group[entry]
        if group < 0:
            raise KeyError(f"cache entry {entry} keeps no keys")
        return self.groups[group].keys[local], self.groups[group].values[local]

    def entry_storage(self, entry: int) -> Dict[str, torch.Tensor]:
        """Every tensor the entry's cache kind keeps, by name: ``[blocks + 1, *shape of one block]``."""
        group, local = self.entry_group[entry]
        if group < 0:
            raise KeyError(f"cache entry {entry} keeps nothing per position")
        return {name: tensor[local] for name, tensor in self.groups[group].storage.items()}

    def entry_group_index(self, entry: int) -> int:
        return self.entry_group[entry][0]

    def state(self, entry: int) -> torch.Tensor:
        """``[max_slots, state_bytes]`` bytes of per-sequence state of one cache entry."""
        return self._state[entry]

    def bytes_per_token(self) -> int:
        return sum(tensor[:, 0].numel() * tensor.element_size() // self.block_size
                   for g in self.groups for tensor in g.storage.values())

    # ---- sequences ---------------------------------------------------------
    def acquire(self) -> int:
        """A free slot for a new sequence; its state rows are zeroed."""
        (slot,) = self.slots.take(1)
        self._serial += 1
        self.sequences[slot] = SequenceRecord(
            serial=self._serial, blocks={g.index: [] for g in self.groups}, dropped={g.index: 0 for g in self.groups})
        for state in self._state.values():
            state[slot].zero_()
        return slot

    def length(self, slot: int) -> int:
        return self.sequences[slot].length

    def _blocks_for(self, length: int) -> int:
        return -(-length // self.block_size)

    def holds(self, slot: int, length: int) -> bool:
        """True if the blocks that the sequence has already cover ``length`` positions in every group."""
        record = self.sequences[slot]
        return all(record.dropped[g.index] + len(record.blocks[g.index]) >= self._blocks_for(length)
                   for g in self.groups)

    def reserve(self, wanted: Dict[int, int]) -> None:
        """``wanted``: slot -> length after the coming step.  Takes every block
        the step needs in every group, or raises ``CacheFull`` and takes none."""
        need = {g.index: 0 for g in self.groups}
        for slot, new_length in wanted.items():
            record = self.sequences[slot]
            if new_length < record.length:
                raise ValueError(f"slot {slot}: length cannot shrink ({record.length} -> {new_length})")
            for group in self.groups:
                have = record.dropped[group.index] + len(record.blocks[group.index])
                need[group.index] += max(0, self._blocks_for(new_length) - have)
        for group in self.groups:
            if need[group.index] > group.blocks.free_count:
                raise CacheFull(
                    f"cache group {group.index}: step needs {need[group.index]} more blocks, "
                    f"{group.blocks.free_count} of {group.blocks.total} are free")
        for slot, new_length in wanted.items():
            record = self.sequences[slot]
            for group in self.groups:
                have = record.dropped[group.index] + len(record.blocks[group.index])
                extra = self._blocks_for(new_length) - have
                if extra > 0:
                    record.blocks[group.index].extend(group.blocks.take(extra))

    def advance(self, slot: int, new_length: int) -> None:
        """Record that the step wrote the sequence up to ``new_length``; a window
        group gives back blocks no later query can see."""
        record = self.sequences[slot]
        record.length = new_length
        for group in self.groups:
            if not group.kind.windowed:
                continue
            # The next query sits at position >= new_length and sees keys at
            # positions > position - window, so keys below new_length - window + 1 are dead.
            first_live = max(0, new_length - group.request.window + 1)
            dead_blocks = first_live // self.block_size
            drop = dead_blocks - record.dropped[group.index]
            if drop > 0:
                group.blocks.give_back(record.blocks[group.index][:drop])
                del record.blocks[group.index][:drop]
                record.dropped[group.index] = dead_blocks

    def release(self, slot: int) -> None:
        """Give the slot and all its blocks back."""
        record = self.sequences.pop(slot)
        for group in self.groups:
            group.blocks.give_back(record.blocks[group.index])
        self.slots.give_back([slot])

    def block_table_rows(self, group: int, slots: Sequence[int], width: int) -> List[List[int]]:
        """Block ids by logical block for each slot, padded to ``width`` with 0
        (padding and dropped blocks lie outside what kernels may read)."""
        rows = []
        for slot in slots:
            record = self.sequences[slot]
            row = [0] * record.dropped[group] + record.blocks[group]
            if len(row) > width:
                raise ValueError(f"slot {slot} holds {len(row)} blocks, table width is {width}")
            rows.append(row + [0] * (width - len(row)))
        return rows

    # ---- accounting ---------------------------------------------------------
    def free_blocks(self) -> List[int]:
        return [g.blocks.free_count for g in self.groups]

    def all_free(self) -> bool:
        return (self.slots.free_count == self.max_slots
                and all(g.blocks.free_count == g.blocks.total for g in self.groups)
                and not self.sequences)
