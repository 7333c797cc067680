"""Decode steps as CUDA graphs.

A decode step of the TinyLlama shape is some two hundred small kernels whose
launch cost from the host exceeds their run time (the reference issues about
445 driver calls per token, ``src/models/transformer_block.cpp:432-599``).  A
step in which every sequence brings one token is therefore captured once per
batch-size bucket into a CUDA graph over fixed device buffers and replayed:
per step the host fills one pinned array (token ids, positions, lengths, block
tables), copies it to the device, and launches the graph.

Rows beyond the live sequences pad the batch up to its bucket; they read and
write a spare cache block that no sequence owns, and their logits are dropped,
so padding changes no result.  Kernel arguments that a graph freezes (token
count, block-table width) are sizes of the bucket, never of the live batch;
what varies per step (positions, lengths, tables) is read from device memory.
"""
from __future__ import annotations

import gc
import weakref
from typing import Dict, List, Sequence

import numpy as np
import torch

from ..parts.base import StepBatch
from ..parts.workspace import Workspace

BUCKETS = (1, 2, 3, 4, 5, 6, 7, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256)


def bucket_for(batch: int) -> int:
    for size in BUCKETS:
        if batch <= size:
            return size
    return -(-batch // 64) * 64


class DecodeGraph:
    def __init__(self, engine, bucket: int, width: int):
        self._engine = weakref.ref(engine)     # no reference cycle: an engine is freed when dropped
        self.bucket = bucket
        self.width = width
        cache = engine.cache
        groups = len(cache.groups)
        b = bucket
        names = [("token_ids", b), ("positions", b), ("token_seq", b), ("cu_q", b + 1), ("ctx_after", b),
                 ("slot_ids", b), ("want_rows", b)] + [(("table", g), b * width) for g in range(groups)]
        self.offsets, total = {}, 0
        for name, count in names:
            self.offsets[name] = (total, count)
            total += count
        # The host array is copied to the device asynchronously; it may be rewritten only
        # after that copy has run, hence the event.
        self.host = torch.zeros(total, dtype=torch.int32, pin_memory=True)
        self.host_np = self.host.numpy()
        self.copied = torch.cuda.Event()
        self.copy_pending = False
        self.staged = None                     # what stage_rows() last prepared, until a fill() uses it
        self.device = torch.zeros(total, dtype=torch.int32, device=engine.device)
        self._np(("token_seq"))[:] = np.arange(b)
        self._np("cu_q")[:] = np.arange(b + 1)
        self._np("want_rows")[:] = np.arange(b)
        self._np("ctx_after")[:] = 1
        for g in range(groups):
            self._np(("table", g))[:] = cache.trash_block
        self.row_signature: Dict[tuple, tuple] = {}
        self.workspace = Workspace(engine.device)
        self.step = StepBatch(
            n_seqs=b, n_tokens=b, slots=[-1] * b, q_lens=[1] * b, ctx_before=[0] * b, max_q_len=1,
            max_ctx=width * cache.block_size,
            token_ids=self._dev("token_ids"), positions=self._dev("positions"), token_seq=self._dev("token_seq"),
            cu_q=self._dev("cu_q"), ctx_after=self._dev("ctx_after"), slot_ids=self._dev("slot_ids"),
            block_tables={g: self._dev(("table", g)).view(b, width) for g in range(groups)}, cache=cache)
        self.want_rows = self._dev("want_rows")
        self.graph = None
        self.logits = None
        self.kernels_per_replay = 0

    @property
    def engine(self):
        return self._engine()

    def _np(self, name):
        start, count = self.offsets[name]
        return self.host_np[start:start + count]

    def _dev(self, name):
        start, count = self.offsets[name]
        return self.device[start:start + count]

    def _key(self, slots: Sequence[int], ctx_before: Sequence[int]):
        sequences = self.engine.cache.sequences
        return tuple((slot, sequences[slot].serial, before) for slot, before in zip(slots, ctx_before))

    def stage_rows(self, slots: Sequence[int], ctx_before: Sequence[int]) -> None:
        """Everything of a step's metadata but the token ids: positions, lengths, slots, block tables.
        It may run while the step before is still on the GPU (the engine calls it right after a launch,
        for the step it expects next), so that only the token ids remain once they are known."""
        cache = self.engine.cache
        live = len(slots)
        b = self.bucket
        if self.copy_pending:
            self.copied.synchronize()
            self.copy_pending = False
        pos, after, slot_ids = self._np("positions"), self._np("ctx_after"), self._np("slot_ids")
        pos[:live] = ctx_before
        after[:live] = pos[:live] + 1
        slot_ids[:live] = slots
        if live < b:
            pos[live:] = 0
            after[live:] = 1
            slot_ids[live:] = 0
        for g, group in enumerate(cache.groups):
            table = self._np(("table", g)).reshape(b, self.width)
            for row in range(b):
                if row < live:
                    record = cache.sequences[slots[row]]
                    blocks = record.blocks[group.index]
                    dropped = record.dropped[group.index]
                    signature = (record.serial, len(blocks), dropped)
                else:
                    signature = None
                if self.row_signature.get((g, row), 0) == signature:
                    continue                       # this row of the table is already up to date
                self.row_signature[(g, row)] = signature
                table[row, :] = cache.trash_block
                if row < live:
                    table[row, dropped:dropped + len(blocks)] = blocks
        self.staged = self._key(slots, ctx_before)

    def staged_for(self, slots: Sequence[int], ctx_before: Sequence[int]) -> bool:
        """True if ``stage_rows`` has prepared exactly this step (these sequences at these lengths)."""
        return self.staged is not None and self.staged == self._key(slots, ctx_before)

    def fill(self, slots: Sequence[int], tokens, ctx_before: Sequence[int], staged: bool = False,
             device_tokens=None) -> None:
        """``staged``: the caller has checked ``staged_for`` for this step.  ``tokens``: the token ids on the host,
        or None with ``device_tokens`` (int32 on the device, the slots' order): they are copied into place on the
        device, behind the copy of everything else."""
        if not staged:
            self.stage_rows(slots, ctx_before)
        self.staged = None
        live = len(slots)
        ids = self._np("token_ids")
        if tokens is not None:
            ids[:live] = tokens
        if live < self.bucket:
            ids[live:] = 0
        self.device.copy_(self.host, non_blocking=True)
        if tokens is None:
            self._dev("token_ids")[:live].copy_(device_tokens[:live], non_blocking=True)
        self.copied.record()
        self.copy_pending = True

    def run(self):
        """Launch the step (captures the graph at first use); returns logits ``[bucket, vocab]``."""
        engine = self.engine
        rt = engine.rt
        if self.graph is None:
            saved = rt.workspace
            rt.workspace = self.workspace
            try:
                engine.model.prepare_positions(self.step.max_ctx)
                self.logits = engine.model.forward(self.step, self.want_rows, self.bucket)    # eager warm-up
                torch.cuda.synchronize(engine.device)
                before = engine.kernel_launches()
                graph = torch.cuda.CUDAGraph()
                # Garbage collection inside a capture could destroy another engine's graph,
                # which is not allowed while a stream captures.
                gc.collect()
                was_enabled = gc.isenabled()
                gc.disable()
                try:
                    with torch.cuda.graph(graph):
                        self.logits = engine.model.forward(self.step, self.want_rows, self.bucket)
                finally:
                    if was_enabled:
                        gc.enable()
                self.kernels_per_replay = engine.kernel_launches() - before
                engine.discount_launches(self.kernels_per_replay)       # recorded, not run
                self.graph = graph
            finally:
                rt.workspace = saved
            # the warm-up already ran this step once; the replay below recomputes the same values
        self.graph.replay()
        engine.graph_launches += self.kernels_per_replay
        return self.logits
