"""The engine: a model, its cache, and the one step function everything uses.

``step`` takes a batch of sequences, each with its next tokens (a whole prompt,
a piece of one, or a single decoded token) and the places whose logits are
wanted; it runs only those tokens, as one packed batch without padding, against
what earlier steps left in the cache, and returns the logits.  The reference's
counterpart handles one token of one sequence per call
(``src/generation/generator.cpp:571-614``, ``src/models/transformer_block.cpp:348-351``).
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import array

import numpy as np
import torch

from .. import models as _models  # noqa: F401  (registers the architectures)
from .. import ops as _ops
from ..cache import CacheFull, KVCache
from ..config import EngineConfig, load_config
from ..config.registry import resolve_architecture
from ..parts.base import Runtime, StepBatch
from ..parts.spec import ModelSpec
from ..parts.workspace import Workspace
from ..weights.loader import load_checkpoint
from .model import Model, cache_requests, default_head_dim, expected_tensors


@dataclass
class StepEntry:
    """One sequence's share of a step: its slot, its next tokens, and the
    indices among these tokens whose logits are wanted."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepError(ValueError):
    pass


def _token_array(tokens) -> np.ndarray:
    """A step's token ids as an integer array.  A list of Python ints, the usual case, goes through the ``array``
    module, which reads such a list twice as fast as numpy does (a 2,048-token prompt: 36 against 72 us)."""
    if isinstance(tokens, np.ndarray) and tokens.dtype.kind in "iu":
        return tokens
    if isinstance(tokens, (list, tuple)):
        try:
            return np.frombuffer(array.array("q", tokens), dtype=np.int64)
        except (TypeError, OverflowError):
            pass                                 # (numpy integers, or something that is no token id: the slow way tells)
    out = np.asarray(tokens)
    if out.dtype.kind not in "iu":
        if out.dtype.kind == "b" or not all(isinstance(t, (int, np.integer)) for t in tokens):
            raise StepError("token ids must be integers")
        try:
            out = np.array([int(t) for t in tokens], dtype=np.int64)
        except OverflowError:
            raise StepError("a token id is outside the vocabulary (it does not even fit 64 bits)") from None
    return out


class Engine:
    def __init__(self, spec: ModelSpec, tensors: Mapping[str, torch.Tensor], config: EngineConfig,
                 kernel_loader=None, verbose: bool = True):
        self.spec = spec
        self.config = config
        # most positions a sequence may reach: the engine's setting, else the model's own limit, else none
        self.max_context = config.max_context or spec.max_positions or 0
        if kernel_loader is None:
            self.device = _ops.require_cuda(config.device)
            kernel_loader = lambda dtype, head_dim: _ops.kernels_for(dtype, head_dim, verbose=verbose)
        else:                                   # tests hand in a stand-in for the kernels
            self.device = torch.device(config.device)
        self.workspace = Workspace(self.device)
        self.rt = Runtime(config.dtype, self.device, self.workspace, kernel_loader, default_head_dim(spec))
        self.model = Model(spec, self.rt)
        self.model.bind(tensors)
        self.cache = KVCache(cache_requests(spec), config.num_blocks, config.block_size, config.slots,
                             config.dtype, self.device)
        self._pinned: Optional[torch.Tensor] = None
        self._meta: Optional[torch.Tensor] = None
        self._copied = None
        self._graphs = {}
        self._use_graphs = (config.use_cuda_graphs and self.device.type == "cuda" and self.model.graph_safe())
        self.graph_launches = 0
        self._launch_base = _ops.Kernels.launches
        self._io_bytes = (0, 0)

    # ---- construction ----------------------------------------------------------
    @classmethod
    def from_folder(cls, model_dir, config: EngineConfig, verbose: bool = True) -> "Engine":
        """Open a folder with ``config.json`` and ``model.safetensors``; the
        architecture named in ``config.json`` chooses the model."""
        arch, model_config = load_config(model_dir)
        spec = arch.build_spec(model_config)
        expected = {name: request.shape for name, request in expected_tensors(spec).items()}
        tensors = load_checkpoint(model_dir, expected, spec.ignorable)
        engine = cls(spec, tensors, config, verbose=verbose)
        engine.model_config = model_config
        return engine

    @classmethod
    def from_config(cls, model_config, config: EngineConfig, seed: int = 0,
                    stored_dtype: Optional[torch.dtype] = None, verbose: bool = True) -> "Engine":
        """Random weights for ``model_config`` made in memory (no folder)."""
        from ..weights.random_init import random_tensors
        spec = resolve_architecture(model_config.architecture).build_spec(model_config)
        tensors = random_tensors(expected_tensors(spec), seed, dtype=stored_dtype or config.dtype)
        engine = cls(spec, tensors, config, verbose=verbose)
        engine.model_config = model_config
        return engine

    # ---- sequences ---------------------------------------------------------------
    def open_sequence(self) -> int:
        return self.cache.acquire()

    def close_sequence(self, slot: int) -> None:
        self.cache.release(slot)

    # ---- the step ------------------------------------------------------------------
    def _metadata(self, count: int) -> Tuple[torch.Tensor, torch.Tensor]:
        if self._meta is None or self._meta.numel() < count:
            capacity = max(count, 4096, 2 * (self._meta.numel() if self._meta is not None else 0))
            self._meta = torch.empty(capacity, dtype=torch.int32, device=self.device)
            pin = self.device.type == "cuda"
            self._pinned = torch.empty(capacity, dtype=torch.int32, pin_memory=pin)
        return self._pinned, self._meta

    def prepare(self, entries: Sequence[StepEntry]):
        """Check a step, reserve its cache blocks, and upload its metadata.
        Returns ``(StepBatch, want_rows, n_want)``; nothing has run yet."""
        if not entries:
            raise StepError("a step needs at least one sequence")
        vocab = self.spec.vocab_size
        slots = [e.slot for e in entries]
        if len(set(slots)) != len(slots):
            raise StepError("a sequence appears twice in one step")
        if len(entries) > self.config.slots:
            raise StepError(f"{len(entries)} sequences in one step; the engine holds {self.config.slots}")
        q_lens, ctx_before, wanted, token_arrays = [], [], {}, []
        for e in entries:
            if e.slot not in self.cache.sequences:
                raise StepError(f"slot {e.slot} is not open")
            if len(e.tokens) == 0:
                raise StepError(f"slot {e.slot}: a step needs at least one token per sequence")
            tokens = _token_array(e.tokens)
            if int(tokens.min()) < 0 or int(tokens.max()) >= vocab:
                outside = np.flatnonzero((tokens < 0) | (tokens >= vocab))
                raise StepError(f"slot {e.slot}: token id {int(tokens[outside[0]])} is outside the vocabulary of {vocab}")
            for w in e.want:
                if not (0 <= int(w) < len(e.tokens)):
                    raise StepError(f"slot {e.slot}: wanted place {w} is outside this step's {len(e.tokens)} tokens")
            before = self.cache.length(e.slot)
            self._check_context(e.slot, before + len(e.tokens))
            token_arrays.append(tokens)
            q_lens.append(len(e.tokens))
            ctx_before.append(before)
            wanted[e.slot] = before + len(e.tokens)
        self.cache.reserve(wanted)              # CacheFull leaves everything as it was

        n, total = len(entries), sum(q_lens)
        max_ctx = max(wanted.values())
        width = -(-max_ctx // self.cache.block_size)
        cu_q = np.zeros(n + 1, dtype=np.int64)
        np.cumsum(q_lens, out=cu_q[1:])
        want_rows = [int(cu_q[index]) + int(w) for index, e in enumerate(entries) for w in e.want]
        tables = [self.cache.block_table_rows(g.index, slots, width) for g in self.cache.groups]
        # everything goes into one pinned array, written through its numpy view, and up in one copy
        pieces = (("token_ids", total), ("positions", total), ("token_seq", total), ("cu_q", n + 1), ("ctx_after", n),
                  ("slot_ids", n), ("want_rows", len(want_rows))) + tuple((("table", g), n * width) for g in range(len(tables)))
        offsets, length = {}, 0
        for name, count in pieces:
            offsets[name] = (length, count)
            length += count
        pinned, meta = self._metadata(length)
        if self._copied is not None:
            self._copied.synchronize()          # the last step's copy must have left the pinned array
        host = pinned.numpy()

        def put(key, values):
            start, count = offsets[key]
            host[start:start + count] = values

        put("token_ids", np.concatenate(token_arrays) if n > 1 else token_arrays[0])
        put("positions", np.concatenate([np.arange(b, b + q) for b, q in zip(ctx_before, q_lens)]))
        put("token_seq", np.repeat(np.arange(n), q_lens))
        put("cu_q", cu_q)
        put("ctx_after", [wanted[slot] for slot in slots])
        put("slot_ids", slots)
        if want_rows:
            put("want_rows", want_rows)
        for g, rows in enumerate(tables):
            put(("table", g), np.asarray(rows, dtype=np.int64).reshape(-1))
        meta[:length].copy_(pinned[:length], non_blocking=True)
        if self.device.type == "cuda":
            self._copied = self._copied or torch.cuda.Event()
            self._copied.record()

        def view(key):
            start, count = offsets[key]
            return meta[start:start + count]

        step = StepBatch(
            n_seqs=n, n_tokens=total, slots=slots, q_lens=q_lens, ctx_before=ctx_before,
            max_q_len=max(q_lens), max_ctx=max_ctx,
            token_ids=view("token_ids"), positions=view("positions"), token_seq=view("token_seq"),
            cu_q=view("cu_q"), ctx_after=view("ctx_after"), slot_ids=view("slot_ids"),
            block_tables={g: view(("table", g)).view(n, width) for g in range(len(tables))},
            cache=self.cache)
        return step, (view("want_rows") if want_rows else None), len(want_rows)

    def _check_context(self, slot: int, length: int) -> None:
        if self.max_context and length > self.max_context:
            raise StepError(f"slot {slot}: the step would bring the sequence to {length} positions; "
                            f"the limit is {self.max_context} (max_position_embeddings, or the engine's max_context)")

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run one step.  Returns float32 logits ``[wanted, vocab]`` on the device,
        in the order of the entries and of their ``want`` (``None`` when nothing
        is wanted).  The tensor is scratch memory: use or copy it before the next step."""
        if self._use_graphs and entries and all(len(e.tokens) == 1 for e in entries):
            return self._decode_step(entries)
        step, want_rows, n_want = self.prepare(entries)
        logits = self.model.forward(step, want_rows, n_want)
        for e in entries:
            self.cache.advance(e.slot, self.cache.length(e.slot) + len(e.tokens))
        return logits

    def _decode_step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """One token per sequence: the step runs as a CUDA graph of its batch-size bucket."""
        vocab = self.spec.vocab_size
        slots = [e.slot for e in entries]
        tokens = [int(e.tokens[0]) for e in entries]
        if min(tokens) < 0 or max(tokens) >= vocab:
            slot, token = next((s, t) for s, t in zip(slots, tokens) if not (0 <= t < vocab))
            raise StepError(f"slot {slot}: token id {token} is outside the vocabulary of {vocab}")
        rows = []
        for index, e in enumerate(entries):
            for w in e.want:
                if int(w) != 0:
                    raise StepError(f"slot {e.slot}: wanted place {w} is outside this step's 1 tokens")
                rows.append(index)
        logits = self._launch_decode(slots, tokens, None)
        if not rows:
            return None
        if len(rows) == len(entries):
            return logits[:len(entries)]
        return logits[torch.tensor(rows, device=self.device)]

    def step_ahead(self, slots: Sequence[int], device_tokens: torch.Tensor) -> torch.Tensor:
        """A decode step whose token ids are already on the device (int32, one per slot, in the slots' order), for
        a caller that launches a step before the host has read the tokens the step before chose.  Returns the
        logits of every sequence.  Only engines that run decode steps as graphs have it (``can_step_ahead``)."""
        if device_tokens.dtype != torch.int32 or device_tokens.numel() < len(slots):
            raise StepError("step_ahead: one int32 token id per slot is needed")
        return self._launch_decode(list(slots), None, device_tokens)[:len(slots)]

    @property
    def can_step_ahead(self) -> bool:
        return bool(self._use_graphs)

    def _launch_decode(self, slots, tokens, device_tokens) -> torch.Tensor:
        from .decode_graph import DecodeGraph, bucket_for
        if len(set(slots)) != len(slots):
            raise StepError("a sequence appears twice in one step")
        if len(slots) > self.config.slots:
            raise StepError(f"{len(slots)} sequences in one step; the engine holds {self.config.slots}")
        sequences = self.cache.sequences
        try:
            ctx_before = [sequences[slot].length for slot in slots]
        except KeyError as missing:
            raise StepError(f"slot {missing.args[0]} is not open") from None
        wanted = {slot: before + 1 for slot, before in zip(slots, ctx_before)}
        if self.max_context and max(ctx_before) + 1 > self.max_context:
            for slot, length in wanted.items():
                self._check_context(slot, length)
        bucket = bucket_for(len(slots))
        graph = self._graphs.get(bucket)
        staged = graph is not None and graph.staged_for(slots, ctx_before)
        if not staged:                          # (a staged step needs no new block and fits its graph: see _stage_next)
            self.cache.reserve(wanted)
            need = -(-max(wanted.values()) // self.cache.block_size)
            if graph is None or graph.width < need:
                width = 4
                while width < need:
                    width *= 2
                graph = DecodeGraph(self, bucket, width)
                self._graphs[bucket] = graph
        graph.fill(slots, tokens, ctx_before, staged, device_tokens)
        logits = graph.run()
        self._io_bytes = (graph.host.numel() * 4, self._io_bytes[1])
        for slot, length in wanted.items():
            self.cache.advance(slot, length)
        self._stage_next(graph, slots)
        return logits

    def _stage_next(self, graph, slots) -> None:
        """While the step just launched runs: prepare the metadata of the step that most likely
        follows (the same sequences, one token further).  It takes nothing from the cache: if a
        sequence would need a new block the work is left to the next step itself.  If another
        step comes instead, nothing is lost: the next fill starts over."""
        lengths = [self.cache.length(slot) for slot in slots]
        if any(not self.cache.holds(slot, length + 1) for slot, length in zip(slots, lengths)):
            return
        graph.stage_rows(slots, lengths)

    # ---- accounting ------------------------------------------------------------------
    def kernel_launches(self) -> int:
        return _ops.Kernels.launches - self._launch_base

    def discount_launches(self, count: int) -> None:
        """Calls made while a graph was being captured were recorded, not run."""
        self._launch_base += count

    def launch_count(self) -> int:
        """Kernels of this library launched so far, graph replays included."""
        return self.kernel_launches() + self.graph_launches

    def last_step_io_bytes(self):
        """(host-to-device, device-to-host) bytes of the most recent decode step."""
        return self._io_bytes

    def generate(self, prompts, max_new_tokens, params=None, stop_ids=None, ignore_eos: bool = False,
                 streams=None):
        """Generate for a list of prompts (lists of token ids).  Returns a
        ``GenerationOutput`` whose ``sequences[i]`` is prompt ``i`` followed by its
        new tokens.  ``stop_ids`` defaults to the model's end-of-sequence ids;
        ``ignore_eos`` generates to the budget regardless."""
        from ..sampling import Sampler, SamplingParams
        from .generate import generate as run
        params = params or SamplingParams()
        sampler = Sampler(self.rt.kernels(), params, self.model.flags)
        if ignore_eos:
            stop_ids = ()
        elif stop_ids is None:
            stop_ids = self.spec.stop_token_ids

        chooser = _Chooser(self, sampler, params, max(1, len(prompts)))
        sync = torch.cuda.synchronize if self.device.type == "cuda" else (lambda: None)
        output = run(self, chooser, prompts, max_new_tokens, stop_ids, streams, sync=sync)
        self.check_flags()
        return output

    def check_flags(self) -> None:
        """Raise if a kernel flagged something since the last check (reads one word per flag from the
        device).  The flags are cleared, so the engine can be used again afterwards."""
        flags = int(self.model.flags.item())
        for kernels in _ops._LOADED.values():
            if getattr(kernels, "error_flag", None) is not None:
                word = int(kernels.error_flag.item())
                if word:
                    kernels.error_flag.zero_()
                    flags |= word
        if flags:
            self.model.flags.zero_()
            raise StepError(f"device flags raised: {flags:#x} ({describe_flags(flags)})")


class _Chooser:
    """Chooses one token per row of a step's logits on the device and brings the ids to the host.

    Called like a function it waits for the ids.  ``launch`` only queues the work and returns a handle;
    ``tokens_device(handle)`` is where the ids will be on the device (a following step can be fed from there),
    ``result(handle)`` waits and returns them.  Three sets of buffers rotate, so two choices may be in flight
    while a third is read.  Streams and counters of a sampled step leave from pinned memory in one copy."""
    RING = 3

    def __init__(self, engine, sampler, params, rows: int):
        self.engine, self.sampler, self.params = engine, sampler, params
        self.on_gpu = engine.device.type == "cuda"
        pin = self.on_gpu
        self.chosen = [torch.empty(rows, dtype=torch.int32, device=engine.device) for _ in range(self.RING)]
        self.landing = [torch.empty(rows, dtype=torch.int32, pin_memory=pin) for _ in range(self.RING)]
        self.landed = [torch.cuda.Event() if self.on_gpu else None for _ in range(self.RING)]
        self.draw_host = [torch.empty((2, rows), dtype=torch.int32, pin_memory=pin) for _ in range(self.RING)]
        self.draw_device = [torch.empty((2, rows), dtype=torch.int32, device=engine.device) for _ in range(self.RING)]
        self.counts = [0] * self.RING
        self.turn = 0

    def launch(self, logits, row_streams, counters) -> int:
        handle = self.turn
        self.turn = (self.turn + 1) % self.RING
        count = logits.shape[0]
        out = self.chosen[handle][:count]
        if self.params.greedy:
            self.sampler.sample(logits, None, None, out)
        else:
            host = self.draw_host[handle].numpy()
            host[0, :count] = row_streams
            host[1, :count] = counters
            self.draw_device[handle].copy_(self.draw_host[handle], non_blocking=True)
            self.sampler.sample(logits, self.draw_device[handle][0, :count], self.draw_device[handle][1, :count], out)
        self.counts[handle] = count
        self.engine._io_bytes = (self.engine._io_bytes[0], count * 4)
        if self.on_gpu:
            self.landing[handle][:count].copy_(out, non_blocking=True)
            self.landed[handle].record()
        return handle

    def tokens_device(self, handle: int) -> torch.Tensor:
        return self.chosen[handle][:self.counts[handle]]

    def result(self, handle: int):
        count = self.counts[handle]
        if not self.on_gpu:
            return self.chosen[handle][:count].tolist()
        self.landed[handle].synchronize()
        return self.landing[handle][:count].tolist()

    def __call__(self, logits, row_streams, counters):
        return self.result(self.launch(logits, row_streams, counters))


FLAG_MEANINGS = {1: "a token id outside the vocabulary reached the embedding",
                 2: "non-finite logits",
                 4: "a wait inside a kernel timed out (its result is not valid)"}


def describe_flags(word: int) -> str:
    """The meaning of every bit set in a flag word that kernels raise."""
    known = [text for bit, text in FLAG_MEANINGS.items() if word & bit]
    unknown = word & ~sum(FLAG_MEANINGS)
    if unknown:
        known.append(f"unknown bits {unknown:#x}")
    return "; ".join(known)
