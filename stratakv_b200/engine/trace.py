"""Trace replay: feed given token ids through the engine step by step and write logits.

Nothing is sampled.  Each input line is one step, ``{"step": s, "entries":
[{"id", "tokens", "want"}], "end": [ids]}``; a request takes a cache slot when
its id first appears and gives it back when a step's ``end`` names it.  The
steps go through ``Engine.step``, the same function generation uses, so the
cache, the kernels and the batching are the ones that serve.  The reference's
nearest tool replays every GPU step on a CPU shadow model and prints the
differences (``src/generation/generator.cpp:596-613``); this one writes the
logits themselves for others to compare.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path
from typing import Dict, IO

import numpy as np

from .engine import Engine, StepEntry, StepError


def replay(engine: Engine, lines: IO[str], out_dir, done: IO[str] = sys.stdout) -> int:
    """Run every step read from ``lines``; returns the number of steps run."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    slots: Dict[str, int] = {}
    count = 0
    for raw in lines:
        raw = raw.strip()
        if not raw:
            continue
        record = json.loads(raw)
        step_id = record["step"]
        entries = []
        for item in record.get("entries", []):
            ident = item["id"]
            if ident not in slots:
                slots[ident] = engine.open_sequence()
            entries.append(StepEntry(slots[ident], item["tokens"], item.get("want", [])))
        if entries:
            logits = engine.step(entries)
            if logits is not None:
                host = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                host.tofile(out_dir / f"{step_id}.f32")
            engine.check_flags()
        for ident in record.get("end", []):
            if ident in slots:
                engine.close_sequence(slots.pop(ident))
        count += 1
        done.write(f"done {step_id}\n")
        done.flush()
    return count
