"""Command line in the manner of the reference's ``stratakv_cli`` (``src/cli.cpp:179-322``).

    stratakv_cli [--temp T] [--top-k K] [--top-p P] <model> <max_new_tokens> <prompt_id>...

Options may stand anywhere among the positionals; an unknown ``--option`` is an
error; at least a model, ``max_new_tokens`` and one prompt token are needed;
token ids are non-negative integers.  All ids (prompt, then generated) go to
standard output on one line; ``[TIMING]`` goes to standard error; exit codes are
0 (ok), 1 (error) and 2 (no arguments).  ``<model>`` is a folder with
``config.json`` and ``model.safetensors`` (or the path of that file): the sizes
come from ``config.json``, where the reference guesses them from tensor shapes.

Added here: ``--seed S`` (reproducible draws; the reference documents the flag
but does not have it), ``--dtype bfloat16|float32``, ``--max-tokens N`` (cache
size), ``--stop-id ID`` (repeatable; default: the model's eos ids),
``--ignore-eos``, ``--block-size N`` (cache block, default 64), ``--max-context N``
(most positions a request may reach, in place of the model's ``max_position_embeddings``),
``--prompt-file FILE``
with one request per line, which are generated as a batch and printed one line
each, and ``--random CONFIG.json``: no checkpoint, weights drawn from
``--weights-seed`` (default 0) for the configuration in that file; ``<model>`` is
left out then.
"""
from __future__ import annotations

import math
import sys
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import List, Optional

USAGE = ("Usage: stratakv_cli [--temp T] [--top-k K] [--top-p P] [--seed S] [--dtype bfloat16|float32]\n"
         "                    [--max-tokens N] [--block-size N] [--max-context N] [--stop-id ID]... [--ignore-eos]\n"
         "                    [--prompt-file FILE] [--random CONFIG.json [--weights-seed S]]\n"
         "                    <model> <max_new_tokens> <prompt_id>...\n"
         "       options may also appear between max_new_tokens and the prompt tokens\n")


class UsageError(ValueError):
    pass


@dataclass
class Arguments:
    model: str = ""
    max_new_tokens: int = 0
    prompts: List[List[int]] = field(default_factory=list)
    temperature: float = 0.0          # src/cli.cpp:191: the CLI's default is greedy
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0
    dtype: str = "bfloat16"
    max_tokens: Optional[int] = None
    stop_ids: Optional[List[int]] = None
    ignore_eos: bool = False
    block_size: int = 64
    max_context: int = 0
    random_config: Optional[str] = None
    weights_seed: int = 0


def _int(text: str, what: str) -> int:
    try:
        return int(text, 10)
    except ValueError:
        raise UsageError(f"invalid {what}: {text}") from None


def _float(text: str, what: str) -> float:
    try:
        value = float(text)
    except ValueError:
        raise UsageError(f"invalid {what}: {text}") from None
    if not math.isfinite(value):
        raise UsageError(f"invalid {what}: {text}")
    return value


def parse_arguments(argv: List[str]) -> Arguments:
    args = Arguments()
    positional: List[str] = []
    prompt_file = None
    index = 0

    def value_of(option: str) -> str:
        nonlocal index
        index += 1
        if index >= len(argv):
            raise UsageError(f"{option} requires a value")
        return argv[index]

    while index < len(argv):
        word = argv[index]
        if word == "--temp":
            args.temperature = _float(value_of(word), "--temp")
        elif word == "--top-k":
            args.top_k = _int(value_of(word), "--top-k")
        elif word == "--top-p":
            args.top_p = _float(value_of(word), "--top-p")
        elif word == "--seed":
            args.seed = _int(value_of(word), "--seed")
        elif word == "--dtype":
            args.dtype = value_of(word)
        elif word == "--max-tokens":
            args.max_tokens = _int(value_of(word), "--max-tokens")
        elif word == "--stop-id":
            args.stop_ids = (args.stop_ids or []) + [_int(value_of(word), "--stop-id")]
        elif word == "--ignore-eos":
            args.ignore_eos = True
        elif word == "--block-size":
            args.block_size = _int(value_of(word), "--block-size")
        elif word == "--max-context":
            args.max_context = _int(value_of(word), "--max-context")
            if args.max_context < 0:
                raise UsageError("--max-context must be nonnegative")
        elif word == "--random":
            args.random_config = value_of(word)
        elif word == "--weights-seed":
            args.weights_seed = _int(value_of(word), "--weights-seed")
        elif word == "--prompt-file":
            prompt_file = value_of(word)
        elif word.startswith("--"):
            raise UsageError(f"unknown option: {word}")
        else:
            positional.append(word)
        index += 1
    if args.random_config is not None:
        positional.insert(0, "")                  # no model folder: the configuration file stands for it
    needed = 2 if prompt_file else 3
    if len(positional) < needed:
        raise UsageError("expected a model path, max_new_tokens, and at least one prompt token")
    args.model = positional[0]
    args.max_new_tokens = _int(positional[1], "max_new_tokens")
    if args.max_new_tokens < 0:
        raise UsageError("max_new_tokens must be nonnegative")

    def tokens(words):
        ids = [_int(w, "prompt token") for w in words]
        if any(t < 0 for t in ids):
            raise UsageError("prompt token must be nonnegative")
        return ids

    if len(positional) > 2:
        args.prompts.append(tokens(positional[2:]))
    if prompt_file:
        for line in Path(prompt_file).read_text().splitlines():
            if line.strip():
                args.prompts.append(tokens(line.split()))
    if not args.prompts:
        raise UsageError("expected at least one prompt")
    return args


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        sys.stderr.write(USAGE)
        return 2
    try:
        args = parse_arguments(argv)
        from . import Engine, EngineConfig
        from .sampling import SamplingParams

        params = SamplingParams(args.temperature, args.top_k, args.top_p, args.seed)
        model = Path(args.model)
        if model.is_file():
            model = model.parent
        load_start = time.perf_counter()
        block = args.block_size
        if block <= 0:
            raise UsageError("--block-size must be positive")
        need = sum(-(-(len(p) + args.max_new_tokens) // block) * block for p in args.prompts)
        config = EngineConfig(max_tokens=args.max_tokens or need, dtype=args.dtype, block_size=block,
                              max_context=args.max_context)
        if args.random_config is not None:
            from .config import load_config
            _, model_config = load_config(args.random_config)
            engine = Engine.from_config(model_config, config, seed=args.weights_seed)
        else:
            engine = Engine.from_folder(model, config)
        load_ms = 1000.0 * (time.perf_counter() - load_start)
        output = engine.generate(args.prompts, args.max_new_tokens, params, stop_ids=args.stop_ids,
                                 ignore_eos=args.ignore_eos)
        t = output.timings
        generated = sum(len(s) - len(p) for s, p in zip(output.sequences, args.prompts))
        gen_ms = t.prefill_ms + t.decode_ms
        # The reference's figure divides by prompt plus decode time (src/cli.cpp:292-304); the
        # parts are given beside it.
        tps = generated / (gen_ms / 1000.0) if gen_ms > 0 else 0.0
        sys.stderr.write(f"[TIMING] load_ms = {load_ms:f}, gen_ms = {gen_ms:f}, tokens = {generated}, "
                         f"pure_decode_tps = {tps:f}\n")
        sys.stderr.write(f"[TIMING_PARTS] prefill_ms = {t.prefill_ms:f}, prefill_tokens = {t.prefill_tokens}, "
                         f"decode_ms = {t.decode_ms:f}, decode_tokens = {t.decode_tokens}, "
                         f"decode_tps = {t.decode_tps:f}, batches = {t.batches}\n")
        for sequence in output.sequences:
            sys.stdout.write(" ".join(str(token) for token in sequence) + "\n")
        return 0
    except Exception as error:  # noqa: BLE001 - the command line's boundary, as in src/cli.cpp:318-321
        sys.stderr.write(f"stratakv_cli: {error}\n")
        return 1


if __name__ == "__main__":
    raise SystemExit(main())
