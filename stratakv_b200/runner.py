"""Python entry point in the manner of the reference's ``runner.py``.

The reference script tokenizes a fixed chat with a downloaded tokenizer, runs
the command-line binary with ``--temp 0.8 --top-k 40 --top-p 0.95`` for 500 new
tokens and decodes what comes back (``runner.py:11-16, 33-47, 58-101``).  This
one keeps those option names and defaults, runs the engine in-process, and
works on token ids alone (there is no network here); with ``--tokenizer DIR``
and a tokenizer library installed it also takes ``--prompt TEXT`` and prints text.

    python -m stratakv_b200.runner --model DIR --prompt-ids 1 15043 3186 --max-new-tokens 32

``run(model_dir, prompts, ...)`` is the same thing as a function.
"""
from __future__ import annotations

import argparse
import sys
from typing import List, Optional, Sequence

MAX_NEW_TOKENS = 500          # runner.py:16


def run(model_dir, prompts: Sequence[Sequence[int]], max_new_tokens: int = MAX_NEW_TOKENS, temp: float = 0.8,
        top_k: int = 40, top_p: float = 0.95, seed: int = 0, dtype: str = "bfloat16",
        max_tokens: Optional[int] = None, ignore_eos: bool = False, engine=None):
    """Generate for ``prompts`` (lists of token ids); returns ``(sequences, timings, engine)``."""
    from . import Engine, EngineConfig
    from .sampling import SamplingParams

    if engine is None:
        block = 64
        need = sum(-(-(len(p) + max_new_tokens) // block) * block for p in prompts)
        engine = Engine.from_folder(model_dir, EngineConfig(max_tokens=max_tokens or need, dtype=dtype,
                                                            block_size=block))
    output = engine.generate([list(p) for p in prompts], max_new_tokens,
                             SamplingParams(temp, top_k, top_p, seed), ignore_eos=ignore_eos)
    return output.sequences, output.timings, engine


def parse_args(argv=None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--temp", type=float, default=0.8, help="sampling temperature (default: 0.8)")
    parser.add_argument("--top-k", type=int, default=40, help="retain only the K highest-logit tokens (default: 40)")
    parser.add_argument("--top-p", type=float, default=0.95,
                        help="retain the smallest nucleus under this probability (default: 0.95)")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--max-new-tokens", type=int, default=MAX_NEW_TOKENS)
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    parser.add_argument("--prompt-ids", type=int, nargs="+", help="the prompt as token ids")
    parser.add_argument("--prompt", help="the prompt as text (needs --tokenizer)")
    parser.add_argument("--tokenizer", help="folder of a tokenizer to encode --prompt and decode the output")
    parser.add_argument("--ignore-eos", action="store_true")
    return parser.parse_args(argv)


def main(argv=None) -> int:
    options = parse_args(argv)
    tokenizer = None
    if options.tokenizer:
        from transformers import AutoTokenizer          # a tokenizer only; no model code is used
        tokenizer = AutoTokenizer.from_pretrained(options.tokenizer, local_files_only=True)
    if options.prompt is not None:
        if tokenizer is None:
            raise SystemExit("runner: --prompt needs --tokenizer; use --prompt-ids otherwise")
        prompt_ids: List[int] = list(tokenizer(options.prompt)["input_ids"])
    elif options.prompt_ids:
        prompt_ids = options.prompt_ids
    else:
        raise SystemExit("runner: give --prompt-ids or --prompt")
    sequences, timings, _ = run(options.model, [prompt_ids], options.max_new_tokens, options.temp, options.top_k,
                                options.top_p, options.seed, options.dtype, ignore_eos=options.ignore_eos)
    print(f"[TIMING] prefill_ms = {timings.prefill_ms:.3f}, decode_ms = {timings.decode_ms:.3f}, "
          f"decode_tokens = {timings.decode_tokens}, decode_tps = {timings.decode_tps:.1f}", file=sys.stderr)
    if tokenizer is not None:
        print(tokenizer.decode(sequences[0], skip_special_tokens=True))
    else:
        print(" ".join(str(t) for t in sequences[0]))
    return 0


if __name__ == "__main__":
    try:
        raise SystemExit(main())
    except Exception as error:  # noqa: BLE001 - user-facing boundary, as runner.py:105-110
        print(f"runner.py: {error}", file=sys.stderr)
        raise SystemExit(1)
