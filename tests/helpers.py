"""Tiny configurations and small utilities shared by the tests."""
from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent

# Two tiny Llama configurations that differ in every size and option.
TINY_A = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=176,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
              vocab_size=256, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=64,
              tie_word_embeddings=False, eos_token_id=2, hidden_act="silu")
TINY_B = dict(architectures=["LlamaForCausalLM"], hidden_size=96, intermediate_size=256,
              num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=3, head_dim=16,
              vocab_size=384, rms_norm_eps=1e-6, rope_theta=500000.0, max_position_embeddings=128,
              tie_word_embeddings=True, eos_token_id=[5, 7], hidden_act="silu")
# A third one with a head size that is not the hidden size over the heads, MHA, and an odd vocabulary.
TINY_C = dict(architectures=["LlamaForCausalLM"], hidden_size=80, intermediate_size=104,
              num_hidden_layers=1, num_attention_heads=3, num_key_value_heads=3, head_dim=32,
              vocab_size=331, rms_norm_eps=3e-6, rope_theta=25000.0, max_position_embeddings=512,
              tie_word_embeddings=False, hidden_act="silu")
# Awkward sizes: a feed-forward width that is no multiple of 8, seven query heads on one KV head.
TINY_D = dict(architectures=["LlamaForCausalLM"], hidden_size=56, intermediate_size=90,
              num_hidden_layers=2, num_attention_heads=7, num_key_value_heads=1, head_dim=16,
              vocab_size=203, rms_norm_eps=1e-5, rope_theta=1000.0, max_position_embeddings=256,
              tie_word_embeddings=True, hidden_act="silu")
# Head size 64: the sizes at which the tcgen05 attention and its TMA cache gathers take over.
TINY_E = dict(architectures=["LlamaForCausalLM"], hidden_size=128, intermediate_size=136,
              num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1, head_dim=64,
              vocab_size=300, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=512,
              tie_word_embeddings=False, hidden_act="silu")
# Head size 208: above what the fused decode attention and the prefill kernels on tensor cores are built
# for, so the general kernels serve; two query heads on one KV head.
TINY_F = dict(architectures=["LlamaForCausalLM"], hidden_size=72, intermediate_size=120,
              num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1, head_dim=208,
              vocab_size=250, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=512,
              tie_word_embeddings=True, hidden_act="silu")
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "F": TINY_F}


def make_folder(folder, raw_config, seed, dtype=torch.float32):
    """A model folder with random weights stored in ``dtype`` (a torch dtype or its name)."""
    if isinstance(dtype, str):
        dtype = getattr(torch, dtype)
    from stratakv_b200.config import LlamaConfig
    from stratakv_b200.weights import write_random_model
    return write_random_model(folder, LlamaConfig.from_dict(raw_config), seed, dtype)


def random_tokens(vocab, length, seed):
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=generator).tolist()


def run_trace(model_dir, dtype, steps, out_dir, max_tokens, timeout=600, random_seed=None):
    """Run bin/trace_run on ``steps`` (a list of dicts); returns {step: array [wanted, vocab]}.
    ``random_seed``: no checkpoint is read; ``--random <model_dir>/config.json --seed`` draws the weights."""
    out_dir = Path(out_dir)
    text = "".join(json.dumps(s) + "\n" for s in steps)
    source = (["--model", str(model_dir)] if random_seed is None
              else ["--random", str(Path(model_dir) / "config.json"), "--seed", str(random_seed)])
    result = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), *source, "--dtype", dtype,
         "--out", str(out_dir), "--max-tokens", str(max_tokens)],
        input=text, capture_output=True, text=True, timeout=timeout)
    assert result.returncode == 0, result.stderr[-4000:]
    done = [line for line in result.stdout.splitlines() if line.startswith("done ")]
    assert [line.split()[1] for line in done] == [str(s["step"]) for s in steps], result.stdout
    vocab = json.loads((Path(model_dir) / "config.json").read_text())["vocab_size"]
    logits = {}
    for s in steps:
        wanted = sum(len(e.get("want", [])) for e in s["entries"])
        path = out_dir / f"{s['step']}.f32"
        if wanted:
            logits[s["step"]] = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
        else:
            assert not path.exists()
    return logits


def stored_dtype(dtype):
    """Test folders hold their weights in the dtype the engine computes in, so that the plain
    implementation (which widens whatever is stored to float32) works on the very same values."""
    return torch.bfloat16 if dtype in ("bfloat16", torch.bfloat16) else torch.float32


def tolerance(dtype, ref=None, noise=0.025):
    """(rtol, atol) for logits against the plain float32 implementation on the same stored weights.

    float32: rounding of sums taken in another order.  bfloat16: the engine rounds the inputs of every
    projection and the cache to 8 bits of mantissa, which moves a logit by a fraction of the logits'
    spread: measured at most 0.017 of their standard deviation over the tiny configurations (whole
    prompts, decoding, batches), while ONE wrong cache row among a hundred moves some logit by 0.05 or
    more of it.  So the allowance is ``noise`` = 0.025 standard deviations of ``ref``, absolute: tight
    enough that a single misplaced key fails (tests/test_engine_gpu.py shows it by making one)."""
    if dtype in ("float32", torch.float32):
        return 1e-4, 2e-5
    if ref is None:
        raise ValueError("the bfloat16 tolerance is a fraction of the reference logits' spread")
    spread = float(np.asarray(ref, dtype=np.float64).std())
    return 0.0, noise * spread
