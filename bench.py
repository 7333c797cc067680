"""Benchmark: decode tokens a second and prefill tokens a second on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]

The default run has the layer sizes of the TinyLlama-1.1B shape (22 layers,
hidden 2048, 32 heads, 4 KV heads, head size 64, feed-forward 5632, vocabulary
32000) with random bfloat16 weights, a batch of 8 and a context that ends at
2,048 tokens.  A "step" is one decode step of the whole batch.  It prints one
JSON line:

  value        decoded tokens a second, timed on the device around K steps
  e2e          the same through the Python entry point (``Engine.generate``):
               token ids go in from pinned host memory and come back to the
               host every step
  prefill      one 2,048-token prompt: tokens a second, ms, and the fraction
               of the bf16 tensor peak its FLOPs reach
  roofline     the decode step against HBM: bytes it must read (every weight
               once, plus the cache of the live requests) over its time
  points       decode tokens a second at batch 1 and 64

Peaks come from MEASURED_PEAKS.json beside this file when it exists.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# The TinyLlama-1.1B shape (sizes only; weights are random).
TINYLLAMA = dict(architectures=["LlamaForCausalLM"], hidden_size=2048, intermediate_size=5632,
                 num_hidden_layers=22, num_attention_heads=32, num_key_value_heads=4, head_dim=64,
                 vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=2048,
                 tie_word_embeddings=False, hidden_act="silu")
# Larger shapes of the same family (sizes only), for --shape.
LLAMA2_7B = dict(TINYLLAMA, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32,
                 num_key_value_heads=32, head_dim=128, vocab_size=32000, max_position_embeddings=4096)
LLAMA3_8B = dict(TINYLLAMA, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                 num_key_value_heads=8, head_dim=128, vocab_size=128256, rope_theta=500000.0,
                 max_position_embeddings=8192)
SHAPES = {"tinyllama-1.1b": TINYLLAMA, "llama2-7b": LLAMA2_7B, "llama3-8b": LLAMA3_8B}
# Generation workloads of the larger shapes: requests that start together with prompt lengths drawn uniformly
# (seeded) from a range, a number of new tokens each, greedy or sampled.
WORKLOADS = {
    "llama2-7b": dict(shape="llama2-7b", batch=8, prompt_range=(256, 2048), new_tokens=256, temperature=0.0),
    "llama3-8b": dict(shape="llama3-8b", batch=64, prompt_range=(128, 1024), new_tokens=128, temperature=0.8),
    "tinyllama-1.1b": dict(shape="tinyllama-1.1b", batch=8, prompt_range=(256, 2048), new_tokens=256, temperature=0.0),
}
CONTEXT = 2048
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "source": "measured"}
        except (ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index=0):
        self.samples, self.process, self.thread = [], None, None
        self.device_index = device_index

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.process.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def stop(self):
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        clocks, reasons, max_clock = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for parts in self.samples:
            try:
                clocks.append(float(parts[0]))
                max_clock = float(parts[1])
            except ValueError:
                continue
            for name, value in zip(names, parts[2:]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


def make_engine(layers: int, max_tokens: int, max_batch: int, shape=None):
    import torch
    from stratakv_b200 import Engine, EngineConfig, LlamaConfig
    raw = dict(shape or TINYLLAMA, num_hidden_layers=layers)
    config = LlamaConfig.from_dict(raw)
    engine_config = EngineConfig(max_tokens=max_tokens, dtype="bfloat16", max_batch=max_batch, max_context=max_tokens)
    from stratakv_b200.config.registry import resolve_architecture
    from stratakv_b200.engine.model import expected_tensors
    from stratakv_b200.weights import random_tensors
    spec = resolve_architecture(config.architecture).build_spec(config)
    tensors = random_tensors(expected_tensors(spec), seed=0, dtype=torch.bfloat16, device="cuda")
    engine = Engine(spec, tensors, engine_config, verbose=False)
    engine.model_config = config
    return engine, config


def random_ids(count, vocab, seed):
    import torch
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count,), generator=generator).tolist()


def fill_context(engine, batch, context, vocab):
    """Open ``batch`` sequences and prefill each with ``context`` random tokens."""
    from stratakv_b200 import StepEntry
    slots = []
    for index in range(batch):
        slot = engine.open_sequence()
        engine.step([StepEntry(slot, random_ids(context, vocab, 1000 + index), [])])
        slots.append(slot)
    return slots


def time_decode(engine, batch, start_context, steps, warmup, vocab):
    """Device time of ``steps`` decode steps of ``batch`` sequences (ms per step), sampling included."""
    import torch
    from stratakv_b200.sampling import Sampler, SamplingParams
    from stratakv_b200 import StepEntry
    slots = fill_context(engine, batch, start_context, vocab)
    sampler = Sampler(engine.rt.kernels(), SamplingParams(), engine.model.flags)
    chosen = torch.empty(batch, dtype=torch.int32, device=engine.device)
    entries = [StepEntry(slot, [token], [0]) for slot, token in zip(slots, random_ids(batch, vocab, 7))]

    def one_step():
        sampler.sample(engine.step(entries), None, None, chosen)

    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    launches_before = engine.launch_count()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        one_step()
    end.record()
    torch.cuda.synchronize()
    launches = engine.launch_count() - launches_before
    final_context = engine.cache.length(slots[0])
    for slot in slots:
        engine.close_sequence(slot)
    return begin.elapsed_time(end) / steps, launches, final_context


def time_e2e(engine, batch, start_context, steps, vocab):
    """Tokens a second through ``Engine.generate``: host token ids in, host token ids out, every step."""
    prompts = [random_ids(start_context, vocab, 2000 + i) for i in range(batch)]
    engine.generate(prompts[:1], 4, ignore_eos=True)                          # warm-up of both step kinds
    output = engine.generate(prompts, steps + 1, ignore_eos=True)
    timings = output.timings
    return timings, engine.last_step_io_bytes()


def time_prefill(engine, tokens, vocab, repeats=3):
    import torch
    from stratakv_b200 import StepEntry
    import gc
    times = []
    for repeat in range(repeats + 1):
        slot = engine.open_sequence()
        ids = random_ids(tokens, vocab, 3000 + repeat)
        gc.collect()                                  # a collection of the generation runs' garbage inside the
        gc.disable()                                  # timed step would be host noise, not the step's time
        try:
            torch.cuda.synchronize()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            engine.step([StepEntry(slot, ids, [tokens - 1])])
            end.record()
            torch.cuda.synchronize()
        finally:
            gc.enable()
        engine.close_sequence(slot)
        if repeat:                                    # the first run is the warm-up
            times.append(begin.elapsed_time(end))
    return statistics.median(times)


def prefill_flops(config, tokens):
    per_token = 2 * (config.hidden_size * (config.q_dim + 2 * config.kv_dim) + config.q_dim * config.hidden_size
                     + 3 * config.hidden_size * config.intermediate_size)
    linear = config.num_hidden_layers * per_token * tokens + 2 * config.hidden_size * config.vocab_size
    attention = config.num_hidden_layers * 4 * config.num_attention_heads * config.head_dim * tokens * (tokens + 1) // 2
    return linear + attention


REFERENCE_SOURCE = Path("/root/reference")
REFERENCE_BUILD = ROOT / "baseline" / "_ref" / "build"


def reference_cli():
    """Path of the reference's own ``stratakv_cli``, built unmodified out of tree with CMake for sm_100
    (its architecture is a cache variable, CMakeLists.txt:31-33).  Its Release configuration hands MSVC
    options to nvcc's host compiler on every platform (CMakeLists.txt:104-113), so the same optimisation
    flags are given on the command line with no build type instead.  Returns (path, None) or (None, why)."""
    import shutil
    binary = REFERENCE_BUILD / "stratakv_cli"
    if binary.is_file():
        return binary, None
    if not (REFERENCE_SOURCE / "CMakeLists.txt").is_file():
        return None, "the reference's source tree is not on this machine and baseline/_ref/build holds no stratakv_cli"
    cmake, nvcc = shutil.which("cmake"), shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not cmake or not Path(nvcc).is_file():
        return None, "cmake or nvcc is missing: the reference cannot be built here"
    cuda_include = str(Path(nvcc).resolve().parent.parent / "include")
    configure = [cmake, "-S", str(REFERENCE_SOURCE), "-B", str(REFERENCE_BUILD), "-G", "Ninja", "-DSTRATAKV_CUDA=ON",
                 "-DCMAKE_CUDA_ARCHITECTURES=100", "-DBUILD_TESTING=OFF", "-DCMAKE_BUILD_TYPE=",
                 f"-DCMAKE_CUDA_COMPILER={nvcc}", f"-DCMAKE_CXX_FLAGS=-O3 -mavx2 -mfma -DNDEBUG -I{cuda_include}",
                 "-DCMAKE_CUDA_FLAGS=-O3 --use_fast_math -Xptxas=-O3 -DNDEBUG"]
    for command in (configure, [cmake, "--build", str(REFERENCE_BUILD), "--target", "stratakv_cli", "-j", "8"]):
        done = subprocess.run(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if done.returncode != 0:
            return None, "building the reference with CMake failed: " + done.stdout.strip().splitlines()[-1][:200]
    return (binary, None) if binary.is_file() else (None, "the CMake build left no stratakv_cli")


def reference_arm(args) -> int:
    """The unmodified reference on the same workload, through its stock path: ``stratakv_cli
    <model.safetensors> <max_new_tokens> <ids...>`` (src/cli.cpp:179-322), one sequence per process, the way
    its own benchmark.py drives it.  The reference runs one sequence at a time and takes a prompt one token
    per step, so the batch of 8 becomes 8 runs one after another.  Its only timer covers prompt and
    decoding together (src/generation/generator.cpp:635, 800-801), so each sequence runs twice: with 1 new
    token and with 1 + steps; the difference of the two ``gen_ms`` is the time of ``steps`` decode steps
    whose context ends at 2,048.  Nothing of this repo's kernels or engine is used; only the safetensors
    writer makes the random checkpoint."""
    import re
    import shutil
    import tempfile
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.shape != "tinyllama-1.1b":
        print(json.dumps({"impl": "reference", "unavailable": "the reference arm runs the headline shape only"}))
        return 0
    cli, why = reference_cli()
    if cli is None:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    import torch
    from stratakv_b200.config import LlamaConfig
    from stratakv_b200.weights import write_random_model
    steps, sequences = max(args.steps, 1), args.batch
    shape = dict(SHAPES[args.shape], num_hidden_layers=args.layers or SHAPES[args.shape]["num_hidden_layers"])
    prompt_length = CONTEXT - steps
    work = Path(tempfile.mkdtemp(prefix="skv_reference_"))
    pattern = re.compile(r"\[TIMING\].*?load_ms = ([0-9.eE+-]+), gen_ms = ([0-9.eE+-]+), tokens = (\d+)")

    def run(prompt, new_tokens):
        command = [str(cli), str(work / "model.safetensors"), str(new_tokens)] + [str(t) for t in prompt]
        try:
            done = subprocess.run(command, capture_output=True, text=True, timeout=900)
        except subprocess.TimeoutExpired:
            raise RuntimeError("the reference's stratakv_cli did not finish one sequence within 900 s")
        found = pattern.search(done.stderr)
        if done.returncode != 0 or not found:
            raise RuntimeError(f"the reference's stratakv_cli exited with {done.returncode}: "
                               + (done.stderr.strip().splitlines() or ["no output"])[-1][:200])
        return float(found.group(2)), int(found.group(3)), float(found.group(1))

    try:
        write_random_model(work, LlamaConfig.from_dict(shape), seed=0, dtype=torch.bfloat16)
        sampler = ClockSampler()
        sampler.start()
        decode_ms, decoded, per_sequence, prompt_ms, load_ms = 0.0, 0, [], [], []
        for index in range(sequences):
            prompt = random_ids(prompt_length, shape["vocab_size"], 1000 + index)
            short_ms, short_tokens, _ = run(prompt, 1)
            long_ms, long_tokens, loaded = run(prompt, 1 + steps)
            decode_ms += long_ms - short_ms
            decoded += long_tokens - short_tokens
            per_sequence.append((long_tokens - short_tokens) * 1000.0 / max(long_ms - short_ms, 1e-9))
            prompt_ms.append(short_ms)
            load_ms.append(loaded)
        clocks = sampler.stop()
    except (RuntimeError, OSError) as error:
        print(json.dumps({"impl": "reference", "unavailable": str(error)}))
        return 0
    finally:
        shutil.rmtree(work, ignore_errors=True)
    if decoded <= 0 or decode_ms <= 0:
        print(json.dumps({"impl": "reference", "unavailable": "the reference generated no tokens beyond the first "
                          "(its greedy choice hit its end-of-sequence id 2)"}))
        return 0
    value = decoded * 1000.0 / decode_ms
    vocab_bytes = shape["vocab_size"] * 4
    print(json.dumps({
        "metric": f"decode tokens/s ({args.shape} shape, bf16, batch {sequences}, context {CONTEXT})",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": max(args.warmup, 3),
        "ms_per_step": sequences * 1000.0 / value, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random N(0,0.02) weights, uniform random token ids",
        "config": {"model": f"{args.shape} shape", "layers": shape["num_hidden_layers"],
                   "layers_of_model": SHAPES[args.shape]["num_hidden_layers"], "hidden": shape["hidden_size"],
                   "heads": shape["num_attention_heads"], "kv_heads": shape["num_key_value_heads"],
                   "head_dim": shape["head_dim"], "ffn": shape["intermediate_size"], "vocab": shape["vocab_size"],
                   "global_batch": sequences, "seq_len": CONTEXT, "context_at_end": CONTEXT,
                   "parallelism": "single GPU, one sequence at a time (the reference's stock path)",
                   "timing": "difference of gen_ms of two stratakv_cli runs per sequence (1 and 1+steps new tokens)",
                   "warm": f"the {prompt_length} prompt tokens, which the reference runs one per step, precede the timed steps",
                   "cache_block": 16, "l2": "inputs larger than L2 (weights 2.1 GB per token)"},
        "clocks": clocks,
        # its stock path is end to end already: token ids come from the host, every step copies the logits to
        # the host and samples there
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": vocab_bytes,
                "prefill_ms": statistics.median(prompt_ms), "load_ms": statistics.median(load_ms)},
        "prefill": {"value": prompt_length * 1000.0 / statistics.median(prompt_ms), "tokens": prompt_length,
                    "ms": statistics.median(prompt_ms), "note": "the reference takes a prompt one token per step"},
        "per_sequence_tokens_per_s": per_sequence, "gpu_launches": None, "impl": "reference"}))
    return 0


def workload_arm(args) -> int:
    """A whole workload through the Python entry point: ``Engine.generate`` on host token ids, every chosen token
    read back to the host each step.  Reports decode tokens a second, the time of a decode step, the prompt step's
    tokens a second, and the decode step against HBM from the bytes that are live (every weight once per step, and the
    cache of the sequences at their mean length)."""
    import random
    import torch
    from stratakv_b200.sampling import SamplingParams
    if not torch.cuda.is_available():
        print("bench.py: no CUDA device")
        return 1
    work = WORKLOADS[args.workload]
    shape = SHAPES[work["shape"]]
    layers = args.layers or shape["num_hidden_layers"]
    batch, new_tokens = work["batch"], work["new_tokens"]
    rng = random.Random(0)
    lengths = [rng.randint(*work["prompt_range"]) for _ in range(batch)]
    prompts = [random_ids(length, shape["vocab_size"], 5000 + i) for i, length in enumerate(lengths)]
    max_tokens = sum(-(-(length + new_tokens) // 64) * 64 for length in lengths) + 64
    engine, config = make_engine(layers, max_tokens, batch, shape)
    params = SamplingParams(temperature=work["temperature"], seed=1)
    # warm-up: the same requests once (kernels loaded, buffers sized, decode graphs of every table width captured)
    engine.generate(prompts, new_tokens, params, ignore_eos=True)
    torch.cuda.synchronize()
    sampler = ClockSampler()
    sampler.start()
    output = engine.generate(prompts, new_tokens, params, ignore_eos=True)
    clocks = sampler.stop()
    t = output.timings
    steps = new_tokens - 1                                   # the last chosen token is not fed
    ms_per_step = t.decode_ms / steps
    peak = peaks()
    weight_bytes = engine.model.weight_bytes()
    mean_context = sum(lengths) / batch + new_tokens / 2
    kv_bytes = batch * mean_context * engine.cache.bytes_per_token()
    achieved = (weight_bytes + kv_bytes) / (ms_per_step * 1e-3) / 1e9
    io_bytes = engine.last_step_io_bytes()
    value = t.decode_tps
    print(json.dumps({
        "metric": f"decode tokens/s ({args.workload} workload through Engine.generate, bf16, batch {batch})",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": steps, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random N(0,0.02) weights, uniform random token ids, seeded prompt lengths",
        "config": {"model": f"{work['shape']} shape", "layers": layers, "layers_of_model": shape["num_hidden_layers"],
                   "hidden": config.hidden_size, "heads": config.num_attention_heads,
                   "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim, "ffn": config.intermediate_size,
                   "vocab": config.vocab_size, "global_batch": batch, "prompt_min": work["prompt_range"][0],
                   "prompt_max": work["prompt_range"][1], "prompt_tokens": sum(lengths), "new_tokens": new_tokens,
                   "temperature": work["temperature"], "parallelism": "single GPU",
                   "l2": f"inputs larger than L2 (weights {weight_bytes / 1e9:.1f} GB per step)"},
        "clocks": clocks,
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": io_bytes[0], "d2h_bytes_per_step": io_bytes[1],
                "prefill_ms": t.prefill_ms},
        "prefill": {"value": t.prefill_tokens * 1000.0 / t.prefill_ms, "tokens": t.prefill_tokens, "ms": t.prefill_ms,
                    "frac": prefill_flops_of(config, lengths) / (t.prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12),
                    "of": peak["source"]},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peak["hbm_gbs"], "of": peak["source"], "weight_bytes": weight_bytes,
                     "kv_bytes": int(kv_bytes)},
        "gpu_launches": engine.launch_count(), "impl": "ours"}))
    return 0


def prefill_flops_of(config, lengths):
    """FLOPs of one step that runs prompts of these lengths (the head runs on one row per prompt)."""
    per_token = 2 * (config.hidden_size * (config.q_dim + 2 * config.kv_dim) + config.q_dim * config.hidden_size
                     + 3 * config.hidden_size * config.intermediate_size)
    linear = config.num_hidden_layers * per_token * sum(lengths) + 2 * config.hidden_size * config.vocab_size * len(lengths)
    attention = sum(config.num_hidden_layers * 4 * config.num_attention_heads * config.head_dim * n * (n + 1) // 2
                    for n in lengths)
    return linear + attention


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (both are reported)")
    parser.add_argument("--shape", default="tinyllama-1.1b", choices=sorted(SHAPES))
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64 and the prefill")
    parser.add_argument("--context", type=int, default=CONTEXT, help="context at which the timed decode steps end")
    parser.add_argument("--workload", choices=sorted(WORKLOADS),
                        help="a whole generation workload through Engine.generate instead of the step benchmark")
    args = parser.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.workload:
        return workload_arm(args)
    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)

    import torch
    if not torch.cuda.is_available():
        print("bench.py: no CUDA device")
        return 1
    shape = SHAPES[args.shape]
    if args.layers is None:
        args.layers = shape["num_hidden_layers"]
    vocab = shape["vocab_size"]
    context = args.context
    start_context = context - steps - warmup                 # the timed steps end at the named context
    if start_context < 1:
        print(f"bench.py: --steps plus --warmup must stay below the context of {context}")
        return 1
    biggest = 64 if not args.skip_points else args.batch
    max_tokens = max(biggest * (context + 64), PREFILL_TOKENS + 64)
    engine, config = make_engine(args.layers, max_tokens, max(biggest, args.batch), shape)
    peak = peaks()

    sampler = ClockSampler()
    sampler.start()
    ms_per_step, launches, final_context = time_decode(engine, args.batch, start_context, steps, warmup, vocab)
    clocks = sampler.stop()
    value = args.batch * 1000.0 / ms_per_step

    timings, io_bytes = time_e2e(engine, args.batch, start_context, steps, vocab)
    e2e = {"value": timings.decode_tps, "unit": "tokens/s", "h2d_bytes_per_step": io_bytes[0],
           "d2h_bytes_per_step": io_bytes[1], "prefill_ms": timings.prefill_ms}

    weight_bytes = engine.model.weight_bytes()
    mean_context = final_context - steps / 2
    kv_bytes = args.batch * mean_context * engine.cache.bytes_per_token()
    achieved = (weight_bytes + kv_bytes) / (ms_per_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peak["hbm_gbs"], "of": peak["source"], "weight_bytes": weight_bytes,
                "kv_bytes": int(kv_bytes)}

    result = {
        "metric": f"decode tokens/s ({args.shape} shape, bf16, batch {args.batch}, context {context})",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random N(0,0.02) weights, uniform random token ids",
        "config": {"model": f"{args.shape} shape", "layers": args.layers, "layers_of_model": shape["num_hidden_layers"],
                   "hidden": config.hidden_size, "heads": config.num_attention_heads,
                   "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
                   "ffn": config.intermediate_size, "vocab": config.vocab_size, "global_batch": args.batch,
                   "seq_len": context, "context_at_end": final_context, "parallelism": "single GPU",
                   "cache_block": engine.cache.block_size, "l2": f"inputs larger than L2 (weights {engine.model.weight_bytes() / 1e9:.1f} GB per step)"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "roofline": roofline, "impl": "ours",
    }
    if not args.skip_points:
        prefill_ms = time_prefill(engine, PREFILL_TOKENS, vocab)
        flops = prefill_flops(config, PREFILL_TOKENS)
        result["prefill"] = {"value": PREFILL_TOKENS * 1000.0 / prefill_ms, "tokens": PREFILL_TOKENS,
                             "ms": prefill_ms, "frac": flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12),
                             "of": peak["source"]}
        points = {}
        for batch in (1, 64):
            ms, _, _ = time_decode(engine, batch, start_context, steps, warmup, vocab)
            points[f"decode_b{batch}"] = batch * 1000.0 / ms
        result["points"] = points
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
