"""Generation through the entry points on the GPU: greedy tokens against the plain model,
stop tokens and early finishers, batched equals solo, long decoding, the first tokens of
a sequence, the command line."""
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama
from helpers import ROOT, TINY, make_folder, random_tokens, stored_dtype, tolerance

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("gen_models")
    made = {name: make_folder(root / name, raw, seed=31 + i) for i, (name, raw) in enumerate(TINY.items())}
    # the same weights stored in bfloat16, for runs that compute in bfloat16 (the plain model then sees the same values)
    made.update({(name, "bfloat16"): make_folder(root / (name + "_bf16"), raw, seed=31 + i, dtype="bfloat16")
                 for i, (name, raw) in enumerate(TINY.items())})
    made.update({(name, "float32"): made[name] for name in TINY})
    return made


def engine_for(folder, dtype, max_tokens=4096):
    from stratakv_b200 import Engine, EngineConfig
    return Engine.from_folder(folder, EngineConfig(max_tokens=max_tokens, dtype=dtype, max_context=max_tokens), verbose=False)


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_float32_equals_the_plain_model(folders, name):
    config, weights = plain_llama.load_folder(folders[name])
    engine = engine_for(folders[name], "float32")
    lengths, budget = ((5, 9, 13), 8) if name == "A" else ((1, 7, 16, 31), 12)
    prompts = [random_tokens(TINY[name]["vocab_size"], n, seed=n) for n in lengths]
    out = engine.generate(prompts, budget, ignore_eos=True)
    for prompt, sequence in zip(prompts, out.sequences):
        assert sequence == plain_llama.greedy(config, weights, prompt, budget)
    assert engine.cache.all_free()
    assert out.timings.decode_tokens == len(prompts) * (budget - 1)


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_bfloat16_picks_a_top_token(folders, name):
    """In bfloat16 near-ties may fall the other way: every chosen token must score within
    the bfloat16 tolerance of the plain model's best, given the same tokens before it."""
    config, weights = plain_llama.load_folder(folders[name, "bfloat16"])
    engine = engine_for(folders[name, "bfloat16"], "bfloat16")
    prompts = [random_tokens(TINY[name]["vocab_size"], n, seed=n) for n in (4, 19)]
    out = engine.generate(prompts, 10, ignore_eos=True)
    for prompt, sequence in zip(prompts, out.sequences):
        assert sequence[:len(prompt)] == prompt and len(sequence) == len(prompt) + 10
        logits = plain_llama.logits_of(config, weights, sequence[:-1]).numpy()
        for position in range(len(prompt) - 1, len(sequence) - 1):
            row = logits[position]
            _, atol = tolerance("bfloat16", row)
            assert row[sequence[position + 1]] >= row.max() - 2 * atol


def test_stop_tokens_and_early_finishers(folders):
    config, weights = plain_llama.load_folder(folders["B"])
    engine = engine_for(folders["B"], "float32")
    prompts = [random_tokens(384, n, seed=70 + n) for n in (3, 12, 6)]
    free_run = [plain_llama.greedy(config, weights, p, 12) for p in prompts]
    stop = free_run[1][len(prompts[1]) + 2]                   # the third token request 1 generates
    expected = [plain_llama.greedy(config, weights, p, 12, stop_ids=(stop,)) for p in prompts]
    out = engine.generate(prompts, 12, stop_ids=[stop])
    assert out.sequences == expected
    assert len(expected[1]) <= len(prompts[1]) + 3 and expected[1][-1] == stop
    assert engine.cache.all_free()
    # the model's own eos ids are the default; a prompt that ends in one comes back unchanged
    assert engine.generate([[9, 5]], 4).sequences == [[9, 5]]
    assert engine.generate([[9, 8]], 0).sequences == [[9, 8]]


def test_batches_one_after_another_reuse_slots(folders):
    from stratakv_b200 import Engine, EngineConfig
    config, weights = plain_llama.load_folder(folders["A"])
    engine = Engine.from_folder(folders["A"], EngineConfig(max_tokens=3 * 64, dtype="float32", max_batch=3),
                                verbose=False)
    prompts = [random_tokens(256, 3 + 5 * i, seed=i) for i in range(7)]
    out = engine.generate(prompts, [2 + i for i in range(7)], ignore_eos=True)
    assert out.timings.batches == 3
    for i, (prompt, sequence) in enumerate(zip(prompts, out.sequences)):
        assert sequence == plain_llama.greedy(config, weights, prompt, 2 + i)
    assert engine.cache.all_free()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sampling_batched_equals_solo_and_is_seeded(folders, dtype):
    from stratakv_b200.sampling import SamplingParams
    engine = engine_for(folders["B"], dtype)
    prompts = [random_tokens(384, n, seed=n) for n in (2, 9, 30)]
    params = SamplingParams(temperature=0.8, top_k=40, top_p=0.95, seed=7)
    together = engine.generate(prompts, 16, params, ignore_eos=True).sequences
    again = engine.generate(prompts, 16, params, ignore_eos=True).sequences
    assert together == again
    if dtype == "float32":
        for i, prompt in enumerate(prompts):
            alone = engine.generate([prompt], 16, params, ignore_eos=True, streams=[i]).sequences[0]
            assert alone == together[i]
    other = engine.generate(prompts, 16, SamplingParams(0.8, 40, 0.95, seed=8), ignore_eos=True).sequences
    assert other != together


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, dtype):
    """Four hundred tokens one by one (many cache blocks), checked against whole-sequence logits."""
    from stratakv_b200 import StepEntry
    config, weights = plain_llama.load_folder(folders["C", dtype])
    engine = engine_for(folders["C", dtype], dtype)
    tokens = random_tokens(331, 400, seed=3)
    ref = plain_llama.logits_of(config, weights, tokens).numpy()
    rtol, atol = tolerance(dtype, ref)
    slot = engine.open_sequence()
    for position, token in enumerate(tokens):
        got = engine.step([StepEntry(slot, [token], [0])])
        if position < 4 or position % 37 == 0 or position in (63, 64, 65, 127, 128, 399):
            np.testing.assert_allclose(got.float().cpu().numpy()[0], ref[position], rtol=rtol, atol=atol,
                                       err_msg=f"position {position}")
    engine.close_sequence(slot)


def test_command_line(folders):
    config, weights = plain_llama.load_folder(folders["A"])
    prompt = random_tokens(256, 6, seed=1)
    command = [sys.executable, str(ROOT / "bin" / "stratakv_cli"), "--dtype", "float32", str(folders["A"]), "5",
               *map(str, prompt[:3]), "--ignore-eos", *map(str, prompt[3:])]
    result = subprocess.run(command, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr
    assert [int(t) for t in result.stdout.split()] == plain_llama.greedy(config, weights, prompt, 5)
    assert "[TIMING] load_ms = " in result.stderr and "pure_decode_tps = " in result.stderr
    bad = subprocess.run([sys.executable, str(ROOT / "bin" / "stratakv_cli"), "--frobnicate", "x", "1", "2"],
                         capture_output=True, text=True, timeout=120)
    assert bad.returncode == 1 and "unknown option: --frobnicate" in bad.stderr
    assert subprocess.run([sys.executable, str(ROOT / "bin" / "stratakv_cli")], capture_output=True).returncode == 2


def test_command_line_with_random_weights(tmp_path):
    """--random CONFIG.json: no checkpoint; the same weights as the folder that the writer makes from the
    same configuration and seed, so the plain implementation can check the tokens."""
    import json
    from stratakv_b200.weights import random_init
    config_file = tmp_path / "config.json"
    config_file.write_text(json.dumps(TINY["B"]))
    assert random_init.main([str(config_file), str(tmp_path / "model"), "--seed", "9", "--dtype", "float32"]) == 0
    config, weights = plain_llama.load_folder(tmp_path / "model")
    prompt = random_tokens(TINY["B"]["vocab_size"], 5, seed=4)
    command = [sys.executable, str(ROOT / "bin" / "stratakv_cli"), "--dtype", "float32", "--random", str(config_file),
               "--weights-seed", "9", "--block-size", "16", "--ignore-eos", "6", *map(str, prompt)]
    result = subprocess.run(command, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr
    assert [int(t) for t in result.stdout.split()] == plain_llama.greedy(config, weights, prompt, 6)


def test_python_entry_point(folders):
    from stratakv_b200.runner import run
    config, weights = plain_llama.load_folder(folders["A"])
    prompt = random_tokens(256, 7, seed=2)
    sequences, timings, engine = run(folders["A"], [prompt], max_new_tokens=6, temp=0.0, dtype="float32",
                                     ignore_eos=True)
    assert sequences == [plain_llama.greedy(config, weights, prompt, 6)]
    assert timings.decode_tokens == 5 and engine.cache.all_free()


@pytest.mark.parametrize("name", ["B", "E"])
def test_many_batches_twice_give_the_same_tokens(folders, name):
    """Batches of many sizes (up to 24, so every projection kernel takes part), greedy and sampled, with
    stop tokens and budgets that end requests early: nothing is left held afterwards, no kernel raises
    a flag, and a second engine given the same requests returns the same tokens (no kernel's result
    depends on timing)."""
    import random
    from stratakv_b200 import Engine, EngineConfig
    from stratakv_b200.sampling import SamplingParams
    vocab = TINY[name]["vocab_size"]

    def run():
        rng = random.Random(7)
        engine = Engine.from_folder(folders[name], EngineConfig(max_tokens=4096, dtype="bfloat16", block_size=16, max_context=4096),
                                    verbose=False)
        outputs = []
        for round_ in range(8):
            count = rng.choice([1, 3, 8, 9, 13, 17, 24])
            prompts = [random_tokens(vocab, rng.randint(1, 90), seed=rng.randint(0, 10 ** 6)) for _ in range(count)]
            budgets = [rng.randint(0, 30) for _ in range(count)]
            params = SamplingParams() if round_ % 3 else SamplingParams(temperature=0.9, top_k=20, top_p=0.9, seed=round_)
            stop = [rng.randrange(vocab) for _ in range(6)]
            outputs.append(engine.generate(prompts, budgets, params, stop_ids=stop).sequences)
            assert engine.cache.all_free()
        return outputs

    assert run() == run()
