"""bin/trace_run as a user runs it: a subprocess fed steps on standard input."""
import numpy as np
import pytest

import plain_llama
from helpers import TINY, make_folder, random_tokens, run_trace, tolerance

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_three_ways(tmp_path, dtype, name):
    folder = make_folder(tmp_path / "model", TINY[name], seed=21, dtype=dtype)
    config, weights = plain_llama.load_folder(folder)
    vocab = TINY[name]["vocab_size"]
    requests = {f"r{i}": random_tokens(vocab, n, seed=200 + i) for i, n in enumerate((40, 33, 75))}
    ref = {k: plain_llama.logits_of(config, weights, v).numpy() for k, v in requests.items()}
    steps, expect = [], {}
    # (1) each request alone and whole
    for ident, tokens in requests.items():
        expect[len(steps)] = ref[ident]
        steps.append({"step": len(steps), "entries": [{"id": "w" + ident, "tokens": tokens,
                                                       "want": list(range(len(tokens)))}], "end": ["w" + ident]})
    # (2) the last 32 tokens one by one
    for ident, tokens in requests.items():
        head = len(tokens) - 32
        steps.append({"step": len(steps), "entries": [{"id": "d" + ident, "tokens": tokens[:head], "want": []}],
                      "end": []})
        for p in range(head, len(tokens)):
            expect[len(steps)] = ref[ident][p:p + 1]
            steps.append({"step": len(steps), "entries": [{"id": "d" + ident, "tokens": [tokens[p]], "want": [0]}],
                          "end": ["d" + ident] if p == len(tokens) - 1 else []})
    # (3) a batch of unequal lengths; the shorter requests end earlier; twice, so slots are used again
    for round_ in range(2):
        names = list(requests)
        prompt = {k: len(requests[k]) - 10 - 3 * i for i, k in enumerate(names)}
        expect[len(steps)] = np.stack([ref[k][prompt[k] - 1] for k in names])
        steps.append({"step": len(steps), "end": [], "entries": [
            {"id": f"b{round_}{k}", "tokens": requests[k][:prompt[k]], "want": [prompt[k] - 1]} for k in names]})
        fed = dict(prompt)
        live = list(names)
        while live:
            ending = [k for k in live if fed[k] + 1 >= len(requests[k])]
            expect[len(steps)] = np.stack([ref[k][fed[k]] for k in live])
            steps.append({"step": len(steps), "end": [f"b{round_}{k}" for k in ending], "entries": [
                {"id": f"b{round_}{k}", "tokens": [requests[k][fed[k]]], "want": [0]} for k in live]})
            for k in live:
                fed[k] += 1
            live = [k for k in live if k not in ending]
    got = run_trace(folder, dtype, steps, tmp_path / "out", max_tokens=64 * 2 * 3)
    assert set(got) == set(expect)
    for step, want in expect.items():
        rtol, atol = tolerance(dtype, want)
        np.testing.assert_allclose(got[step], want, rtol=rtol, atol=atol, err_msg=f"step {step}")


def test_replay_with_random_weights_equals_the_folder_of_the_same_seed(tmp_path):
    """``--random CONFIG --seed S`` draws the tensors that the random-weights mode writes to a folder for the same
    seed, so a replay without a checkpoint gives the logits of a replay of that folder, bit for bit."""
    folder = make_folder(tmp_path / "model", TINY["B"], seed=33, dtype="bfloat16")
    tokens = random_tokens(TINY["B"]["vocab_size"], 20, seed=4)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:12], "want": [0, 11]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[12:13], "want": [0]}], "end": ["a"]}]
    from_folder = run_trace(folder, "bfloat16", steps, tmp_path / "a", max_tokens=64)
    drawn = run_trace(folder, "bfloat16", steps, tmp_path / "b", max_tokens=64, random_seed=33)
    other = run_trace(folder, "bfloat16", steps, tmp_path / "c", max_tokens=64, random_seed=34)
    for step in (0, 1):
        assert np.array_equal(from_folder[step], drawn[step])
        assert not np.array_equal(from_folder[step], other[step])
