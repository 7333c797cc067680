"""The generation loop's decisions, on a scripted engine (no GPU, no model)."""
import pytest
import torch

from stratakv_b200.cache import KVCache
from stratakv_b200.engine.generate import RequestError, generate, plan_batches
from stratakv_b200.parts.base import CacheRequest


class ScriptedEngine:
    """Next token = (last token + 1) mod vocab; records every step."""

    class Spec:
        vocab_size = 50

    def __init__(self, blocks=8, slots=4, block_size=16):
        self.spec = self.Spec()
        self.cache = KVCache([CacheRequest("kv", 1, 16)], blocks, block_size, slots, torch.float32, "cpu")
        self.steps = []

    def open_sequence(self):
        return self.cache.acquire()

    def close_sequence(self, slot):
        self.cache.release(slot)

    def step(self, entries):
        self.cache.reserve({e.slot: self.cache.length(e.slot) + len(e.tokens) for e in entries})
        self.steps.append([(e.slot, list(e.tokens), list(e.want)) for e in entries])
        logits = torch.zeros(len(entries), self.spec.vocab_size)
        for row, e in enumerate(entries):
            assert list(e.want) == [len(e.tokens) - 1]
            logits[row, (e.tokens[-1] + 1) % self.spec.vocab_size] = 1.0
            self.cache.advance(e.slot, self.cache.length(e.slot) + len(e.tokens))
        return logits


def choose(logits, streams, counters):
    return torch.argmax(logits, dim=-1).tolist()


def test_toy_sequence_with_eos_like_the_reference():
    """{0} -> {0,1,2} with EOS 2, twice, then other budgets (tests/phase5_smoke.cpp:173-192)."""
    engine = ScriptedEngine()
    for _ in range(2):
        out = generate(engine, choose, [[0]], 10, stop_ids=[2])
        assert out.sequences == [[0, 1, 2]] and engine.cache.all_free()
    assert generate(engine, choose, [[0]], 1, stop_ids=[2]).sequences == [[0, 1]]
    assert generate(engine, choose, [[0]], 0, stop_ids=[2]).sequences == [[0]]
    assert generate(engine, choose, [[5, 6, 2]], 4, stop_ids=[2]).sequences == [[5, 6, 2]]     # prompt ends in EOS
    assert generate(engine, choose, [[3, 4, 5, 6, 7]], 3, stop_ids=[2]).sequences == [[3, 4, 5, 6, 7, 8, 9, 10]]
    assert engine.cache.all_free()


def test_last_token_is_never_fed_and_steps_shrink():
    engine = ScriptedEngine()
    out = generate(engine, choose, [[10, 11], [20], [30, 31, 32]], [4, 1, 2])
    assert out.sequences == [[10, 11, 12, 13, 14, 15], [20, 21], [30, 31, 32, 33, 34]]
    sizes = [len(step) for step in engine.steps]
    assert sizes == [3, 2, 1, 1]                     # prompts together, then only the live ones
    assert engine.steps[1] == [(0, [12], [0]), (2, [33], [0])]
    assert engine.steps[-1] == [(0, [14], [0])]      # 15 was chosen last and never fed
    assert out.timings.prefill_tokens == 6 and out.timings.decode_tokens == 4 and out.timings.batches == 1
    assert engine.cache.all_free()


def test_stop_token_ends_one_request_only():
    engine = ScriptedEngine()
    out = generate(engine, choose, [[7], [1]], 5, stop_ids=[9])
    assert out.sequences == [[7, 8, 9], [1, 2, 3, 4, 5, 6]]
    assert [len(step) for step in engine.steps] == [2, 2, 1, 1, 1]


def test_more_requests_than_slots_run_in_batches():
    engine = ScriptedEngine(blocks=4, slots=2)
    prompts = [[i] for i in range(5)]
    out = generate(engine, choose, prompts, 3)
    assert out.sequences == [[i, i + 1, i + 2, i + 3] for i in range(5)]
    assert out.timings.batches == 3 and engine.cache.all_free()
    first = {entry[0] for entry in engine.steps[0]}
    assert {entry[0] for entry in engine.steps[3]} == first      # the second batch reuses the same slots


def test_plan_batches_respects_blocks():
    assert plan_batches([2, 2, 2, 1], free_blocks=4, free_slots=8) == [[0, 1], [2, 3]]
    assert plan_batches([1, 1, 1], free_blocks=9, free_slots=2) == [[0, 1], [2]]
    with pytest.raises(RequestError, match="needs 5 cache blocks"):
        plan_batches([1, 5], free_blocks=4, free_slots=4)


@pytest.mark.parametrize("prompts,budget,message", [
    ([[]], 3, "empty"),
    ([[1, 50]], 3, "outside the vocabulary"),
    ([[-1]], 3, "outside the vocabulary"),
    ([[1]], -1, "nonnegative"),
    ([[1] * 100], 100, "cache blocks"),
])
def test_bad_requests_are_refused_before_anything_runs(prompts, budget, message):
    engine = ScriptedEngine()
    with pytest.raises(RequestError, match=message):
        generate(engine, choose, prompts, budget)
    assert engine.steps == [] and engine.cache.all_free()


def test_an_error_in_a_step_gives_everything_back():
    engine = ScriptedEngine()
    calls = {"n": 0}

    def failing(logits, streams, counters):
        calls["n"] += 1
        if calls["n"] == 3:
            raise RuntimeError("boom")
        return choose(logits, streams, counters)
    with pytest.raises(RuntimeError, match="boom"):
        generate(engine, failing, [[1], [2]], 10)
    assert engine.cache.all_free()


def test_streams_and_counters_follow_the_request():
    engine = ScriptedEngine()
    seen = []

    def spy(logits, streams, counters):
        seen.append((list(streams), list(counters)))
        return choose(logits, streams, counters)
    generate(engine, spy, [[1], [2], [3]], [3, 1, 2], streams=[7, 8, 9])
    assert seen == [([7, 8, 9], [0, 0, 0]), ([7, 9], [1, 1]), ([7], [2])]


def test_a_request_beyond_the_context_limit_is_refused_before_anything_runs():
    """src/generation/generator.cpp:619-632 refuses what cannot fit before it touches anything; the
    limit here is the engine's ``max_context`` (the model's max_position_embeddings unless overridden)."""
    engine = ScriptedEngine()
    engine.max_context = 12
    # a prompt of 8 and 5 new tokens holds 12 positions (the last chosen token is never fed): allowed
    assert len(generate(engine, choose, [[1] * 8], 5).sequences[0]) == 13
    with pytest.raises(RequestError, match=r"request 1: a prompt of 8 tokens plus 6 new ones exceeds the context limit of 12"):
        generate(engine, choose, [[1, 2], [1] * 8], [3, 6])
    assert engine.steps[-1][0][1] != [1, 2] and engine.cache.all_free()      # the first request did not run either
    assert generate(engine, choose, [[1] * 40], 0).sequences == [[1] * 40]   # nothing to run, nothing to refuse


class AheadEngine(ScriptedEngine):
    """A scripted engine that can also take a step's tokens from where the chooser left them ("on the device"),
    as the real engine does for a host that runs one step behind."""
    can_step_ahead = True

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.ahead_steps = 0

    def step_ahead(self, slots, device_tokens):
        from stratakv_b200.engine.engine import StepEntry
        self.ahead_steps += 1
        return self.step([StepEntry(slot, [int(token)], [0]) for slot, token in zip(slots, device_tokens.tolist())])


class LaggingChooser:
    """Chooses at once but hands the ids out only through ``result``; counts what was asked for."""

    def __init__(self):
        self.pending, self.launched = {}, 0

    def launch(self, logits, streams, counters):
        self.launched += 1
        self.pending[self.launched] = torch.argmax(logits, dim=-1).to(torch.int32)
        return self.launched

    def tokens_device(self, handle):
        return self.pending[handle]

    def result(self, handle):
        return self.pending.pop(handle).tolist()

    def __call__(self, logits, streams, counters):
        return self.result(self.launch(logits, streams, counters))


@pytest.mark.parametrize("budgets,stop_ids", [([6, 6, 6], []), ([4, 1, 9], []), ([9, 9, 9], [13]), ([5, 7, 2], [33, 22]),
                                              ([1, 1, 1], []), ([12, 3, 12], [12, 35])])
def test_a_host_one_step_behind_gives_the_same_sequences(budgets, stop_ids):
    """The loop that launches a step before it has read the last one's tokens returns what the loop in turn
    returns, for every mix of budgets and stop tokens, gives every slot back, and drops the rows that ran in vain."""
    prompts = [[10, 11], [20], [30, 31, 32]]
    in_turn = generate(ScriptedEngine(), choose, prompts, budgets, stop_ids=stop_ids).sequences
    engine, chooser = AheadEngine(), LaggingChooser()
    out = generate(engine, chooser, prompts, budgets, stop_ids=stop_ids)
    assert out.sequences == in_turn
    assert engine.cache.all_free() and not chooser.pending
    assert out.timings.decode_tokens == sum(len(s) - len(p) - 1 for s, p in zip(in_turn, prompts))
    if max(budgets) > 2:
        assert engine.ahead_steps > 0
