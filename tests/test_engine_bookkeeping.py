"""The step function's bookkeeping on the CPU: batch packing, positions, block tables and
the order of parts, with a torch stand-in for the kernels (tests/ops_double.py), against
the plain implementation."""
import numpy as np
import pytest
import torch

import plain_llama
from helpers import TINY, make_folder, random_tokens
from ops_double import double_loader
from stratakv_b200 import EngineConfig, StepEntry, StepError
from stratakv_b200.cache import CacheFull
from stratakv_b200.config import load_config
from stratakv_b200.engine.engine import Engine
from stratakv_b200.engine.model import expected_tensors
from stratakv_b200.weights import load_checkpoint


def cpu_engine(folder, max_tokens=512, block_size=16, max_context=None):
    arch, config = load_config(folder)
    spec = arch.build_spec(config)
    tensors = load_checkpoint(folder, {n: r.shape for n, r in expected_tensors(spec).items()}, spec.ignorable)
    return Engine(spec, tensors, EngineConfig(max_tokens=max_tokens, dtype="float32", device="cpu",
                                              block_size=block_size,
                                              max_context=max_tokens if max_context is None else max_context),
                  kernel_loader=double_loader())


@pytest.mark.parametrize("name", ["A", "B"])
def test_cuttings_agree_with_the_plain_model(tmp_path, name):
    folder = make_folder(tmp_path / name, TINY[name], seed=4)
    config, weights = plain_llama.load_folder(folder)
    engine = cpu_engine(folder)
    prompts = [random_tokens(TINY[name]["vocab_size"], n, seed=n) for n in (5, 33, 18)]
    refs = [plain_llama.logits_of(config, weights, p).numpy() for p in prompts]
    slots = [engine.open_sequence() for _ in prompts]
    cut = [3, 20, 17]
    got = engine.step([StepEntry(s, p[:c], list(range(c))) for s, p, c in zip(slots, prompts, cut)])
    np.testing.assert_allclose(got.numpy(), np.concatenate([r[:c] for r, c in zip(refs, cut)]), rtol=1e-4, atol=2e-5)
    # a second piece of each prompt (unequal), then single tokens for the one that is left
    got = engine.step([StepEntry(slots[0], prompts[0][3:], [1]), StepEntry(slots[1], prompts[1][20:30], [9]),
                       StepEntry(slots[2], prompts[2][17:], [0])])
    np.testing.assert_allclose(got.numpy(), np.stack([refs[0][4], refs[1][29], refs[2][17]]), rtol=1e-4, atol=2e-5)
    engine.close_sequence(slots[0]); engine.close_sequence(slots[2])
    for position in range(30, 33):
        got = engine.step([StepEntry(slots[1], [prompts[1][position]], [0])])
        np.testing.assert_allclose(got.numpy()[0], refs[1][position], rtol=1e-4, atol=2e-5)
    engine.close_sequence(slots[1])
    assert engine.cache.all_free()


def test_step_checks(tmp_path):
    folder = make_folder(tmp_path / "A", TINY["A"], seed=4)
    engine = cpu_engine(folder, max_tokens=64, max_context=1000)
    slot = engine.open_sequence()
    with pytest.raises(StepError, match="outside the vocabulary"):
        engine.step([StepEntry(slot, [1, 256], [0])])
    with pytest.raises(StepError, match="wanted place"):
        engine.step([StepEntry(slot, [1, 2], [2])])
    import numpy as np
    for not_ids in ([1.5, 2], ["3"], [1, 2 ** 70], np.array([True, False])):
        with pytest.raises(StepError, match="integers|outside the vocabulary"):
            engine.step([StepEntry(slot, not_ids, [0])])
    # token ids may come as a list, a tuple, numpy integers or an integer array
    for ids in ((1, 2), [np.int64(1), np.int32(2)], np.array([1, 2], dtype=np.int32), np.array([1, 2], dtype=np.uint8)):
        probe = engine.open_sequence()
        assert engine.step([StepEntry(probe, ids, [1])]).shape == (1, 256)
        engine.close_sequence(probe)
    with pytest.raises(StepError, match="at least one token"):
        engine.step([StepEntry(slot, [], [])])
    with pytest.raises(StepError, match="twice"):
        engine.step([StepEntry(slot, [1], []), StepEntry(slot, [2], [])])
    with pytest.raises(StepError, match="not open"):
        engine.step([StepEntry(3, [1], [])])
    with pytest.raises(CacheFull):
        engine.step([StepEntry(slot, [1] * 65, [])])
    assert engine.cache.length(slot) == 0 and engine.cache.free_blocks() == [4]      # nothing was taken
    assert engine.step([StepEntry(slot, [1, 2, 3], [])]) is None
    assert engine.cache.length(slot) == 3
    engine.close_sequence(slot)
    assert engine.cache.all_free()


def test_schedule_may_repeat_a_layer_and_share_a_cache(tmp_path):
    """The order of layers is data: layer 0 run twice (two cache entries), and a run that
    reads the cache another run wrote.  Compared with the plain parts composed the same way."""
    import dataclasses
    from stratakv_b200.parts.spec import ScheduleEntry
    folder = make_folder(tmp_path / "A", TINY["A"], seed=9)
    arch, config = load_config(folder)
    spec = arch.build_spec(config)
    spec = dataclasses.replace(spec, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2),
                                               ScheduleEntry(1, 1, writes_cache=False)))
    tensors = load_checkpoint(folder, {n: r.shape for n, r in expected_tensors(spec).items()}, spec.ignorable)
    engine = Engine(spec, tensors, EngineConfig(max_tokens=256, dtype="float32", device="cpu", block_size=16),
                    kernel_loader=double_loader())
    assert len(engine.cache.groups) == 1 and len(engine.cache.groups[0].entries) == 3
    raw, weights = plain_llama.load_folder(folder)
    tokens = random_tokens(256, 21, seed=1)

    def plain(tokens):
        ids = torch.tensor(tokens)
        x = weights["model.embed_tokens.weight"][ids]
        positions = torch.arange(len(tokens))
        x = plain_llama.decoder_layer(x, weights, 0, raw, positions)
        x_before_1 = x
        x = plain_llama.decoder_layer(x, weights, 1, raw, positions)
        x = plain_llama.decoder_layer(x, weights, 0, raw, positions)
        # layer 1 again, attending to the keys and values its first run cached
        prefix = "model.layers.1."
        h = plain_llama.rmsnorm(x, weights[prefix + "input_layernorm.weight"], raw["rms_norm_eps"])
        h_first = plain_llama.rmsnorm(x_before_1, weights[prefix + "input_layernorm.weight"], raw["rms_norm_eps"])
        heads, kv_heads, hd = 4, 2, 16
        n = len(tokens)
        cos, sin = plain_llama.rope_angles(hd, raw["rope_theta"], positions)
        q = plain_llama.rope((h @ weights[prefix + "self_attn.q_proj.weight"].T).view(n, heads, hd), cos, sin)
        k = plain_llama.rope((h_first @ weights[prefix + "self_attn.k_proj.weight"].T).view(n, kv_heads, hd), cos, sin)
        v = (h_first @ weights[prefix + "self_attn.v_proj.weight"].T).view(n, kv_heads, hd)
        ctx = plain_llama.attention(q, k, v, hd ** -0.5).reshape(n, heads * hd)
        x = x + ctx @ weights[prefix + "self_attn.o_proj.weight"].T
        h = plain_llama.rmsnorm(x, weights[prefix + "post_attention_layernorm.weight"], raw["rms_norm_eps"])
        x = x + plain_llama.feed_forward(h, weights[prefix + "mlp.gate_proj.weight"],
                                         weights[prefix + "mlp.up_proj.weight"], weights[prefix + "mlp.down_proj.weight"])
        x = plain_llama.rmsnorm(x, weights["model.norm.weight"], raw["rms_norm_eps"])
        return x @ weights["lm_head.weight"].T

    slot = engine.open_sequence()
    got = engine.step([StepEntry(slot, tokens[:15], list(range(15)))]).clone()
    ref = plain(tokens)
    np.testing.assert_allclose(got.numpy(), ref[:15].numpy(), rtol=1e-4, atol=2e-5)
    for position in range(15, 21):
        got = engine.step([StepEntry(slot, [tokens[position]], [0])])
        np.testing.assert_allclose(got.numpy()[0], ref[position].numpy(), rtol=1e-4, atol=2e-5)
    engine.close_sequence(slot)


def test_the_context_limit_holds_in_every_step(tmp_path):
    """A sequence may reach max_position_embeddings positions (64 for configuration A) and no more,
    whether the step brings many tokens or one; an engine-level max_context replaces the model's limit."""
    folder = make_folder(tmp_path / "A", TINY["A"], seed=4)
    engine = cpu_engine(folder, max_tokens=256, max_context=0)
    assert engine.max_context == 64
    slot = engine.open_sequence()
    with pytest.raises(StepError, match="65 positions; the limit is 64"):
        engine.step([StepEntry(slot, [1] * 65, [])])
    assert engine.cache.length(slot) == 0 and engine.cache.free_blocks() == [16]    # nothing was taken
    engine.step([StepEntry(slot, [1] * 63, [])])
    engine.step([StepEntry(slot, [2], [0])])
    with pytest.raises(StepError, match="slot 0: the step would bring the sequence to 65 positions"):
        engine.step([StepEntry(slot, [3], [0])])
    assert engine.cache.length(slot) == 64
    engine.close_sequence(slot)
    wider = cpu_engine(folder, max_tokens=256, max_context=100)
    slot = wider.open_sequence()
    wider.step([StepEntry(slot, [1] * 100, [])])
    with pytest.raises(StepError, match="the limit is 100"):
        wider.step([StepEntry(slot, [1], [])])


def test_flag_words_are_decoded_and_cleared(tmp_path):
    """Kernels report trouble by raising bits in a device word; nothing here makes a kernel wait or
    fail: the words are written by the test, and the host's reading of them is what is checked."""
    from stratakv_b200 import ops
    folder = make_folder(tmp_path / "A", TINY["A"], seed=4)
    engine = cpu_engine(folder)
    engine.check_flags()                                         # nothing raised: no error
    engine.model.flags[0] = 4
    with pytest.raises(StepError, match=r"0x4 \(a wait inside a kernel timed out"):
        engine.check_flags()
    engine.check_flags()                                         # cleared by the report
    engine.model.flags[0] = 3
    with pytest.raises(StepError, match=r"0x3 \(a token id outside the vocabulary.*; non-finite logits\)"):
        engine.check_flags()

    class LoadedLibrary:                                         # a kernel library's own flag word
        error_flag = torch.tensor([4], dtype=torch.int32)
    ops._LOADED[("forged", 0)] = LoadedLibrary()
    try:
        engine.model.flags[0] = 2
        with pytest.raises(StepError, match=r"0x6 \(non-finite logits; a wait inside a kernel timed out"):
            engine.check_flags()
        assert int(LoadedLibrary.error_flag) == 0 and int(engine.model.flags) == 0
        engine.model.flags[0] = 8
        with pytest.raises(StepError, match=r"unknown bits 0x8"):
            engine.check_flags()
    finally:
        del ops._LOADED[("forged", 0)]
