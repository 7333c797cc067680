"""The engine at the layer sizes of real models, against the plain implementation.

The tiny configurations of the other suites never make a projection walk more than a tile or two, never
wrap a kernel's ring of stages and never meet a head size of 128.  Here the layers have the sizes of the
TinyLlama-1.1B shape (hidden 2048, 32 query heads on 4 KV heads of size 64, feed-forward 5632, vocabulary
32000; 2 of its 22 layers, which is what keeps the files small) and of the head-size-128 layouts of the
larger shapes (32 heads on 32 and on 8 KV heads; hidden size reduced to 1024).  The reference's own kernel
test goes to the model's shapes in the same way (tests/gemv_smoke.cu:329-357, 562-581).

The plain implementation runs on the GPU here (float32 with the same double-precision steps as on the
CPU; it shares no code with the engine either way): a 2,048-token sequence would take it minutes on the CPU.
"""
import numpy as np
import pytest
import torch

import plain_llama
from helpers import make_folder, random_tokens, stored_dtype, tolerance

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
BASE = dict(architectures=["LlamaForCausalLM"], hidden_act="silu")
MODELS = {
    # two layers of the TinyLlama-1.1B shape
    "tinyllama": dict(BASE, hidden_size=2048, intermediate_size=5632, num_hidden_layers=2, num_attention_heads=32,
                      num_key_value_heads=4, head_dim=64, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0,
                      max_position_embeddings=2048, tie_word_embeddings=False),
    # head size 128, every query head with a KV head of its own (the Llama-2-7B layout), an odd vocabulary
    "mha128": dict(BASE, hidden_size=1024, intermediate_size=2816, num_hidden_layers=1, num_attention_heads=32,
                   num_key_value_heads=32, head_dim=128, vocab_size=4001, rms_norm_eps=1e-5, rope_theta=10000.0,
                   max_position_embeddings=4096, tie_word_embeddings=False),
    # head size 128, four query heads per KV head (the Llama-3-8B layout), tied embeddings
    "gqa128": dict(BASE, hidden_size=1024, intermediate_size=3584, num_hidden_layers=2, num_attention_heads=32,
                   num_key_value_heads=8, head_dim=128, vocab_size=8016, rms_norm_eps=1e-5, rope_theta=500000.0,
                   max_position_embeddings=8192, tie_word_embeddings=True),
}
# bfloat16 noise as a fraction of the logits' spread.  Sums over 2,048 and 5,632 rounded inputs, and the
# maximum over 32,000 x 2,048 logits, reach further than at the tiny sizes: measured 0.047 (TinyLlama
# layers) and 0.030 (the others) at most.  (helpers.tolerance explains the measure.)
NOISE = {"tinyllama": 0.07, "mha128": 0.045, "gqa128": 0.045}


class Models:
    def __init__(self, root):
        self.root, self.folders, self.weights, self.logits = root, {}, {}, {}

    def folder(self, name, dtype):
        key = (name, dtype)
        if key not in self.folders:
            self.folders[key] = make_folder(self.root / f"{name}_{dtype}", MODELS[name], seed=5,
                                            dtype=stored_dtype(dtype))
        return self.folders[key]

    def plain(self, name, dtype, tokens):
        """Logits of the whole sequence at every position, float32 on the GPU."""
        key = (name, dtype, tuple(tokens))
        if key not in self.logits:
            if (name, dtype) not in self.weights:
                self.weights.clear()                      # one model's float32 copy at a time
                self.weights[name, dtype] = plain_llama.load_folder(self.folder(name, dtype), device="cuda")
            config, weights = self.weights[name, dtype]
            self.logits[key] = plain_llama.logits_of(config, weights, tokens)
        return self.logits[key]

    def forget(self):
        self.logits.clear()


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return Models(tmp_path_factory.mktemp("model_sizes"))


def engine_for(models, name, dtype, max_tokens, max_batch=0):
    from stratakv_b200 import Engine, EngineConfig
    return Engine.from_folder(models.folder(name, dtype),
                              EngineConfig(max_tokens=max_tokens, dtype=dtype, max_batch=max_batch,
                                           max_context=max_tokens), verbose=False)


def check(got, ref, name, dtype, what):
    """``ref`` rows (a GPU tensor) against the engine's; the measure of helpers.tolerance."""
    ref = ref.float().cpu().numpy()
    rtol, atol = tolerance(dtype, ref, noise=NOISE[name])
    np.testing.assert_allclose(got.float().cpu().numpy(), ref, rtol=rtol, atol=atol, err_msg=f"{name} {dtype} {what}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(MODELS))
def test_whole_then_the_last_32_one_by_one_then_in_pieces(models, name, dtype):
    from stratakv_b200 import StepEntry
    engine = engine_for(models, name, dtype, max_tokens=3 * 2048 + 64)
    vocab = MODELS[name]["vocab_size"]
    for length in (300, 2048):
        tokens = random_tokens(vocab, length, seed=length)
        ref = models.plain(name, dtype, tokens)
        # whole, every position's logits
        slot = engine.open_sequence()
        check(engine.step([StepEntry(slot, tokens, list(range(length)))]), ref, name, dtype, f"whole {length}")
        engine.close_sequence(slot)
        # all but 32 tokens in one step, the rest one by one
        slot = engine.open_sequence()
        head = length - 32
        check(engine.step([StepEntry(slot, tokens[:head], [head - 1])]), ref[head - 1:head], name, dtype,
              f"prefix of {length}")
        for position in range(head, length):
            check(engine.step([StepEntry(slot, [tokens[position]], [0])]), ref[position:position + 1], name, dtype,
                  f"length {length} position {position}")
        engine.close_sequence(slot)
        # in pieces of many tokens that end inside cache blocks
        slot = engine.open_sequence()
        cuts = [0, 70, 135, 175, length] if length == 300 else [0, 1000, 1500, 1501, length]
        for lo, hi in zip(cuts[:-1], cuts[1:]):
            check(engine.step([StepEntry(slot, tokens[lo:hi], list(range(hi - lo)))]), ref[lo:hi], name, dtype,
                  f"length {length} piece {lo}:{hi}")
        engine.close_sequence(slot)
        models.forget()
    assert engine.cache.all_free()
    engine.check_flags()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tinyllama", "gqa128"])
def test_unequal_batches_of_8_and_64_with_early_finishers(models, name, dtype):
    """A batch of 8 and then one of 64 requests with unequal prompts that start together and end one after
    another; the second batch takes the slots and blocks the first gave back."""
    from stratakv_b200 import StepEntry
    engine = engine_for(models, name, dtype, max_tokens=64 * 4 * 64 + 8 * 8 * 64, max_batch=64)
    vocab = MODELS[name]["vocab_size"]
    rng = np.random.default_rng(3)
    for batch in (8, 64):
        longest = 450 if batch == 8 else 200
        requests = []
        for i in range(batch):
            prompt, decode = int(rng.integers(1, longest)), int(rng.integers(1, 9))
            tokens = random_tokens(vocab, prompt + decode, seed=1000 * batch + i)
            requests.append(dict(tokens=tokens, prompt=prompt, total=prompt + decode, slot=engine.open_sequence(),
                                 ref=models.plain(name, dtype, tokens)))
        got = engine.step([StepEntry(r["slot"], r["tokens"][:r["prompt"]], [r["prompt"] - 1]) for r in requests])
        check(got, torch.stack([r["ref"][r["prompt"] - 1] for r in requests]), name, dtype, f"prompts of batch {batch}")
        fed = {id(r): r["prompt"] for r in requests}
        live = list(requests)
        while live:
            for r in [r for r in live if fed[id(r)] >= r["total"]]:
                engine.close_sequence(r["slot"])
                live.remove(r)
            if not live:
                break
            got = engine.step([StepEntry(r["slot"], [r["tokens"][fed[id(r)]]], [0]) for r in live])
            check(got, torch.stack([r["ref"][fed[id(r)]] for r in live]), name, dtype,
                  f"batch {batch}, {len(live)} live")
            for r in live:
                fed[id(r)] += 1
        assert engine.cache.all_free()
        models.forget()
    engine.check_flags()
