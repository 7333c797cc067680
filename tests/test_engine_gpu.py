"""The engine against the plain implementation: whole requests, the last 32 tokens one by
one, and batches of unequal lengths whose shorter requests end earlier, one batch after
another so that slots and blocks are used again; in float32 and in bfloat16."""
import numpy as np
import pytest
import torch

import plain_llama
from helpers import TINY, make_folder, random_tokens, stored_dtype, tolerance

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


class Folders:
    """Model folders by configuration name and compute dtype, made at first use; the weights are stored
    in the dtype the engine will compute in, so that the plain implementation sees the same values."""

    def __init__(self, root):
        self.root, self.made, self.logits = root, {}, {}

    def __getitem__(self, key):
        name, dtype = key
        if key not in self.made:
            seed = 11 + list(TINY).index(name)
            self.made[key] = make_folder(self.root / f"{name}_{dtype}", TINY[name], seed=seed, dtype=stored_dtype(dtype))
        return self.made[key]

    def plain(self, name, dtype, tokens):
        key = (name, dtype, tuple(tokens))
        if key not in self.logits:
            config, weights = plain_llama.load_folder(self[name, dtype])
            self.logits[key] = plain_llama.logits_of(config, weights, tokens).numpy()
        return self.logits[key]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return Folders(tmp_path_factory.mktemp("models"))


@pytest.fixture(scope="module")
def plain(folders):
    return folders.plain


def engine_for(folder, dtype, max_tokens=2048, block_size=64):
    from stratakv_b200 import Engine, EngineConfig
    return Engine.from_folder(folder, EngineConfig(max_tokens=max_tokens, dtype=dtype, block_size=block_size,
                                                      max_context=max_tokens),
                              verbose=False)


def check(got, ref, dtype, what=""):
    rtol, atol = tolerance(dtype, ref)
    got = got.detach().float().cpu().numpy() if isinstance(got, torch.Tensor) else got
    np.testing.assert_allclose(got, ref, rtol=rtol, atol=atol, err_msg=what)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(TINY))
def test_whole_requests(folders, plain, dtype, name):
    from stratakv_b200 import StepEntry
    engine = engine_for(folders[name, dtype], dtype)
    vocab = TINY[name]["vocab_size"]
    for length in (1, 2, 17, 64, 65, 150):
        tokens = random_tokens(vocab, length, seed=length)
        slot = engine.open_sequence()
        got = engine.step([StepEntry(slot, tokens, list(range(length)))])
        check(got, plain(name, dtype, tokens), dtype, f"{name} whole length {length}")
        engine.close_sequence(slot)
    assert engine.cache.all_free()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(TINY))
def test_last_32_tokens_one_by_one(folders, plain, dtype, name):
    from stratakv_b200 import StepEntry
    engine = engine_for(folders[name, dtype], dtype)
    vocab = TINY[name]["vocab_size"]
    for length in (33, 80, 131):
        tokens = random_tokens(vocab, length, seed=100 + length)
        ref = plain(name, dtype, tokens)
        slot = engine.open_sequence()
        head = length - 32
        got = engine.step([StepEntry(slot, tokens[:head], [head - 1])])
        check(got, ref[head - 1:head], dtype, f"{name} prefix of {length}")
        for position in range(head, length):
            got = engine.step([StepEntry(slot, [tokens[position]], [0])])
            check(got, ref[position:position + 1], dtype, f"{name} length {length} position {position}")
        engine.close_sequence(slot)
    assert engine.cache.all_free()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(TINY))
def test_unequal_batches_with_slot_reuse(folders, plain, dtype, name):
    """Batches start together with unequal prompts, decode together, and the shorter
    requests leave earlier; the next batch takes the freed slots and blocks."""
    from stratakv_b200 import StepEntry
    engine = engine_for(folders[name, dtype], dtype, max_tokens=64 * 6, block_size=16)
    vocab = TINY[name]["vocab_size"]
    batches = [[(5, 8), (9, 3), (13, 12)], [(1, 12), (7, 1), (16, 5), (31, 9)], [(40, 2), (3, 30)]]
    seed = 0
    for batch in batches:
        requests = []
        for prompt_len, decode_len in batch:
            seed += 1
            tokens = random_tokens(vocab, prompt_len + decode_len, seed=seed)
            requests.append(dict(tokens=tokens, prompt=prompt_len, total=prompt_len + decode_len,
                                 slot=engine.open_sequence(), ref=plain(name, dtype, tokens)))
        got = engine.step([StepEntry(r["slot"], r["tokens"][:r["prompt"]], [r["prompt"] - 1]) for r in requests])
        check(got, np.stack([r["ref"][r["prompt"] - 1] for r in requests]), dtype, f"{name} prompts {batch}")
        fed = {id(r): r["prompt"] for r in requests}
        live = list(requests)
        while live:
            for r in [r for r in live if fed[id(r)] >= r["total"]]:
                engine.close_sequence(r["slot"])
                live.remove(r)
            if not live:
                break
            got = engine.step([StepEntry(r["slot"], [r["tokens"][fed[id(r)]]], [0]) for r in live])
            check(got, np.stack([r["ref"][fed[id(r)]] for r in live]), dtype,
                  f"{name} decode at {[fed[id(r)] for r in live]}")
            for r in live:
                fed[id(r)] += 1
        assert engine.cache.all_free()


@pytest.mark.parametrize("dtype", DTYPES)
def test_padding_and_company_change_nothing(folders, dtype):
    """A request's logits are the same alone and in a batch, up to rounding of the same kernels."""
    from stratakv_b200 import StepEntry
    name = "B"
    engine = engine_for(folders[name, dtype], dtype)
    vocab = TINY[name]["vocab_size"]
    tokens = random_tokens(vocab, 23, seed=5)
    slot = engine.open_sequence()
    alone = engine.step([StepEntry(slot, tokens, [22])]).clone()
    engine.close_sequence(slot)
    others = [random_tokens(vocab, n, seed=50 + n) for n in (3, 61, 8)]
    slots = [engine.open_sequence() for _ in range(4)]
    entries = [StepEntry(slots[0], others[0], []), StepEntry(slots[1], others[1], [0]),
               StepEntry(slots[2], tokens, [22]), StepEntry(slots[3], others[2], [])]
    together = engine.step(entries)[1:2].clone()
    rtol, atol = (1e-5, 1e-6) if dtype == "float32" else tolerance(dtype, alone.cpu().numpy())
    torch.testing.assert_close(together, alone, rtol=rtol, atol=atol)
    for s in slots:
        engine.close_sequence(s)


@pytest.mark.parametrize("dtype", DTYPES)
def test_batches_that_do_not_fill_a_graph_bucket(folders, plain, dtype):
    """Nine, then five, eleven, twenty and forty sequences decode together: the decode graph pads its batch
    up to a bucket, and the padding rows (which read and write a spare cache block) must change nothing.
    The larger batches run their projections on the tensor-memory kernels for few tokens."""
    from stratakv_b200 import StepEntry
    name = "B"
    engine = engine_for(folders[name, dtype], dtype, max_tokens=64 * 200)
    vocab = TINY[name]["vocab_size"]
    for batch in (9, 5, 11, 20, 40):
        requests = []
        for i in range(batch):
            tokens = random_tokens(vocab, 3 + 5 * i + 6, seed=1000 + batch * 31 + i)
            requests.append(dict(tokens=tokens, prompt=3 + 5 * i, slot=engine.open_sequence(), ref=plain(name, dtype, tokens)))
        got = engine.step([StepEntry(r["slot"], r["tokens"][:r["prompt"]], [r["prompt"] - 1]) for r in requests])
        check(got, np.stack([r["ref"][r["prompt"] - 1] for r in requests]), dtype, f"prompts of batch {batch}")
        for step in range(6):
            wanted = [r for i, r in enumerate(requests) if (i + step) % 3 != 0]      # some rows want no logits
            entries = [StepEntry(r["slot"], [r["tokens"][r["prompt"] + step]], [0] if r in wanted else [])
                       for r in requests]
            got = engine.step(entries)
            check(got, np.stack([r["ref"][r["prompt"] + step] for r in wanted]), dtype, f"batch {batch} step {step}")
        for r in requests:
            engine.close_sequence(r["slot"])
        assert engine.cache.all_free()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_slot_taken_again_at_the_same_length(folders, plain, dtype):
    """Decode steps prepare the next step's positions and block tables ahead.  A request that ends and
    another that takes its slot and happens to stand at the same length must not inherit them: the
    second request's blocks are others (the first request's blocks are held by a third one meanwhile)."""
    from stratakv_b200 import StepEntry
    name = "B"
    vocab = TINY[name]["vocab_size"]
    engine = engine_for(folders[name, dtype], dtype, max_tokens=1024, block_size=16)
    first, second, third = (random_tokens(vocab, 40, seed=s) for s in (71, 72, 73))
    slot = engine.open_sequence()
    engine.step([StepEntry(slot, first[:30], [])])
    for position in range(30, 36):
        got = engine.step([StepEntry(slot, [first[position]], [0])])
        check(got[0], plain(name, dtype, first)[position], dtype, f"first request, position {position}")
    engine.close_sequence(slot)
    keeper = engine.open_sequence()                      # takes the slot and the blocks just given back
    engine.step([StepEntry(keeper, third[:36], [])])
    again = engine.open_sequence()
    engine.step([StepEntry(again, second[:30], [])])
    engine.close_sequence(keeper)
    slot = engine.open_sequence()
    assert slot == keeper
    engine.step([StepEntry(slot, third[:30], [])])
    for position in range(30, 36):
        got = engine.step([StepEntry(again, [second[position]], [0]), StepEntry(slot, [third[position]], [0])])
        check(got[0], plain(name, dtype, second)[position], dtype, f"second request, position {position}")
        check(got[1], plain(name, dtype, third)[position], dtype, f"third request, position {position}")
    engine.close_sequence(slot)
    engine.close_sequence(again)
    assert engine.cache.all_free()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "E"])
def test_a_prompt_in_several_pieces(folders, plain, dtype, name):
    """A prompt fed in three steps of many tokens each (70 + 65 + 40 with cache blocks of 64): the second and
    third piece attend over keys that earlier steps cached, across block boundaries inside a piece."""
    from stratakv_b200 import StepEntry
    engine = engine_for(folders[name, dtype], dtype, block_size=64)
    tokens = random_tokens(TINY[name]["vocab_size"], 175, seed=9)
    other = random_tokens(TINY[name]["vocab_size"], 100, seed=10)
    ref, ref_other = plain(name, dtype, tokens), plain(name, dtype, other)
    slot, company = engine.open_sequence(), engine.open_sequence()
    got = engine.step([StepEntry(slot, tokens[:70], [0, 69])])
    check(got, ref[[0, 69]], dtype, "first piece")
    # the second piece shares its step with another request's whole prompt
    got = engine.step([StepEntry(company, other, [99]), StepEntry(slot, tokens[70:135], list(range(65)))])
    check(got[:1], ref_other[99:100], dtype, "the other request")
    check(got[1:], ref[70:135], dtype, "second piece")
    engine.close_sequence(company)
    got = engine.step([StepEntry(slot, tokens[135:], list(range(40)))])
    check(got, ref[135:], dtype, "third piece")
    engine.close_sequence(slot)
    assert engine.cache.all_free()


def _decode_after(engine, tokens, meddle=None):
    """Prefill all but the last token, let ``meddle(engine, slot)`` change what the host or the cache holds,
    decode the last token; returns its logits."""
    from stratakv_b200 import StepEntry
    slot = engine.open_sequence()
    engine.step([StepEntry(slot, tokens[:-1], [])])
    undo = meddle(engine, slot) if meddle else None
    got = engine.step([StepEntry(slot, [tokens[-1]], [0])]).float().cpu().numpy()
    if undo:
        undo()
    engine.close_sequence(slot)
    return got


@pytest.mark.parametrize("name", list(TINY))
def test_one_wrong_cache_row_fails_the_bfloat16_comparison(folders, plain, name):
    """The bfloat16 comparisons above are only worth something if a single misplaced key makes them
    fail.  Here the test itself misplaces one, from the host: after the prompt, the cached key and value
    of ONE position out of 99 are overwritten with another position's (in every layer), as a kernel that
    wrote or read one wrong row would leave them.  The comparison passes before and fails after."""
    dtype = "bfloat16"
    engine = engine_for(folders[name, dtype], dtype, block_size=16)
    tokens = random_tokens(TINY[name]["vocab_size"], 100, seed=77)
    ref = plain(name, dtype, tokens)[99:100]
    check(_decode_after(engine, tokens), ref, dtype, "untouched")
    for wrong in (3, 50, 98):
        def overwrite(engine, slot, wrong=wrong):
            group = engine.cache.groups[0]
            blocks = engine.cache.sequences[slot].blocks[0]
            source = 20
            for store in (group.keys, group.values):
                store[:, blocks[wrong // 16], :, wrong % 16] = store[:, blocks[source // 16], :, source % 16]
        with pytest.raises(AssertionError):
            check(_decode_after(engine, tokens, overwrite), ref, dtype, f"position {wrong} overwritten")
    assert engine.cache.all_free()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_wrong_block_table_entry_fails_the_comparison(folders, plain, dtype):
    """The same for the host's own bookkeeping: one entry of the sequence's block list names another of its
    blocks (sixteen positions read from the wrong place).  Done on the host's record before the step."""
    name = "B"
    engine = engine_for(folders[name, dtype], dtype, block_size=16)
    tokens = random_tokens(TINY[name]["vocab_size"], 100, seed=78)
    ref = plain(name, dtype, tokens)[99:100]
    check(_decode_after(engine, tokens), ref, dtype, "untouched")

    def repoint(engine, slot):
        blocks = engine.cache.sequences[slot].blocks[0]
        kept = blocks[2]
        blocks[2] = blocks[4]

        def undo():
            blocks[2] = kept
        return undo
    with pytest.raises(AssertionError):
        check(_decode_after(engine, tokens, repoint), ref, dtype, "block 2 read from block 4")
    assert engine.cache.all_free()
