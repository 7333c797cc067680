"""The cache's bookkeeping: no slot or block is lost, held twice or freed twice."""
import random

import pytest
import torch

from stratakv_b200.cache import CacheFull, IdAllocator, KVCache
from stratakv_b200.parts.base import CacheRequest


def test_allocator_hands_out_each_id_once():
    pool = IdAllocator(5)
    first = pool.take(3)
    assert first == [0, 1, 2] and pool.free_count == 2           # block 0 first, as src/memory/block_pool.cpp:72-75
    with pytest.raises(CacheFull):
        pool.take(3)
    assert pool.free_count == 2                                   # a refused request takes nothing
    pool.give_back([1])
    assert pool.take(1) == [1]                                    # the lowest free id first
    with pytest.raises(ValueError, match="not held"):
        pool.give_back([4])
    with pytest.raises(ValueError, match="outside"):
        pool.give_back([5])
    with pytest.raises(ValueError, match="twice"):
        pool.give_back([0, 0])
    pool.give_back([0, 1, 2])
    with pytest.raises(ValueError, match="not held"):
        pool.give_back([2])                                       # freed twice
    assert pool.free_count == 5 and pool.held_count == 0


def kv(entries=2, blocks=8, block_size=16, slots=4, window=0, state=0):
    kind = "kv_window" if window else "kv"
    requests = [CacheRequest(kind, 2, 16, window, state) for _ in range(entries)]
    return KVCache(requests, blocks, block_size, slots, torch.float32, "cpu")


def test_growth_and_release():
    cache = kv()
    a, b = cache.acquire(), cache.acquire()
    cache.reserve({a: 5, b: 17})
    assert cache.free_blocks() == [8 - 1 - 2]
    cache.advance(a, 5); cache.advance(b, 17)
    cache.reserve({a: 16, b: 18})                                  # still inside the blocks they hold
    assert cache.free_blocks() == [5]
    cache.reserve({a: 17})
    assert cache.free_blocks() == [4]
    rows = cache.block_table_rows(0, [a, b], 3)
    assert rows[0][:2] == [0, 3] and rows[1][:2] == [1, 2]        # sequences' blocks interleave (src/main.cpp:366-393)
    cache.release(a)
    assert cache.free_blocks() == [6]
    with pytest.raises(KeyError):
        cache.release(a)
    cache.release(b)
    assert cache.all_free()


def test_reserve_is_all_or_nothing():
    cache = kv(blocks=4)
    a, b = cache.acquire(), cache.acquire()
    cache.reserve({a: 16})
    with pytest.raises(CacheFull):
        cache.reserve({a: 48, b: 33})                              # needs 2 + 3 > 3 free
    assert cache.free_blocks() == [3] and len(cache.sequences[a].blocks[0]) == 1
    with pytest.raises(ValueError, match="shrink"):
        cache.advance(a, 10) or cache.reserve({a: 5})
    cache.release(a); cache.release(b)
    assert cache.all_free()


def test_slots_run_out_and_come_back():
    cache = kv(slots=2)
    a, b = cache.acquire(), cache.acquire()
    with pytest.raises(CacheFull):
        cache.acquire()
    cache.release(a)
    assert cache.acquire() == a
    cache.release(a); cache.release(b)
    assert cache.all_free()


def test_groups_have_storage_of_their_own():
    requests = [CacheRequest("kv", 2, 16), CacheRequest("kv_window", 2, 16, 20), CacheRequest("kv", 2, 16),
                CacheRequest("kv", 4, 32), CacheRequest("none")]
    cache = KVCache(requests, 6, 16, 3, torch.float32, "cpu")
    assert len(cache.groups) == 3
    assert cache.entry_group == [(0, 0), (1, 0), (0, 1), (2, 0), (-1, -1)]
    assert cache.groups[0].keys.shape == (2, 7, 2, 16, 16) and cache.groups[2].values.shape == (1, 7, 4, 16, 32)
    k0, _ = cache.entry_kv(0)
    k2, _ = cache.entry_kv(2)
    assert k0.data_ptr() != k2.data_ptr() and k0.shape == (7, 2, 16, 16)      # 6 blocks and the spare one
    with pytest.raises(KeyError):
        cache.entry_kv(4)
    slot = cache.acquire()
    cache.reserve({slot: 70})
    cache.advance(slot, 70)
    # the window group gave back the blocks no later query can see (keys below 70 - 20 + 1 = 51 -> 3 blocks)
    assert cache.free_blocks() == [1, 4, 1]
    assert cache.block_table_rows(1, [slot], 5)[0][:3] == [0, 0, 0]
    cache.reserve({slot: 96})
    cache.advance(slot, 96)
    cache.release(slot)
    assert cache.all_free()


def test_state_is_zeroed_when_a_slot_is_taken():
    cache = KVCache([CacheRequest("none", state_bytes=8), CacheRequest("kv", 1, 16)], 4, 16, 2, torch.float32, "cpu")
    slot = cache.acquire()
    cache.state(0)[slot] = 7
    cache.release(slot)
    again = cache.acquire()
    assert again == slot and int(cache.state(0)[again].sum()) == 0


def test_random_traffic_never_loses_a_block():
    rng = random.Random(0)
    cache = kv(entries=1, blocks=12, slots=5)
    live = {}
    for _ in range(2000):
        action = rng.random()
        if action < 0.3 and len(live) < 5:
            live[cache.acquire()] = 0
        elif action < 0.8 and live:
            slot = rng.choice(list(live))
            target = live[slot] + rng.randint(1, 40)
            try:
                cache.reserve({slot: target})
                cache.advance(slot, target)
                live[slot] = target
            except CacheFull:
                pass
        elif live:
            slot = rng.choice(list(live))
            cache.release(slot)
            del live[slot]
        held = [b for record in cache.sequences.values() for b in record.blocks[0]]
        assert len(held) == len(set(held)) == cache.groups[0].blocks.held_count
        assert cache.groups[0].blocks.free_count + len(held) == 12
        assert all(len(cache.sequences[s].blocks[0]) == -(-live[s] // 16) for s in live)
    for slot in list(live):
        cache.release(slot)
    assert cache.all_free()


def test_a_cache_kind_registered_elsewhere_gets_its_own_storage():
    """What a block holds is the cache kind's business: a kind registered by the test keeps one narrow
    tensor per position instead of keys and values, beside ordinary layers whose values are wider than
    their keys; the allocator, the slots and the block tables do not change."""
    from stratakv_b200.cache import CacheKind, register_cache_kind
    register_cache_kind(CacheKind("toy_latent", paged=True, windowed=False,
                                  block_tensors=lambda request, block_size: {"latent": (block_size, request.extra[0])}))
    requests = [CacheRequest("kv", 2, 16, v_head_dim=40), CacheRequest("toy_latent", extra=(24,)),
                CacheRequest("toy_latent", extra=(24,)), CacheRequest("none", state_bytes=8)]
    cache = KVCache(requests, 6, 16, 3, torch.bfloat16, "cpu")
    assert len(cache.groups) == 2 and cache.entry_group == [(0, 0), (1, 0), (1, 1), (-1, -1)]
    k, v = cache.entry_kv(0)
    assert k.shape == (7, 2, 16, 16) and v.shape == (7, 2, 16, 40)
    assert set(cache.entry_storage(2)) == {"latent"} and cache.entry_storage(2)["latent"].shape == (7, 16, 24)
    assert cache.bytes_per_token() == 2 * (2 * 16 + 2 * 40) + 2 * 2 * 24
    slot = cache.acquire()
    cache.reserve({slot: 40})
    assert cache.free_blocks() == [3, 3]
    cache.release(slot)
    assert cache.all_free()
    with pytest.raises(ValueError, match="unknown cache kind 'nothing_like_it'"):
        KVCache([CacheRequest("nothing_like_it")], 4, 16, 2, torch.float32, "cpu")
