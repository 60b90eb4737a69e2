"""The cache's bookkeeping: no slot or page lost, held twice or freed twice; groups
of layers with their own storage; ring of a window group; state zeroed on reuse."""
import random

import pytest
import torch

from llm_b200.cache import FreeList, KvRequest, PagedCache, StateRequest
from llm_b200.errors import CacheFull, ContextFull, LlmError


def make(requests=None, states=None, **options):
    requests = requests if requests is not None else [KvRequest(2, 16)] * 3
    states = states if states is not None else [None] * len(requests)
    defaults = dict(max_tokens=64 * 8, max_seq_len=64 * 4, max_slots=4, dtype=torch.float32, device="cpu")
    return PagedCache(requests, states, **{**defaults, **options})


def test_free_list_refuses_double_take_and_double_free():
    pool = FreeList(3, "page")
    a, b, c = pool.take(), pool.take(), pool.take()
    assert (a, b, c) == (0, 1, 2)
    with pytest.raises(CacheFull):
        pool.take()
    pool.give_back(b)
    with pytest.raises(LlmError):
        pool.give_back(b)
    with pytest.raises(LlmError):
        pool.give_back(7)
    assert pool.take() == 1
    pool.check()


def test_random_traffic_loses_nothing():
    cache = make()
    rng = random.Random(0)
    live = {}
    for _ in range(2000):
        action = rng.random()
        if action < 0.3 and cache.slots.n_free:
            live[cache.acquire()] = 0
        elif action < 0.8 and live:
            slot = rng.choice(list(live))
            grow = live[slot] + rng.randint(1, 90)
            try:
                cache.reserve(slot, grow)
                cache.set_length(slot, grow)
                live[slot] = grow
            except (CacheFull, ContextFull):
                pass
        elif live:
            slot = rng.choice(list(live))
            cache.release(slot)
            del live[slot]
        cache.check()
        held = sum(len(p) for p in cache.groups[0].slot_pages.values())
        assert held == cache.groups[0].pool.n_held
        assert held + cache.groups[0].pool.n_free == cache.groups[0].pool.count
    for slot in list(live):
        cache.release(slot)
    cache.check()
    assert cache.slots.n_free == 4 and cache.groups[0].pool.n_free == 8


def test_errors_change_nothing():
    cache = make()
    a, b = cache.acquire(), cache.acquire()
    cache.reserve(a, 64 * 4)
    with pytest.raises(ContextFull):
        cache.reserve(a, 64 * 4 + 1)
    cache.reserve(b, 64 * 3)
    c = cache.acquire()
    with pytest.raises(CacheFull):
        cache.reserve_many([(c, 64), (b, 64 * 4)])        # needs 2 pages, 1 is free
    assert cache.groups[0].slot_pages[c] == [] and len(cache.groups[0].slot_pages[b]) == 3
    with pytest.raises(LlmError):
        cache.release(3)                                   # never acquired
    cache.release(a)
    with pytest.raises(LlmError):
        cache.release(a)
    cache.check()


def test_groups_have_storage_of_their_own_and_windows_are_rings():
    requests = [KvRequest(2, 16), KvRequest(2, 16, window=100), KvRequest(2, 16), None,
                KvRequest(1, 32, window=100)]
    cache = make(requests, max_tokens=64 * 16, max_seq_len=64 * 16, max_slots=2, step_tokens=64)
    kinds = [(g.kind, g.n_kv_heads, g.head_dim, g.entries) for g in cache.groups]
    assert kinds == [("full", 2, 16, [0, 2]), ("window", 2, 16, [1]), ("window", 1, 32, [4])]
    assert cache.entry_group == [(0, 0), (1, 0), (0, 1), None, (2, 0)]
    assert cache.layer_view(3) is None
    group, keys, values = cache.layer_view(2)
    assert group == 0 and keys.shape == (16, 2, 64, 16) and keys.data_ptr() != values.data_ptr()
    ring = cache.groups[1].ring_pages
    assert ring == (100 + 64 - 2) // 64 + 2 and ring < 16
    slot = cache.acquire()
    cache.reserve(slot, 64 * 16)
    assert len(cache.groups[0].slot_pages[slot]) == 16
    assert len(cache.groups[1].slot_pages[slot]) == ring          # the ring never grows past itself
    table = cache.block_table_rows(1, [slot])
    assert table.shape == (1, ring) and table.dtype == torch.int32
    assert table[0].tolist() == cache.groups[1].slot_pages[slot]
    cache.release(slot)
    cache.check()


def test_state_is_zeroed_when_a_slot_is_taken_again():
    cache = make([None, None], [StateRequest((5,)), None])
    assert cache.state_view(1) is None
    slot = cache.acquire()
    cache.state_view(0)[slot] = 3.0
    cache.release(slot)
    again = cache.acquire()
    assert again == slot and float(cache.state_view(0)[slot].abs().sum()) == 0.0


def test_can_hold_counts_pages_and_slots():
    cache = make()
    assert cache.can_hold([64 * 4, 64 * 4]) and not cache.can_hold([64 * 4] * 3)
    assert not cache.can_hold([1] * 5)                  # five sequences, four slots
    assert not cache.can_hold([64 * 4 + 1])             # longer than a sequence may be
    s = cache.acquire()
    cache.reserve(s, 64 * 4)
    assert cache.can_hold([64 * 4]) and not cache.can_hold([64 * 4, 1, 1, 1])
    cache.set_length(s, 130)
    assert cache.held_tokens() == 192


def test_keys_and_values_of_different_widths_get_storage_of_their_own():
    """A mixer may keep values that are wider or narrower than its keys: such runs form a group of
    their own with one tensor for the keys and one for the values, beside the groups of the rest."""
    import torch
    from llm_b200.cache import KvRequest, PagedCache
    requests = [KvRequest(2, 16), KvRequest(2, 16, value_dim=24), KvRequest(2, 16), KvRequest(2, 16, value_dim=24)]
    cache = PagedCache(requests, [None] * 4, max_tokens=256, max_seq_len=128, max_slots=2,
                       dtype=torch.float32, device="cpu")
    assert len(cache.groups) == 2 and [g.value_dim for g in cache.groups] == [16, 24]
    g0, k0, v0 = cache.layer_view(0)
    g1, k1, v1 = cache.layer_view(1)
    g3, k3, v3 = cache.layer_view(3)
    assert (g0, g1, g3) == (0, 1, 1)
    assert k0.shape == v0.shape == (4, 2, 64, 16)
    assert k1.shape == (4, 2, 64, 16) and v1.shape == (4, 2, 64, 24)
    assert k1.data_ptr() != k3.data_ptr() and v1.data_ptr() != v3.data_ptr()
    assert cache.bytes() == 4 * (2 * 2 * 4 * 2 * 64 * 16 + 2 * 4 * 2 * 64 * (16 + 24))
    slot = cache.acquire()
    cache.reserve(slot, 100)
    assert len(cache.groups[1].slot_pages[slot]) == 2
    cache.release(slot)
    cache.check()
