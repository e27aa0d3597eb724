"""The cache manager without a GPU: pages, prefix cache, groups, windows, state slots.

The random-walk test plays admit / portion / decode / fork / preempt / finish / evict in random
orders against a shadow store that remembers which token every slot of every page holds, and
checks after every move that no page is lost, held twice or freed twice and that every sequence
still reads back its own tokens.
"""

from __future__ import annotations

import random
from types import SimpleNamespace

import numpy as np
import pytest

from paged_kv_serving_b200.cache import (
    NULL_PAGE, AllocatorInvariantError, GroupSpec, KVCacheManager, OutOfPages, PageAllocator, PrefixCache,
    RecordingPageStore, StateSlotPool, hash_chain, plan_groups,
)
from paged_kv_serving_b200.engine.sequence import PageTable, Request, SamplingParams, Sequence
from paged_kv_serving_b200.parts import PagedKVRequest, StateRequest


def _sequence(name, tokens, groups=1, key="k"):
    request = Request(request_id=name, prompt_token_ids=tuple(tokens), key_id=key, sampling=SamplingParams())
    return Sequence.from_request(request, 0, num_groups=groups)


def _manager(num_blocks=8, block_size=4, groups=None, **kwargs):
    groups = groups or [GroupSpec((0, 1), 2, 16, None)]
    store = RecordingPageStore()
    return KVCacheManager(groups, num_blocks=num_blocks, block_size=block_size, store=store, **kwargs), store


# --- allocator ---------------------------------------------------------------------------------


def test_allocator_fifo_counts_and_all_or_nothing():
    a = PageAllocator(4, 8)
    assert [a.take(), a.take()] == [0, 1]
    a.release(0)
    assert a.take() == 2 and a.take() == 3 and a.take() == 0   # a freed page goes to the back
    with pytest.raises(OutOfPages):
        a.take()
    a.release(1)
    with pytest.raises(OutOfPages):
        a.take_many(2)
    assert a.num_free == 1                                      # nothing was taken
    a.check_invariants()


def test_allocator_refuses_double_free_and_unknown_pages():
    a = PageAllocator(2, 4)
    page = a.take()
    a.release(page)
    with pytest.raises(AllocatorInvariantError, match="twice"):
        a.release(page)
    with pytest.raises(AllocatorInvariantError, match="outside"):
        a.holders(7)
    with pytest.raises(AllocatorInvariantError, match="free and cannot be shared"):
        a.share(page)


def test_private_copy_copies_only_shared_pages():
    store = RecordingPageStore()
    a = PageAllocator(4, 4, group=3, store=store)
    page = a.take()
    assert a.private_copy(page) == page and store.page_copies == []
    a.share(page)
    a.share(page)
    fresh = a.private_copy(page)
    assert fresh != page and store.page_copies == [(3, page, fresh)]
    assert a.holders(page) == 2 and a.holders(fresh) == 1
    a.check_invariants()


def test_corrupted_free_list_is_noticed():
    a = PageAllocator(3, 4)
    a._free.append(0)
    with pytest.raises(AllocatorInvariantError):
        a.check_invariants()


# --- prefix cache ------------------------------------------------------------------------------


def test_hash_chain_commits_to_history_and_scope():
    a = hash_chain(list(range(12)), 4, 3, b"x")
    b = hash_chain([9, 9, 9, 9] + list(range(4, 12)), 4, 3, b"x")
    assert a[1] != b[1] and a[2] != b[2]                      # same later tokens, other history
    assert hash_chain(list(range(12)), 4, 3, b"y")[0] != a[0]
    with pytest.raises(ValueError):
        hash_chain(list(range(7)), 4, 2)


def test_prefix_cache_lookup_stops_at_first_miss_and_evicts_lru_unused():
    a = PageAllocator(8, 4)
    cache = PrefixCache([a])
    keys = hash_chain(list(range(16)), 4, 4)
    pages = [a.take() for _ in range(4)]
    for key, page in zip(keys[:2], pages[:2]):
        assert cache.register(key, (page,))
    assert not cache.register(keys[0], (pages[3],))            # duplicate key keeps the first page
    cache.register(keys[3], (pages[3],))
    found = cache.lookup(keys)
    assert [p[0] for p in found] == pages[:2]                  # block 3 is cached but block 2 is not
    assert a.holders(pages[0]) == 3
    for page in pages:
        a.release(page)
    assert cache.evict(5) == 1                                 # only block 3 is held by the cache alone
    a.release(pages[0]); a.release(pages[1])
    assert cache.flush() == 2 and len(cache) == 0
    a.check_invariants()
    assert a.num_free == 8


# --- manager -----------------------------------------------------------------------------------


def test_reserve_grows_tables_and_is_all_or_nothing():
    manager, _ = _manager(num_blocks=4)
    s = _sequence("a", range(20))
    manager.reserve(s, 9)
    assert len(s.block_table) == 3
    before = (list(s.block_table), manager.allocators[0].snapshot())
    with pytest.raises(OutOfPages):
        manager.reserve(s, 20)
    assert (list(s.block_table), manager.allocators[0].snapshot()) == before
    with pytest.raises(ValueError):
        manager.reserve(s, 21)
    assert manager.free(s) == 3 and manager.num_free_blocks == 4


def test_attach_prefix_leaves_a_token_and_is_scoped_by_key():
    manager, _ = _manager(num_blocks=16)
    first = _sequence("a", range(8), key="tenant")
    manager.reserve(first, 8)
    first.num_computed_tokens = 8
    assert manager.publish_full_blocks(first) == 2
    same = _sequence("b", range(8), key="tenant")
    reuse = manager.attach_prefix(same)
    assert (reuse.blocks, reuse.tokens, same.num_computed_tokens) == (1, 4, 4)   # (8-1)//4 = 1 page reusable
    longer = _sequence("c", list(range(8)) + [1, 2], key="tenant")
    assert manager.attach_prefix(longer).blocks == 2
    other = _sequence("d", range(8), key="someone-else")
    assert manager.attach_prefix(other).blocks == 0
    manager.detach_prefix(longer)
    assert longer.num_computed_tokens == 0 and not longer.holds_pages
    manager.check_invariants()


def test_fork_shares_pages_and_first_write_copies_one_page():
    manager, store = _manager(num_blocks=8, enable_prefix_cache=False)
    parent = _sequence("p", range(6))
    manager.reserve(parent, 6)
    parent.num_computed_tokens = 6
    child = _sequence("c", range(6))
    manager.fork(parent, child)
    assert child.block_table == parent.block_table and child.num_computed_tokens == 6
    child.token_ids.append(7)
    manager.reserve(child, 7)
    assert store.page_copies == [(0, parent.block_table[1], child.block_table[1])]
    assert child.block_table[0] == parent.block_table[0]
    parent.token_ids.append(8)
    manager.reserve(parent, 7)                                  # now the only holder: no second copy
    assert len(store.page_copies) == 1
    manager.free(parent); manager.free(child)
    manager.check_invariants()
    assert manager.num_free_blocks == 8


def test_eviction_under_pressure_and_evictable_count():
    manager, _ = _manager(num_blocks=4)
    a = _sequence("a", range(8))
    manager.reserve(a, 8)
    a.num_computed_tokens = 8
    manager.publish_full_blocks(a)
    manager.free(a)
    assert manager.num_free_blocks == 2 and manager.evictable_blocks() == 2
    b = _sequence("b", range(100, 116))
    manager.reserve(b, 16)                                      # needs all four pages: the cache gives way
    assert manager.prefix_cache.stats.evicted_blocks == 2
    manager.free(b)
    manager.check_invariants()


def test_groups_are_planned_by_shape_and_window():
    groups, states = plan_groups([(0, PagedKVRequest(2, 16)), (1, PagedKVRequest(2, 16, 8)), (2, PagedKVRequest(2, 16)),
                                  (3, StateRequest((4, 8)))])
    assert [(g.entries, g.window) for g in groups] == [((0, 2), None), ((1,), 8)]
    assert states == [(3, StateRequest((4, 8)))]


def test_window_group_gives_pages_back_and_disables_prefix_cache():
    groups = [GroupSpec((0,), 2, 16, None), GroupSpec((1,), 2, 16, 6)]
    manager, _ = _manager(num_blocks=8, block_size=4, groups=groups)
    assert not manager.prefix_cache.enabled
    s = _sequence("w", range(30), groups=2)
    manager.reserve(s, 17)
    s.num_computed_tokens = 17
    # the next query is at 17 and reads keys 12..17 of the windowed group: pages 0..2 are dead
    assert manager.release_behind_window(s) == 3
    assert s.block_tables[1][:3] == [NULL_PAGE] * 3 and NULL_PAGE not in s.block_tables[0]
    assert manager.allocators[1].num_free == 8 - 2 and manager.allocators[0].num_free == 8 - 5
    manager.reserve(s, 30)
    manager.free(s)
    manager.check_invariants()
    assert manager.num_free_blocks == 8


def test_state_slots_follow_admission_fork_and_release():
    manager, store = _manager(num_blocks=8, num_state_slots=3)
    assert not manager.prefix_cache.enabled
    a, b = _sequence("a", range(4)), _sequence("b", range(4))
    manager.acquire_state_slot(a)
    assert manager.state_slots.take_slots_to_clear() == [a.state_slot]
    manager.reserve(a, 4)
    manager.fork(a, b)
    assert store.state_copies == [(a.state_slot, b.state_slot)]
    assert manager.state_slots.take_slots_to_clear() == []      # a forked state is copied, not cleared
    manager.free(a); manager.free(b)
    assert a.state_slot is None and manager.state_slots.num_free == 3
    pool = StateSlotPool(1)
    slot = pool.acquire()
    with pytest.raises(RuntimeError):
        pool.acquire()
    pool.release(slot)
    with pytest.raises(AssertionError):
        pool.release(slot)


# --- random orders -------------------------------------------------------------------------------


class ShadowStore:
    """Remembers which (sequence content) token every slot of every page holds."""

    def __init__(self, block_size):
        self.block_size = block_size
        self.slots: dict[tuple[int, int, int], int] = {}

    def copy_page(self, group, source, destination):
        assert source != destination
        for offset in range(self.block_size):
            if (group, source, offset) in self.slots:
                self.slots[(group, destination, offset)] = self.slots[(group, source, offset)]
            else:
                self.slots.pop((group, destination, offset), None)

    def copy_state(self, source, destination):
        pass

    def write(self, sequence, start, stop):
        for g, table in enumerate(sequence.block_tables):
            for position in range(start, stop):
                page = table[position // self.block_size]
                assert page != NULL_PAGE
                self.slots[(g, page, position % self.block_size)] = sequence.token_ids[position]

    def check(self, sequence, windows):
        for g, table in enumerate(sequence.block_tables):
            for position in range(sequence.num_computed_tokens):
                page = table[position // self.block_size]
                if page == NULL_PAGE:
                    assert windows[g] is not None and position <= sequence.num_computed_tokens - windows[g]
                    continue
                assert self.slots[(g, page, position % self.block_size)] == sequence.token_ids[position]


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("windowed", [False, True])
def test_random_orders_keep_the_books(seed, windowed):
    rng = random.Random(seed)
    block_size = rng.choice([2, 4, 8])
    groups = [GroupSpec((0,), 2, 16, None)] + ([GroupSpec((1,), 1, 8, 2 * block_size + 1)] if windowed else [])
    windows = [g.window for g in groups]
    store = ShadowStore(block_size)
    manager = KVCacheManager(groups, num_blocks=24, block_size=block_size, store=store, prefix_scope="global")
    live: list[Sequence] = []
    prompts = [[rng.randrange(5) for _ in range(rng.randrange(1, 40))] for _ in range(4)]
    counter = 0
    for _ in range(500):
        move = rng.choice(["admit", "advance", "advance", "advance", "fork", "preempt", "finish", "evict"])
        if move == "admit" and len(live) < 6:
            base = rng.choice(prompts)
            tokens = base[: rng.randrange(1, len(base) + 1)] + [rng.randrange(5) for _ in range(rng.randrange(0, 6))]
            s = _sequence(f"s{counter}", tokens, groups=len(groups))
            counter += 1
            manager.attach_prefix(s)
            live.append(s)
        elif move == "advance" and live:
            s = rng.choice(live)
            if s.num_uncomputed_tokens == 0:
                s.token_ids.append(rng.randrange(5))
            count = rng.randrange(1, s.num_uncomputed_tokens + 1)
            try:
                manager.reserve(s, s.num_computed_tokens + count)
            except OutOfPages:
                continue
            store.write(s, s.num_computed_tokens, s.num_computed_tokens + count)
            s.num_computed_tokens += count
            manager.publish_full_blocks(s)
            manager.release_behind_window(s)
        elif move == "fork" and live and len(live) < 6:
            parent = rng.choice(live)
            child = _sequence(f"s{counter}", list(parent.token_ids), groups=len(groups))
            counter += 1
            manager.fork(parent, child)
            live.append(child)
        elif move == "preempt" and live:
            s = rng.choice(live)
            manager.free(s)
            s.reset_for_recompute()
            manager.attach_prefix(s)
        elif move == "finish" and live:
            s = live.pop(rng.randrange(len(live)))
            manager.free(s)
        elif move == "evict":
            manager.prefix_cache.evict(rng.randrange(1, 4))
        manager.check_invariants()
        # every page is accounted for exactly: holders = tables that list it + cache entries
        for g, allocator in enumerate(manager.allocators):
            expected = [0] * allocator.num_pages
            for s in live:
                for page in s.block_tables[g]:
                    if page != NULL_PAGE:
                        expected[page] += 1
            for pages in manager.prefix_cache.cached_pages():
                expected[pages[g]] += 1
            assert tuple(expected) == allocator.snapshot()
        for s in live:
            store.check(s, windows)
            # the immutable copy a table hands to a step follows every change made to the table
            assert all(isinstance(t, PageTable) and t.snapshot() == tuple(t) and t.snapshot().array.tolist() == list(t)
                       for t in s.block_tables)
    for s in live:
        manager.free(s)
    manager.prefix_cache.flush()
    manager.check_invariants()
    assert all(a.num_free == a.num_pages for a in manager.allocators)


def test_a_page_table_makes_its_copy_once_and_again_after_any_change():
    table = PageTable([4, 7])
    first = table.snapshot()
    assert first == (4, 7) and table.snapshot() is first and first.array.dtype == np.int32
    changes = [lambda t: t.append(1), lambda t: t.extend([2, 3]), lambda t: t.__setitem__(0, NULL_PAGE), lambda t: t.pop(),
               lambda t: t.insert(1, 9), lambda t: t.__delitem__(0), lambda t: t.__iadd__([5]), lambda t: t.clear()]
    for change in changes:
        before = table.snapshot()
        frozen = tuple(before)
        change(table)
        after = table.snapshot()
        assert after == tuple(table) and after is not before and before == frozen, "a copy never changes, a change makes a new one"
        assert after.array.tolist() == list(table) and not after.array.flags.writeable
