"""The cache manager: page tables of every live sequence, over one or more page groups.

A *page group* is a set of cache entries (layer calls) with the same needs: the same page shape
and the same retention rule (every key, or a window of the last W positions). Each group has its
own pool of pages and its own table per sequence; a sequence's position ``p`` lives in page
``table[p // page_size]`` at offset ``p % page_size`` of each group. This module is the only
place that changes a sequence's tables.

Behaviour follows the reference's single-group manager
(src/paged_kv_serving/engine/kvcache.py:36-211): prefix reuse that always leaves one token to
compute, publishing of full pages, all-or-nothing reservation with eviction and copy-on-write,
forking by sharing, and release on finish, abort or preemption. What is new here: several groups,
the window rule (pages that every later query has moved past are given back between steps and
their table entry becomes ``NULL_PAGE``), and a slot for per-request state of fixed size.
The prefix cache is used only when every group keeps every key and no mixer has a state of its
own, since a cached prefix must be complete in every group.
"""

from __future__ import annotations

from dataclasses import dataclass

from paged_kv_serving_b200.cache.pages import NULL_PAGE, AllocatorInvariantError, OutOfPages, PageAllocator, PageStore
from paged_kv_serving_b200.cache.prefix_cache import PrefixCache, chain_start, extend_chain
from paged_kv_serving_b200.cache.state_slots import StateSlotPool

__all__ = ["GroupSpec", "KVCacheManager", "PrefixReuse", "plan_groups"]


@dataclass(frozen=True, slots=True)
class GroupSpec:
    """One page group: the cache entries it serves and what a page of it holds."""

    entries: tuple[int, ...]
    n_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True, slots=True)
class PrefixReuse:
    blocks: int
    tokens: int
    queried_blocks: int


def plan_groups(cache_entries: list[tuple[int, object]]) -> tuple[list[GroupSpec], list[tuple[int, object]]]:
    """Sort a model's cache entries into page groups (same heads, head size and window share a
    group) and state entries. Returns ``(groups, state_entries)``."""
    from paged_kv_serving_b200.parts.base import PagedKVRequest, StateRequest

    grouped: dict[tuple, list[int]] = {}
    states: list[tuple[int, object]] = []
    for number, request in cache_entries:
        if isinstance(request, PagedKVRequest):
            grouped.setdefault((request.n_kv_heads, request.head_dim, request.window), []).append(number)
        elif isinstance(request, StateRequest):
            states.append((number, request))
        else:
            raise TypeError(f"unknown cache request {request!r}")
    groups = [GroupSpec(tuple(entries), kv, hd, window) for (kv, hd, window), entries in grouped.items()]
    return groups, states


class KVCacheManager:
    """Page tables, prefix reuse, copy-on-write and state slots for every live sequence.

    Sequences are any objects with ``token_ids``, ``num_tokens``, ``num_computed_tokens``,
    ``block_tables`` (one list per group), ``block_hashes``, ``cached_prefix_blocks``,
    ``state_slot`` and ``request.key_id``.
    """

    def __init__(self, groups: list[GroupSpec], *, num_blocks: int, block_size: int, store: PageStore | None = None,
                 enable_prefix_cache: bool = True, prefix_scope: str = "per_key", num_state_slots: int = 0) -> None:
        if not groups:
            groups = []
        self.group_specs = list(groups)
        self._windowed = any(spec.window is not None for spec in self.group_specs)
        self.block_size = block_size
        self.num_blocks = num_blocks
        self.store = store
        self.allocators = [PageAllocator(num_blocks, block_size, group=g, store=store) for g in range(len(groups))]
        complete_prefixes = all(spec.window is None for spec in groups) and num_state_slots == 0 and bool(groups)
        self.prefix_cache = PrefixCache(self.allocators, enabled=enable_prefix_cache and complete_prefixes,
                                        scope=prefix_scope)
        self.state_slots = StateSlotPool(num_state_slots) if num_state_slots > 0 else None

    # --- capacity ------------------------------------------------------------------------

    @property
    def num_groups(self) -> int:
        return len(self.allocators)

    @property
    def num_free_blocks(self) -> int:
        """Free pages of the tightest group."""
        return min((a.num_free for a in self.allocators), default=self.num_blocks)

    @property
    def utilization(self) -> float:
        return max((a.utilization for a in self.allocators), default=0.0)

    def evictable_blocks(self) -> int:
        return self.prefix_cache.evictable()

    def new_tables(self) -> list[list[int]]:
        return [[] for _ in self.allocators]

    def blocks_required(self, sequence, up_to_tokens: int) -> int:
        needed = -(-up_to_tokens // self.block_size)
        return max((max(0, needed - len(table)) for table in sequence.block_tables), default=0)

    def can_reserve(self, count: int) -> bool:
        return count <= self.num_free_blocks + self.evictable_blocks()

    def coverable_tokens(self, sequence, keep_free: int = 0, enough: int | None = None) -> int:
        """How many more tokens of ``sequence`` the pools could hold beyond those computed,
        leaving ``keep_free`` pages free (the scheduler's memory bound for a portion). Cached
        pages that only the prefix cache holds count as available; they are counted (a walk over
        the whole cache) only when the free pages alone do not cover ``enough`` tokens."""
        def covered(evictable: int) -> int:
            best = None
            for allocator, table in zip(self.allocators, sequence.block_tables):
                available = max(0, allocator.num_free + evictable - keep_free)
                tokens = (len(table) + available) * self.block_size - sequence.num_computed_tokens
                best = tokens if best is None else min(best, tokens)
            return best if best is not None else 1 << 30

        from_free_pages = covered(0)
        if enough is not None and from_free_pages >= enough:
            return from_free_pages
        return covered(self.evictable_blocks())

    # --- prefix reuse --------------------------------------------------------------------

    def attach_prefix(self, sequence, *, record: bool = True) -> PrefixReuse:
        """Adopt cached pages for the longest cached prefix of a sequence that holds nothing yet;
        at least one token is left to compute so that the step produces logits."""
        if sequence.num_computed_tokens or any(sequence.block_tables):
            raise AllocatorInvariantError("attach_prefix runs before any page is taken")
        if not self.prefix_cache.enabled:
            return PrefixReuse(0, 0, 0)
        reusable = (sequence.num_tokens - 1) // self.block_size
        if reusable < 1:
            return PrefixReuse(0, 0, 0)
        parent = chain_start(self.prefix_cache.scope_bytes(sequence.request.key_id))
        hashes = []
        for i in range(reusable):
            parent = extend_chain(parent, sequence.token_ids[i * self.block_size:(i + 1) * self.block_size],
                                  self.block_size)
            hashes.append(parent)
        found = self.prefix_cache.lookup(hashes, record=record)
        for pages in found:
            for table, page in zip(sequence.block_tables, pages):
                table.append(page)
        sequence.block_hashes.extend(hashes[:len(found)])
        sequence.cached_prefix_blocks = len(found)
        sequence.num_computed_tokens = len(found) * self.block_size
        return PrefixReuse(len(found), len(found) * self.block_size, reusable)

    def record_prefix(self, reuse: PrefixReuse) -> None:
        self.prefix_cache.record_lookup(reuse.queried_blocks, reuse.blocks)

    def detach_prefix(self, sequence) -> None:
        """Undo ``attach_prefix`` for a sequence that was not admitted after all."""
        for table in sequence.block_tables:
            if sequence.num_computed_tokens != len(table) * self.block_size:
                raise AllocatorInvariantError("only a freshly attached prefix can be detached")
        self.free(sequence)
        sequence.num_computed_tokens = 0

    def publish_full_blocks(self, sequence) -> int:
        """Offer every page that the computed tokens now fill completely to the prefix cache."""
        if not self.prefix_cache.enabled:
            return 0
        # only pages whose tokens are all final: ids sampled on the device and not read back yet
        # stand at the end of the sequence's tokens and cannot be hashed
        known = sequence.num_tokens - getattr(sequence, "num_unsettled_tokens", 0)
        complete = min(sequence.num_computed_tokens, known) // self.block_size
        if len(sequence.block_hashes) >= complete:
            return 0                       # the usual case of a decode step: no page was filled
        scope = self.prefix_cache.scope_bytes(sequence.request.key_id)
        accepted = 0
        while len(sequence.block_hashes) < complete:
            i = len(sequence.block_hashes)
            parent = sequence.block_hashes[-1] if sequence.block_hashes else chain_start(scope)
            key = extend_chain(parent, sequence.token_ids[i * self.block_size:(i + 1) * self.block_size], self.block_size)
            sequence.block_hashes.append(key)
            if self.prefix_cache.register(key, tuple(table[i] for table in sequence.block_tables)):
                accepted += 1
        return accepted

    # --- reservation ---------------------------------------------------------------------

    def reserve(self, sequence, up_to_tokens: int) -> None:
        """Make positions ``[num_computed_tokens, up_to_tokens)`` writable in every group.

        Missing pages are taken (cached ones evicted when the free list is short) and every page
        in the write range that has another holder is replaced by a private copy. Either all of
        it happens or ``OutOfPages`` is raised with tables and counts as they were.
        """
        if up_to_tokens > sequence.num_tokens:
            raise ValueError("cannot reserve beyond the tokens the sequence has")
        bs = self.block_size
        first = sequence.num_computed_tokens // bs
        last = -(-up_to_tokens // bs)
        # the usual decode step: the token's page is there and nobody else holds it
        if last == first + 1:
            for allocator, table in zip(self.allocators, sequence.block_tables):
                if first >= len(table) or (table[first] != NULL_PAGE and allocator.holders(table[first]) != 1):
                    break
            else:
                return
        plans = []
        for allocator, table in zip(self.allocators, sequence.block_tables):
            extra = max(0, last - len(table))
            shared = [i for i in range(first, min(last, len(table)))
                      if table[i] != NULL_PAGE and allocator.holders(table[i]) > 1]
            plans.append((extra, shared))
        for allocator, (extra, shared) in zip(self.allocators, plans):
            needed = extra + len(shared)
            if needed > allocator.num_free:
                self.prefix_cache.evict(needed - allocator.num_free)
        for allocator, (extra, shared) in zip(self.allocators, plans):
            if extra + len(shared) > allocator.num_free:
                raise OutOfPages(f"group {allocator.group}: {extra + len(shared)} pages wanted, "
                                 f"{allocator.num_free} free")
        for allocator, table, (extra, shared) in zip(self.allocators, sequence.block_tables, plans):
            for i in shared:
                table[i] = allocator.private_copy(table[i])
            if extra:
                table.extend(allocator.take_many(extra))

    def release_behind_window(self, sequence) -> int:
        """Give back the pages of windowed groups that no later query can reach.

        A query at position ``p`` of a group with window ``W`` reads keys ``p-W+1 .. p``; the next
        query sits at ``num_computed_tokens`` or later, so every position up to
        ``num_computed_tokens - W`` is out of reach. Returns the number of pages given back.
        """
        released = 0
        if not self._windowed:
            return released
        for spec, allocator, table in zip(self.group_specs, self.allocators, sequence.block_tables):
            if spec.window is None:
                continue
            dead_positions = sequence.num_computed_tokens - spec.window + 1   # positions < this are dead
            dead_pages = max(0, dead_positions // self.block_size)
            # pages are given back from the front, so the ones already gone form a prefix: walk
            # back from the newest dead page until one of them is met
            i = min(dead_pages, len(table)) - 1
            while i >= 0 and table[i] != NULL_PAGE:
                allocator.release(table[i])
                table[i] = NULL_PAGE
                released += 1
                i -= 1
        return released

    # --- state slots ---------------------------------------------------------------------

    def acquire_state_slot(self, sequence) -> None:
        if self.state_slots is not None and sequence.state_slot is None:
            sequence.state_slot = self.state_slots.acquire(clear=True)

    def release_state_slot(self, sequence) -> None:
        if self.state_slots is not None and sequence.state_slot is not None:
            self.state_slots.release(sequence.state_slot)
            sequence.state_slot = None

    # --- fork and release ----------------------------------------------------------------

    def fork(self, parent, child) -> None:
        """Let ``child`` share every page of ``parent``; the first write of either to a shared
        page gets a private copy through ``reserve``. A state slot is copied at once."""
        if any(child.block_tables):
            raise AllocatorInvariantError("the fork target already holds pages")
        for allocator, parent_table, child_table in zip(self.allocators, parent.block_tables, child.block_tables):
            for page in parent_table:
                if page != NULL_PAGE:
                    allocator.share(page)
            child_table.extend(parent_table)
        child.block_hashes.extend(parent.block_hashes)
        child.num_computed_tokens = parent.num_computed_tokens
        child.cached_prefix_blocks = parent.cached_prefix_blocks
        if self.state_slots is not None and parent.state_slot is not None:
            child.state_slot = self.state_slots.acquire(clear=False)
            if self.store is not None:
                self.store.copy_state(parent.state_slot, child.state_slot)

    def free(self, sequence) -> int:
        """Give back every page (and the state slot) of a sequence; returns the pages it held in
        the first group."""
        held = 0
        for index, (allocator, table) in enumerate(zip(self.allocators, sequence.block_tables)):
            if index == 0:
                held = sum(1 for page in table if page != NULL_PAGE)
            allocator.release_many(table)
            table.clear()
        sequence.block_hashes.clear()
        sequence.cached_prefix_blocks = 0
        self.release_state_slot(sequence)
        return held

    def check_invariants(self) -> None:
        for allocator in self.allocators:
            allocator.check_invariants()
        for pages in self.prefix_cache.cached_pages():
            for allocator, page in zip(self.allocators, pages):
                if allocator.holders(page) < 1:
                    raise AllocatorInvariantError(f"cached page {page} has no holder")
        if self.state_slots is not None:
            self.state_slots.check_invariants()
