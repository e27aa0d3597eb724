"""Prefix cache: full pages of earlier requests, found again by a hash chain over their tokens.

Keys follow the reference (src/paged_kv_serving/engine/prefix_cache.py:43-83): the chain starts
at ``BLAKE2b-128(domain | scope)`` and each full page extends it with
``BLAKE2b-128(parent || page_size as u32 LE || tokens as u32 LE)``, so a key commits to the whole
history before the page. An entry holds one share of a page in every page group (all groups
fill in step, so a cached prefix is usable only when every group can supply it). Entries leave
least-recently-used first, and only when the cache is their last holder
(src/paged_kv_serving/engine/prefix_cache.py:170-198).
"""

from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict
from collections.abc import Sequence
from dataclasses import dataclass

from paged_kv_serving_b200.cache.pages import PageAllocator

__all__ = ["PrefixCache", "PrefixCacheStats", "chain_start", "extend_chain", "hash_chain"]

_DOMAIN = b"paged-kv-serving/prefix-v1"
_DIGEST = 16


def chain_start(scope: bytes = b"") -> bytes:
    return hashlib.blake2b(_DOMAIN + b"|" + scope, digest_size=_DIGEST).digest()


_PAGE_PACKERS: dict[int, struct.Struct] = {}


def extend_chain(parent: bytes, tokens: Sequence[int], page_size: int) -> bytes:
    if len(tokens) != page_size:
        raise ValueError("only full pages are hashed")
    packer = _PAGE_PACKERS.get(page_size)
    if packer is None:
        # the page size, then every token id, as unsigned 32-bit little-endian integers
        packer = _PAGE_PACKERS[page_size] = struct.Struct(f"<{page_size + 1}I")
    try:
        body = packer.pack(page_size, *tokens)
    except struct.error as error:
        raise OverflowError(f"a token id does not fit 32 unsigned bits: {error}") from None
    return hashlib.blake2b(parent + body, digest_size=_DIGEST).digest()


def hash_chain(tokens: Sequence[int], page_size: int, num_pages: int, scope: bytes = b"") -> list[bytes]:
    if num_pages * page_size > len(tokens):
        raise ValueError("not enough tokens for that many full pages")
    parent = chain_start(scope)
    out = []
    for i in range(num_pages):
        parent = extend_chain(parent, tokens[i * page_size:(i + 1) * page_size], page_size)
        out.append(parent)
    return out


@dataclass(slots=True)
class PrefixCacheStats:
    queried_blocks: int = 0
    hit_blocks: int = 0
    registered_blocks: int = 0
    evicted_blocks: int = 0

    @property
    def hit_ratio(self) -> float:
        return self.hit_blocks / self.queried_blocks if self.queried_blocks else 0.0

    def as_dict(self) -> dict[str, float]:
        return {"queried_blocks": float(self.queried_blocks), "hit_blocks": float(self.hit_blocks),
                "registered_blocks": float(self.registered_blocks), "evicted_blocks": float(self.evicted_blocks),
                "hit_ratio": self.hit_ratio}


class PrefixCache:
    """LRU map: chained hash -> one page per group, the cache holding a share of each."""

    def __init__(self, allocators: list[PageAllocator], enabled: bool = True, scope: str = "per_key") -> None:
        if scope not in ("per_key", "global"):
            raise ValueError("scope must be 'per_key' or 'global'")
        self._allocators = allocators
        self._entries: OrderedDict[bytes, tuple[int, ...]] = OrderedDict()
        self.enabled = enabled
        self.scope = scope
        self.stats = PrefixCacheStats()

    def __len__(self) -> int:
        return len(self._entries)

    def scope_bytes(self, key_id: str) -> bytes:
        return key_id.encode("utf-8") if self.scope == "per_key" else b"shared"

    def lookup(self, hashes: Sequence[bytes], record: bool = True) -> list[tuple[int, ...]]:
        """Pages of the longest cached prefix of ``hashes`` (stops at the first miss); the caller
        becomes a holder of every returned page."""
        found: list[tuple[int, ...]] = []
        if self.enabled:
            for key in hashes:
                pages = self._entries.get(key)
                if pages is None:
                    break
                self._entries.move_to_end(key)
                for allocator, page in zip(self._allocators, pages):
                    allocator.share(page)
                found.append(pages)
        if record:
            self.record_lookup(len(hashes), len(found))
        return found

    def record_lookup(self, queried: int, hit: int) -> None:
        self.stats.queried_blocks += queried
        self.stats.hit_blocks += hit

    def register(self, key: bytes, pages: tuple[int, ...]) -> bool:
        """Cache a page set that has just become full; False when the key is already cached."""
        if not self.enabled or key in self._entries:
            return False
        for allocator, page in zip(self._allocators, pages):
            allocator.share(page)
        self._entries[key] = tuple(pages)
        self.stats.registered_blocks += 1
        return True

    def _sole_holder(self, pages: tuple[int, ...]) -> bool:
        return all(a.holders(p) == 1 for a, p in zip(self._allocators, pages))

    def evict(self, count: int = 1) -> int:
        """Drop up to ``count`` least-recently-used entries that only the cache still holds."""
        dropped = 0
        if count <= 0:
            return 0
        victims = []
        for key, pages in self._entries.items():          # least recently used first
            if len(victims) >= count:
                break
            if self._sole_holder(pages):
                victims.append(key)
        for key in victims:
            pages = self._entries.pop(key)
            for allocator, page in zip(self._allocators, pages):
                allocator.release(page)
            dropped += 1
        self.stats.evicted_blocks += dropped
        return dropped

    def evict_until_free(self, needed: int) -> int:
        shortfall = needed - min(a.num_free for a in self._allocators)
        return self.evict(shortfall) if shortfall > 0 else 0

    def flush(self) -> int:
        return self.evict(len(self._entries))

    def evictable(self) -> int:
        return sum(1 for pages in self._entries.values() if self._sole_holder(pages))

    def cached_pages(self) -> tuple[tuple[int, ...], ...]:
        return tuple(self._entries.values())
