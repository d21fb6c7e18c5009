"""Radix prefix cache over KV positions for pools of ANY page size.

Same role and method surface as the reference's ``RadixPrefixCache``
(``kestrel/prefix_cache/radix_cache.py:63-574``: ``match_prefix``, ``insert``, ``lock`` /
``unlock``, ``lock_prefill`` / ``unlock_prefill``, ``evict``, ``evictable_page_count``,
``reclaimable_page_count``; ``MatchResult`` / ``InsertResult`` / ``CacheNamespace`` /
``ImageToken``), but the reference only works with one KV position per page
(``kestrel/kv_cache.py:331-335`` refuses anything else).  Here a page holds ``page_size``
positions, so a node boundary may fall inside a page:

* a node covers KV positions ``[start, start + kv_len)`` of its root path and keeps the physical
  pages of logical pages ``start // P .. ceil(end / P) - 1``;
* the page straddling a parent/child boundary appears in both nodes; it is *owned* by the upper
  one.  A child that diverged inside that page starts with its own copy instead (made by
  :meth:`kestrel_b200.kv_cache.PageTable.cow_page`), which it owns;
* a match returns the full pages and, when the matched length is not a multiple of the page size,
  the partially filled last page, which the caller must copy before appending to it
  (:func:`attach_cached_prefix` does the mapping and queues the copy);
* eviction removes unlocked leaves, least recently used first, and returns the pages they own.

With ``page_size == 1`` every operation returns what the reference returns (pinned by traces
recorded from the reference, ``tests/golden/radix_traces.json``).
"""

from __future__ import annotations

import heapq
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Optional, Protocol, runtime_checkable


@runtime_checkable
class CacheToken(Protocol):
    """A token the cache can key on: hashable identity plus the KV positions it occupies."""

    def cache_key(self) -> tuple[Any, ...]: ...

    def kv_length(self) -> int: ...


@dataclass(frozen=True, slots=True)
class ImageToken:
    """An image in the prompt: one cache token spanning many KV positions (729 for Moondream)."""

    content_hash: int
    kv_length_: int

    def cache_key(self) -> tuple:
        return (3, self.content_hash, self.kv_length_)

    def kv_length(self) -> int:
        return self.kv_length_


@dataclass(frozen=True, slots=True)
class CacheNamespace:
    """Isolation key of a tree: runtime, LoRA adapter and image hash never share prefixes."""

    runtime_id: str | None = None
    lora_id: str | None = None
    image_hash: int | None = None


@dataclass(slots=True, eq=False)
class TreeNode:
    """Tokens of one tree edge, the KV range they cover and the physical pages under that range."""

    children: dict = field(default_factory=dict)
    parent: Optional["TreeNode"] = None
    tokens: tuple = ()
    start: int = 0          # first KV position of this node on its root path
    kv_len: int = -1        # KV positions covered; -1: one per page (the reference's page-size-1 invariant)
    physical_pages: tuple = ()
    lock_ref: int = 0
    prefill_lock_ref: int = 0
    last_access_time: float = 0.0
    heap_version: int = 0
    namespace: CacheNamespace | None = None

    def __post_init__(self) -> None:
        if self.kv_len < 0:
            self.kv_len = len(self.physical_pages)

    @property
    def total_kv_length(self) -> int:
        """KV positions in this node (``len(physical_pages)`` at page size 1, as
        ``kestrel/prefix_cache/radix_cache.py:34-37``)."""
        return self.kv_len

    def is_leaf(self) -> bool:
        return not self.children


@dataclass(slots=True)
class MatchResult:
    matched_pages: list[int]      # pages covering the matched positions; the last may be partly filled
    matched_kv_length: int
    matched_token_count: int
    last_node: TreeNode | None
    unmatched_tokens: list
    partial_page_tokens: int = 0  # matched positions inside the last page (0: it is full)


@dataclass(slots=True)
class InsertResult:
    node: TreeNode
    inserted_pages: int


def _idle(node: TreeNode) -> bool:
    return node.lock_ref == 0 and node.prefill_lock_ref == 0


class PagedRadixCache:
    """Prefix tree over token sequences whose leaves hold KV pages of ``page_size`` positions."""

    page_granular = True  # what PageTable looks for before accepting a cache at page_size > 1

    def __init__(self, page_size: int = 1, free_pages_sink: Callable[[list[int]], None] | None = None) -> None:
        if page_size < 1:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self._free_pages_sink = free_pages_sink
        self._trees: dict[CacheNamespace, TreeNode] = {}
        self._default_namespace = CacheNamespace()
        self._total = 0         # pages owned by the tree
        self._evictable = 0     # pages owned by idle leaves
        self._reclaimable = 0   # pages owned by idle nodes (leaves or not)
        self._heap: list[tuple[float, int, TreeNode, int]] = []
        self._tick = 0

    # ------------------------------------------------------------------ page ownership
    def _owned(self, node: TreeNode) -> tuple:
        """Pages this node frees when it goes: all of its pages except a first page it shares with
        the tail of its parent."""
        pages = node.physical_pages
        if not pages:
            return ()
        par = node.parent
        if node.start % self.page_size and par is not None and par.physical_pages and par.physical_pages[-1] == pages[0]:
            return pages[1:]
        return pages

    def _n_owned(self, node: TreeNode) -> int:
        return len(self._owned(node))

    def _counts_as_leaf(self, node: TreeNode) -> bool:
        return node.is_leaf() and _idle(node) and node.parent is not None

    @property
    def total_cached_pages(self) -> int:
        return self._total

    def evictable_page_count(self) -> int:
        return self._evictable

    def reclaimable_page_count(self) -> int:
        return self._reclaimable

    # ------------------------------------------------------------------ LRU heap with lazy deletion
    def _push(self, node: TreeNode) -> None:
        if self._counts_as_leaf(node):
            node.heap_version += 1
            heapq.heappush(self._heap, (node.last_access_time, self._tick, node, node.heap_version))
            self._tick += 1

    def _pop(self) -> TreeNode | None:
        while self._heap:
            _, _, node, version = heapq.heappop(self._heap)
            if node.heap_version != version or not self._counts_as_leaf(node) or not node.tokens:
                continue
            if node.parent.children.get(node.tokens[0].cache_key()) is not node:
                continue
            return node
        return None

    def _rebuild_heap(self) -> None:
        self._heap.clear()
        stack = list(self._trees.values())
        while stack:
            node = stack.pop()
            if node.children:
                stack.extend(node.children.values())
            else:
                self._push(node)

    # ------------------------------------------------------------------ tree walking
    @staticmethod
    def _common(tokens, at: int, edge) -> int:
        n = 0
        while n < len(edge) and at + n < len(tokens) and tokens[at + n].cache_key() == edge[n].cache_key():
            n += 1
        return n

    def _split(self, node: TreeNode, n_tokens: int) -> TreeNode:
        """Cut ``node`` after its first ``n_tokens`` tokens; returns the new upper node."""
        assert 0 < n_tokens < len(node.tokens), "Invalid split position"
        assert node.prefill_lock_ref == 0, "Cannot split prefill-locked node"
        P = self.page_size
        was_leaf = self._counts_as_leaf(node)
        idle = _idle(node)
        owned_before = self._n_owned(node)
        cut = sum(t.kv_length() for t in node.tokens[:n_tokens])       # KV positions going to the upper node
        first_page = node.start // P
        upper_pages = node.physical_pages[: -(-(node.start + cut) // P) - first_page]
        lower_pages = node.physical_pages[(node.start + cut) // P - first_page:]
        upper = TreeNode(parent=node.parent, tokens=node.tokens[:n_tokens], start=node.start, kv_len=cut,
                         physical_pages=upper_pages, lock_ref=node.lock_ref, prefill_lock_ref=node.prefill_lock_ref,
                         last_access_time=node.last_access_time)
        node.tokens = node.tokens[n_tokens:]
        node.start += cut
        node.kv_len -= cut
        node.physical_pages = lower_pages
        node.parent = upper
        upper.children[node.tokens[0].cache_key()] = node
        if upper.parent is not None:
            upper.parent.children[upper.tokens[0].cache_key()] = upper
        # ownership is conserved: pages move to the upper node, nothing is gained or lost
        assert self._n_owned(upper) + self._n_owned(node) == owned_before
        if was_leaf:
            self._evictable -= self._n_owned(upper)   # the upper part is no longer on a leaf
        _ = idle  # reclaimable counts idle nodes, leaf or not: unchanged by a split
        node.heap_version += 1
        self._push(node)
        return upper

    def match_prefix(self, tokens: list, namespace: CacheNamespace | None = None) -> MatchResult:
        """Longest cached prefix of ``tokens`` (whole tokens only).  Touches the matched path for LRU
        and splits a node that matches only in part, unless it is prefill-locked."""
        root = self._trees.get(namespace if namespace is not None else self._default_namespace)
        if root is None:
            return MatchResult([], 0, 0, None, list(tokens))
        P = self.page_size
        by_logical: dict[int, int] = {}
        node, at, kv, path = root, 0, 0, [root]
        while at < len(tokens):
            child = node.children.get(tokens[at].cache_key())
            if child is None:
                break
            n = self._common(tokens, at, child.tokens)
            if n < len(child.tokens):
                if child.prefill_lock_ref > 0:
                    break
                child = self._split(child, n)
            for i, page in enumerate(child.physical_pages):   # deeper nodes override a straddling page
                by_logical[child.start // P + i] = page
            at += len(child.tokens)
            kv += child.kv_len
            node = child
            path.append(child)
        now = time.monotonic()
        for n_ in path:
            n_.last_access_time = now
            self._push(n_)
        pages = [by_logical[i] for i in range(-(-kv // P))]
        return MatchResult(pages, kv, at, node if node is not root else None, list(tokens[at:]), kv % P)

    def insert(self, tokens: list, pages: list[int], namespace: CacheNamespace | None = None,
               from_node: TreeNode | None = None, from_token_idx: int = 0, from_page_idx: int = 0) -> InsertResult:
        """Hand the KV of ``tokens`` to the cache.  ``pages`` are the caller's physical pages of logical
        pages ``0 .. ceil(total_kv / P) - 1``.  The part of the sequence already in the tree must sit
        on the tree's own pages (the caller mapped them after a match) except for a page the caller
        copied-on-write; otherwise nothing is inserted.  ``from_node`` resumes below a matched node
        (``from_page_idx`` = KV positions before it, as in the reference where pages == positions)."""
        P = self.page_size
        total_kv = sum(t.kv_length() for t in tokens)
        assert len(pages) == -(-total_kv // P), (
            f"Page count mismatch: got {len(pages)} pages, expected {-(-total_kv // P)} for {len(tokens)} tokens")
        ns = namespace if namespace is not None else self._default_namespace
        root = self._trees.get(ns)
        if root is None:
            root = self._trees[ns] = TreeNode(namespace=ns)
        if from_node is not None:
            node, at, kv = from_node, from_token_idx, from_page_idx
            if __debug__:
                want = sum(t.kv_length() for t in tokens[:from_token_idx])
                assert kv == want, f"from_page_idx mismatch: got {kv}, expected {want} for {from_token_idx} tokens"
        else:
            node, at, kv = root, 0, 0
        while at < len(tokens):
            child = node.children.get(tokens[at].cache_key())
            if child is None:
                break
            n = self._common(tokens, at, child.tokens)
            if n < len(child.tokens):
                if child.prefill_lock_ref > 0:
                    return InsertResult(node=node, inserted_pages=0)
                child = self._split(child, n)
            # pages that lie completely inside the existing node must be the tree's own pages
            lo, hi = -(-child.start // P), (child.start + child.kv_len) // P
            first = child.start // P
            for lp in range(lo, hi):
                if pages[lp] != child.physical_pages[lp - first]:
                    return InsertResult(node=node, inserted_pages=0)
            at += len(child.tokens)
            kv += child.kv_len
            node = child
        if at >= len(tokens):
            return InsertResult(node=node, inserted_pages=0)
        parent_was_leaf = self._counts_as_leaf(node)
        parent_owned = self._n_owned(node)
        new = TreeNode(parent=node, tokens=tuple(tokens[at:]), start=kv, kv_len=total_kv - kv,
                       physical_pages=tuple(pages[kv // P:]), last_access_time=time.monotonic())
        node.children[new.tokens[0].cache_key()] = new
        gained = self._n_owned(new)
        self._total += gained
        self._evictable += gained
        self._reclaimable += gained
        if parent_was_leaf:
            self._evictable -= parent_owned
        self._push(new)
        return InsertResult(node=new, inserted_pages=gained)

    # ------------------------------------------------------------------ locks
    def _lock(self, node: TreeNode | None, attr: str) -> None:
        if node is None:
            return
        if self._counts_as_leaf(node):
            self._evictable -= self._n_owned(node)
        cur = node
        while cur is not None:
            if _idle(cur):
                self._reclaimable -= self._n_owned(cur)
            setattr(cur, attr, getattr(cur, attr) + 1)
            cur = cur.parent

    def _unlock(self, node: TreeNode | None, attr: str, what: str) -> None:
        if node is None:
            return
        cur = node
        while cur is not None:
            assert getattr(cur, attr) > 0, f"{what} underflow"
            setattr(cur, attr, getattr(cur, attr) - 1)
            if _idle(cur):
                self._reclaimable += self._n_owned(cur)
            cur = cur.parent
        if self._counts_as_leaf(node):
            self._evictable += self._n_owned(node)
            self._push(node)

    def lock(self, node: TreeNode | None) -> None:
        """Keep ``node`` and its ancestors from being evicted (counted, re-entrant)."""
        self._lock(node, "lock_ref")

    def unlock(self, node: TreeNode | None) -> None:
        self._unlock(node, "lock_ref", "Lock ref")

    def lock_prefill(self, node: TreeNode | None) -> None:
        """Keep ``node`` and its ancestors from being split or evicted while a prefill reads them."""
        self._lock(node, "prefill_lock_ref")

    def unlock_prefill(self, node: TreeNode | None) -> None:
        self._unlock(node, "prefill_lock_ref", "Prefill lock ref")

    # ------------------------------------------------------------------ eviction
    def evict(self, needed_pages: int) -> int:
        """Drop idle leaves, least recently used first, until ``needed_pages`` pages were returned to
        the pool (through the sink) or nothing evictable is left; returns the number of pages freed."""
        freed = 0
        while freed < needed_pages:
            victim = self._pop()
            if victim is None:
                self._rebuild_heap()
                victim = self._pop()
                if victim is None:
                    break
            pages = list(self._owned(victim))
            freed += len(pages)
            self._total -= len(pages)
            self._evictable -= len(pages)
            self._reclaimable -= len(pages)
            if self._free_pages_sink is not None:
                self._free_pages_sink(pages)
            parent = victim.parent
            if parent.children.get(victim.tokens[0].cache_key()) is victim:
                del parent.children[victim.tokens[0].cache_key()]
            if self._counts_as_leaf(parent):
                self._evictable += self._n_owned(parent)
                self._push(parent)
            if parent.parent is None and parent.is_leaf() and parent.namespace is not None:
                assert _idle(parent), "Namespace root has non-zero lock_ref/prefill_lock_ref during prune"
                del self._trees[parent.namespace]
        return freed


def attach_cached_prefix(page_table, cache: PagedRadixCache, batch_idx: int, tokens: list, prompt_kv_len: int,
                         namespace: CacheNamespace | None = None):
    """Give page-table row ``batch_idx`` the cached prefix of ``tokens``.

    Follows the reference's lookup policy (``kestrel/models/moondream/runtime.py:1572-1623``): match,
    skip at most ``prompt_kv_len - 1`` positions so that one position is always computed, map the
    cached pages into the row, prefill-lock the matched node.  New here: with a page size above 1
    the last mapped page may be only partly valid for this request; it is replaced by a private
    copy (``PageTable.cow_page`` queues the device copy; run ``copy_kv_pages`` with
    ``take_pending_page_copies()`` before the row's first append).

    Returns ``(skip_positions, shared_page_count, match)``; ``shared_page_count`` is what
    ``PageTable.erase(batch_idx, cached_page_count=...)`` must leave alone while the pages stay
    owned by the cache.
    """
    match = cache.match_prefix(tokens, namespace)
    if match.matched_kv_length <= 0:
        return 0, 0, match
    P = page_table.page_size
    skip = min(match.matched_kv_length, prompt_kv_len - 1)
    if skip <= 0:
        return 0, 0, match
    n_full, partial = divmod(skip, P)
    # Lock first: the copy-on-write below allocates a page, and an allocation may evict idle leaves --
    # the matched node among them while it is unlocked (the reference allocates nothing between
    # map_pages and lock_prefill, kestrel/models/moondream/runtime.py:1607-1615).
    cache.lock_prefill(match.last_node)
    held = len(page_table.page_table_cpu[batch_idx])
    try:
        page_table.map_pages(batch_idx, 0, match.matched_pages[: n_full + (1 if partial else 0)])
        if partial:
            page_table.cow_page(batch_idx, n_full)
    except Exception:
        cache.unlock_prefill(match.last_node)
        page_table.unmap_pages(batch_idx, held)
        raise
    return skip, n_full, match


@dataclass(slots=True)
class SequenceCacheState:
    """What a running sequence holds of the cache (the ``cache_lock_node`` / ``cache_owned_page_count``
    fields of the reference's ``SequenceState``): the node it keeps locked and how many leading pages of
    its page-table row belong to the tree (``PageTable.erase`` must leave those alone)."""
    lock_node: TreeNode | None = None
    cache_owned_page_count: int = 0
    cache_owned_kv_length: int = 0


def finalize_cached_prompt(page_table, cache: PagedRadixCache, batch_idx: int, tokens: list, prompt_kv_len: int,
                           skip: int, shared_page_count: int, match: MatchResult,
                           namespace: CacheNamespace | None = None) -> SequenceCacheState:
    """After the prompt was prefilled: hand its KV to the cache and turn the prefill lock taken by
    :func:`attach_cached_prefix` into the sequence's lock
    (``_finalize_cache_after_prefill``, ``kestrel/models/moondream/runtime.py:1745-1815``).

    * whole prompt already cached: nothing to insert, the matched node stays locked;
    * insert refused or redundant (another sequence was first, or the row does not sit on the tree's
      pages): keep the lock on the matched node, the row's own pages stay private;
    * otherwise lock the new node and release the prefill lock; the row's pages up to the end of the
      prompt now belong to the tree.
    """
    if not tokens:
        return SequenceCacheState()
    temp = match.last_node if skip > 0 else None
    if temp is not None and match.matched_kv_length >= prompt_kv_len:
        cache.lock(temp)
        cache.unlock_prefill(temp)
        return SequenceCacheState(temp, shared_page_count, skip)
    n_pages = -(-prompt_kv_len // page_table.page_size)
    result = cache.insert(tokens, page_table.get_pages(batch_idx, 0, n_pages), namespace)
    if result.inserted_pages == 0:
        if temp is None:
            return SequenceCacheState()
        cache.lock(temp)
        cache.unlock_prefill(temp)
        return SequenceCacheState(temp, shared_page_count, skip)
    cache.lock(result.node)
    if temp is not None:
        cache.unlock_prefill(temp)
    return SequenceCacheState(result.node, shared_page_count + result.inserted_pages, prompt_kv_len)


def retain_generated_prefix(page_table, cache: PagedRadixCache, batch_idx: int, state: SequenceCacheState,
                            tokens: list, total_kv_len: int, namespace: CacheNamespace | None = None) -> None:
    """Make decoded KV eligible for reuse: insert prompt + generated tokens (``tokens``, ``total_kv_len``
    positions, all already in the row's pages) and move the sequence's lock to the new node
    (``retain_sequence_prefix``, ``kestrel/models/moondream/runtime.py:2192-2238``).  When the token path
    already exists on other physical pages nothing is inserted and the row's pages stay private."""
    if not tokens or total_kv_len <= state.cache_owned_kv_length:
        return
    n_pages = -(-total_kv_len // page_table.page_size)
    result = cache.insert(tokens, page_table.get_pages(batch_idx, 0, n_pages), namespace)
    if result.inserted_pages == 0:
        return
    if result.node is not state.lock_node:
        cache.lock(result.node)
        cache.unlock(state.lock_node)
        state.lock_node = result.node
    state.cache_owned_page_count = n_pages
    state.cache_owned_kv_length = total_kv_len


def release_cached_sequence(page_table, cache: PagedRadixCache | None, batch_idx: int,
                            state: SequenceCacheState) -> None:
    """End of a sequence: one unlock of its node, then the row goes back; pages the tree owns stay
    allocated (``release_sequence``, ``kestrel/models/moondream/runtime.py:2240-2253``)."""
    if cache is not None and state.lock_node is not None:
        cache.unlock(state.lock_node)
        state.lock_node = None
    page_table.erase(batch_idx, state.cache_owned_page_count)
