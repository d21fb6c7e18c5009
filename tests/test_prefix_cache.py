"""The page-granular radix prefix cache: traces recorded from the reference cache (one position per
page) replay identically; page sizes above one add partial-page matches, copy-on-write and
page ownership across node boundaries."""

import json

import pytest

from kestrel_b200.kv_cache import PageTable
from kestrel_b200.prefix_cache import (CacheNamespace, ImageToken, PagedRadixCache, attach_cached_prefix,
                                       finalize_cached_prompt, release_cached_sequence, retain_generated_prefix)


class Tok:
    def __init__(self, ident, kv=1):
        self.ident, self.kv = ident, kv

    def cache_key(self):
        return (0, self.ident, self.kv)

    def kv_length(self):
        return self.kv


def toks(*ids):
    return [Tok(i) for i in ids]


def test_reference_traces_replay_identically_at_page_size_one(golden_dir):
    traces = json.loads((golden_dir / "radix_traces.json").read_text())
    namespaces = [None, CacheNamespace(lora_id="a"), CacheNamespace(image_hash=7)]
    checked = 0
    for tr in traces:
        freed = []
        cache = PagedRadixCache(page_size=1, free_pages_sink=lambda pages: freed.extend(pages))
        handles = []
        for i, rec in enumerate(tr["ops"]):
            op = rec["op"]
            where = (tr["seed"], i, op)
            if op in ("match", "insert"):
                objs = [Tok(a, k) for a, k in rec["tokens"]]
                ns = namespaces[rec["ns"]]
                m = cache.match_prefix(objs, ns)
                handles.append(m.last_node)
                if op == "match":
                    got = [list(m.matched_pages), m.matched_kv_length, m.matched_token_count, len(m.unmatched_tokens),
                           m.last_node is not None]
                    assert got == rec["ret"], where
                    assert m.partial_page_tokens == 0
                else:
                    if rec["reuse"]:
                        assert rec["pages"][: len(m.matched_pages)] == m.matched_pages, where
                    r = cache.insert(objs, rec["pages"], ns)
                    handles.append(r.node)
                    assert [r.inserted_pages] == rec["ret"], where
            elif op == "lock":
                cache.lock(handles[rec["h"]])
            elif op == "lock_prefill":
                cache.lock_prefill(handles[rec["h"]])
            elif op == "unlock":
                (cache.unlock if rec["kind"] == "lock" else cache.unlock_prefill)(handles[rec["h"]])
            elif op == "evict":
                del freed[:]
                got = cache.evict(rec["n"])
                assert [got, sorted(freed)] == rec["ret"], where
            assert [cache.total_cached_pages, cache.evictable_page_count(), cache.reclaimable_page_count()] == rec["counts"], where
            checked += 1
    assert checked > 1000


def test_match_insert_split_basics():
    c = PagedRadixCache(page_size=1)
    assert c.match_prefix(toks(1, 2)).matched_kv_length == 0
    r = c.insert(toks(1, 2, 3), [10, 11, 12])
    assert r.inserted_pages == 3 and c.total_cached_pages == 3
    m = c.match_prefix(toks(1, 2, 99))
    assert (m.matched_pages, m.matched_token_count, len(m.unmatched_tokens)) == ([10, 11], 2, 1)
    assert m.last_node.tokens[-1].ident == 2 and len(m.last_node.children) == 1   # the node was split
    assert c.insert(toks(1, 2, 3), [10, 11, 12]).inserted_pages == 0             # already there
    assert c.insert(toks(1, 2, 4), [70, 71, 72]).inserted_pages == 0             # foreign pages for a cached prefix
    assert c.insert(toks(1, 2, 4), [10, 11, 72]).inserted_pages == 1
    with pytest.raises(AssertionError, match="Page count mismatch"):
        c.insert(toks(5), [1, 2])
    ns = CacheNamespace(lora_id="x")
    assert c.match_prefix(toks(1, 2), ns).matched_kv_length == 0
    c.insert(toks(1, 2), [40, 41], ns)
    assert c.match_prefix(toks(1, 2), ns).matched_pages == [40, 41]


def test_locks_eviction_order_and_counts():
    freed = []
    c = PagedRadixCache(page_size=1, free_pages_sink=freed.extend)
    a = c.insert(toks(1, 2), [1, 2]).node
    b = c.insert(toks(1, 2, 3), [1, 2, 3]).node
    d = c.insert(toks(7), [9]).node
    assert (c.total_cached_pages, c.evictable_page_count(), c.reclaimable_page_count()) == (4, 2, 4)
    c.lock(b)
    assert (c.evictable_page_count(), c.reclaimable_page_count()) == (1, 1)
    assert c.evict(10) == 1 and freed == [9]         # only the unlocked leaf goes
    c.unlock(b)
    c.match_prefix(toks(1, 2, 3))                    # touch
    assert c.evict(1) == 1 and freed[-1] == 3        # leaf first, then its parent becomes a leaf
    assert c.evict(5) == 2 and sorted(freed[-2:]) == [1, 2]
    assert c.total_cached_pages == 0 and c.match_prefix(toks(1)).matched_kv_length == 0
    with pytest.raises(AssertionError, match="underflow"):
        c.unlock(a)
    _ = d


def test_prefill_lock_blocks_split():
    c = PagedRadixCache(page_size=1)
    n = c.insert(toks(1, 2, 3, 4), [1, 2, 3, 4]).node
    c.lock_prefill(n)
    m = c.match_prefix(toks(1, 2, 9))
    assert m.matched_kv_length == 0 and m.last_node is None     # cannot split a node a prefill is reading
    assert c.insert(toks(1, 2, 9), [1, 2, 50]).inserted_pages == 0
    c.unlock_prefill(n)
    assert c.match_prefix(toks(1, 2, 9)).matched_pages == [1, 2]


def test_partial_page_match_and_ownership_at_page_size_16():
    P = 16
    freed = []
    c = PagedRadixCache(page_size=P, free_pages_sink=freed.extend)
    prefix = [ImageToken(content_hash=1, kv_length_=729)]
    # first request: image + 20 text tokens = 749 positions = 47 pages (the last holds 13 tokens)
    seq_a = prefix + toks(*range(100, 120))
    pages_a = list(range(200, 247))
    ra = c.insert(seq_a, pages_a)
    assert ra.inserted_pages == 47 and c.total_cached_pages == 47
    # second request shares only the image: 45 full pages + 9 tokens of page 46
    m = c.match_prefix(prefix + toks(500, 501))
    assert m.matched_kv_length == 729 and m.partial_page_tokens == 9
    assert m.matched_pages == pages_a[:46]
    upper = m.last_node
    assert upper.kv_len == 729 and len(upper.physical_pages) == 46
    lower = next(iter(upper.children.values()))
    assert lower.start == 729 and lower.physical_pages == tuple(pages_a[45:])   # page 245 straddles the cut
    assert c.total_cached_pages == 47                                              # nothing gained or lost by the split
    # the second request copied page 245 to 300 and continues on its own pages
    seq_b = prefix + toks(500, 501, 502)
    pages_b = pages_a[:45] + [300]
    rb = c.insert(seq_b, pages_b)
    assert rb.inserted_pages == 1 and c.total_cached_pages == 48
    assert rb.node.start == 729 and rb.node.physical_pages == (300,)
    m2 = c.match_prefix(seq_b)
    assert m2.matched_kv_length == 732 and m2.matched_pages == pages_b and m2.partial_page_tokens == 12
    # a request that did not map the shared pages cannot insert over them
    assert c.insert(prefix + toks(7), list(range(900, 946))).inserted_pages == 0
    # eviction: leaves first; the straddling page stays with the image node until that goes too
    c.lock(rb.node)
    assert c.evict(100) == 1 and freed == [246]      # request A's tail owns only its last page
    c.unlock(rb.node)
    assert c.evict(1) == 1 and freed[-1] == 300
    assert c.evict(100) == 46 and sorted(freed[-46:]) == pages_a[:46]
    assert c.total_cached_pages == 0 and c.evictable_page_count() == 0 and c.reclaimable_page_count() == 0


def test_attach_cached_prefix_maps_shared_pages_and_queues_cow():
    P = 16
    cache = PagedRadixCache(page_size=P)
    pt = PageTable(n_pages=200, page_size=P, max_batch_size=6, device="cpu", prefix_cache=cache)
    assert cache._free_pages_sink == pt.free_pages_to_pool
    image = [ImageToken(content_hash=5, kv_length_=729)]
    # request 1: miss, prefill, insert, keep its node locked while it decodes
    r1 = pt.allocate()
    prompt1 = image + toks(*range(10, 40))
    skip, shared, match = attach_cached_prefix(pt, cache, r1, prompt1, 759)
    assert (skip, shared) == (0, 0) and match.last_node is None
    pt.reserve(r1, 759)
    ins = cache.insert(prompt1, pt.get_pages(r1, 0, 48))
    assert ins.inserted_pages == 48
    cache.lock(ins.node)
    # request 2: same image, other text
    r2 = pt.allocate()
    prompt2 = image + toks(*range(50, 60))
    skip, shared, match = attach_cached_prefix(pt, cache, r2, prompt2, 739)
    assert skip == 729 and shared == 45 and match.partial_page_tokens == 9
    row1, row2 = pt.page_table_cpu[r1], pt.page_table_cpu[r2]
    assert row2[:45] == row1[:45] and row2[45] != row1[45] and len(row2) == 46
    assert pt.take_pending_page_copies() == ([row1[45]], [row2[45]])
    pt.reserve(r2, 739)
    cache.unlock_prefill(match.last_node)
    ins2 = cache.insert(prompt2, pt.get_pages(r2, 0, 47))
    assert ins2.inserted_pages == 2          # its copy of the straddling page + one more
    # a full match is capped so that one position is still computed
    r3 = pt.allocate()
    skip, shared, match3 = attach_cached_prefix(pt, cache, r3, prompt2, 739)
    assert skip == 738 and shared == 46 and len(pt.page_table_cpu[r3]) == 47
    cache.unlock_prefill(match3.last_node)
    # releasing: cache-owned leading pages stay, private ones return
    free_before = pt.pages_available
    pt.erase(r3, cached_page_count=shared)
    assert pt.pages_available == free_before + 1          # only the copied page was private
    pt.erase(r2, cached_page_count=47)
    cache.unlock(ins.node)
    pt.erase(r1, cached_page_count=48)
    # pressure: a big reservation evicts cached prefixes through the page table
    big = pt.allocate()
    assert pt.can_reserve_with_eviction(190 * P, big)
    assert pt.reserve(big, 190 * P)
    assert cache.total_cached_pages < 50


@pytest.mark.parametrize("P", [1, 16])
def test_sequence_lifecycle_lookup_finalize_retain_release(P):
    """The runtime policy around the cache (kestrel/models/moondream/runtime.py:1572-1623, 1745-1815,
    2192-2253): miss -> insert and lock; hit -> prefill lock becomes the sequence's lock; generated tokens
    are retained; release unlocks once and frees only private pages."""
    cache = PagedRadixCache(page_size=P)
    pt = PageTable(n_pages=4096 if P == 1 else 400, page_size=P, max_batch_size=6, device="cpu", prefix_cache=cache)
    pages_for = lambda n: -(-n // P)
    image = [ImageToken(content_hash=9, kv_length_=729)]
    free0 = pt.pages_available

    # --- request 1: miss
    r1 = pt.allocate()
    prompt1 = image + toks(*range(100, 120))                     # 749 positions
    skip, shared, match = attach_cached_prefix(pt, cache, r1, prompt1, 749)
    assert (skip, shared) == (0, 0)
    pt.reserve(r1, 749 + 8)
    s1 = finalize_cached_prompt(pt, cache, r1, prompt1, 749, skip, shared, match)
    assert s1.lock_node is not None and s1.cache_owned_page_count == pages_for(749) and s1.lock_node.lock_ref == 1
    assert cache.evictable_page_count() == 0                     # locked: nothing can be evicted

    # --- request 2: same prompt completely cached (skip capped at prompt - 1)
    r2 = pt.allocate()
    skip, shared, match = attach_cached_prefix(pt, cache, r2, prompt1, 749)
    assert skip == 748 and match.last_node.prefill_lock_ref == 1
    pt.take_pending_page_copies()
    pt.reserve(r2, 749 + 8)
    s2 = finalize_cached_prompt(pt, cache, r2, prompt1, 749, skip, shared, match)
    assert s2.lock_node is s1.lock_node and s2.cache_owned_page_count == shared
    assert s2.lock_node.lock_ref == 2 and s2.lock_node.prefill_lock_ref == 0

    # --- request 3: shares the image only; its suffix is inserted below the image node
    r3 = pt.allocate()
    prompt3 = image + toks(*range(200, 230))                     # 759 positions
    skip, shared, match = attach_cached_prefix(pt, cache, r3, prompt3, 759)
    assert skip == 729 and shared == 729 // P
    pt.take_pending_page_copies()
    pt.reserve(r3, 759 + 8)
    s3 = finalize_cached_prompt(pt, cache, r3, prompt3, 759, skip, shared, match)
    assert s3.lock_node is not s1.lock_node and s3.cache_owned_page_count == pages_for(759)
    assert match.last_node.prefill_lock_ref == 0

    # --- request 1 decodes 5 tokens and retains them
    gen = toks(*range(900, 905))
    retain_generated_prefix(pt, cache, r1, s1, prompt1 + gen, 749 + 5)
    assert s1.cache_owned_page_count == pages_for(754) and s1.cache_owned_kv_length == 754
    assert s1.lock_node is not s2.lock_node and s2.lock_node.lock_ref == 2   # ancestors stay locked through r1's new node
    retain_generated_prefix(pt, cache, r1, s1, prompt1 + gen, 749 + 5)        # nothing new: no change
    assert s1.cache_owned_kv_length == 754
    m = cache.match_prefix(prompt1 + gen)
    assert m.matched_kv_length == 754

    # --- releases: private pages come back, cache-owned ones stay with the tree
    for r, st in ((r1, s1), (r2, s2), (r3, s3)):
        release_cached_sequence(pt, cache, r, st)
        assert st.lock_node is None
    assert cache.evictable_page_count() > 0 and cache.reclaimable_page_count() == cache.total_cached_pages
    assert pt.pages_available == free0 - cache.total_cached_pages
    freed = cache.evict(10 ** 6)
    assert freed > 0 and cache.total_cached_pages == 0 and pt.pages_available == free0


def test_finalize_keeps_pages_private_when_the_row_is_not_on_the_trees_pages():
    # a second sequence prefilled the same prompt on its own pages (no lookup): the insert is refused
    P = 16
    cache = PagedRadixCache(page_size=P)
    pt = PageTable(n_pages=200, page_size=P, max_batch_size=4, device="cpu", prefix_cache=cache)
    prompt = toks(*range(40))
    states = []
    for _ in range(2):
        r = pt.allocate()
        pt.reserve(r, 48)
        empty = cache.match_prefix([])
        states.append((r, finalize_cached_prompt(pt, cache, r, prompt, 40, 0, 0, empty)))
    (ra, sa), (rb, sb) = states
    assert sa.cache_owned_page_count == 3 and sb.lock_node is None and sb.cache_owned_page_count == 0
    free_before = pt.pages_available
    release_cached_sequence(pt, cache, rb, sb)
    assert pt.pages_available == free_before + 3          # all of its pages were private
    release_cached_sequence(pt, cache, ra, sa)
    assert pt.pages_available == free_before + 3          # the tree keeps the first sequence's pages


def test_attach_with_an_empty_free_list_cannot_evict_the_prefix_it_just_matched():
    """The partial-page copy allocates a page; with nothing free the allocation evicts idle leaves.
    The matched leaf must already be locked then, or its pages would be freed while the row maps them."""
    P, n_pages = 16, 5
    cache = PagedRadixCache(page_size=P)
    pt = PageTable(n_pages=n_pages, page_size=P, max_batch_size=4, device="cpu", prefix_cache=cache)
    owner = pt.allocate()
    pt.reserve(owner, 40)                                   # 3 pages: positions 0..39
    prompt40 = toks(*range(40))
    st = finalize_cached_prompt(pt, cache, owner, prompt40, 40, 0, 0, cache.match_prefix(prompt40))
    release_cached_sequence(pt, cache, owner, st)           # the tree owns the three pages, nothing is locked
    drained = pt.allocate_pages(pt.pages_available)         # nothing free: the only evictable node is that leaf
    assert pt.pages_available == 0 and cache.evictable_page_count() == 3
    row = pt.allocate()
    prompt50 = toks(*range(50))
    with pytest.raises(RuntimeError):
        attach_cached_prefix(pt, cache, row, prompt50, 50)  # the copy cannot get a page; the prefix survives
    assert cache.total_cached_pages == 3 and cache.evictable_page_count() == 3
    assert pt.page_table_cpu[row] == [] and pt.capacity[row] == 0
    assert not set(pt.free_pages) & {p for r in pt.page_table_cpu for p in r}
    # with one free page the attach succeeds: two shared pages, a private copy of the third
    pt.free_pages_to_pool(drained[:1])
    skip, n_shared, match = attach_cached_prefix(pt, cache, row, prompt50, 50)
    assert (skip, n_shared) == (40, 2)
    src, dst = pt.take_pending_page_copies()
    assert len(src) == 1 and src[0] != dst[0]
    assert not set(pt.free_pages) & set(pt.page_table_cpu[row])
    assert cache.total_cached_pages == 3
    cache.unlock_prefill(match.last_node)


def test_tree_node_reports_its_kv_length_like_the_reference():
    from kestrel_b200.prefix_cache import TreeNode
    assert TreeNode(physical_pages=(1, 2, 3)).total_kv_length == 3     # one position per page unless told otherwise
    assert TreeNode().total_kv_length == 0
    assert TreeNode(physical_pages=(7,), kv_len=9).total_kv_length == 9
