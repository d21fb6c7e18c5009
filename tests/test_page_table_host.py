"""Host-side KV pool / page table behaviour: replay of traces recorded from the reference's
PageTable plus the cases its own tests/test_kv_pool.py and tests/test_page_table.py pin."""

import gc
import json
import threading

import pytest
import torch

from kestrel_b200.kv_cache import (KVMemoryPool, LayerPagedCache, PagedKVCache, PagedKVLayerSpec, PageTable,
                                   _flatten_bshd_tokens, allocate_paged_kv_layers)


def _state(pt):
    return {
        "free_pages": list(pt.free_pages),
        "free_batch_idx": list(pt.free_batch_idx),
        "capacity": list(pt.capacity),
        "rows": [list(r) for r in pt.page_table_cpu],
        "blocks": pt.num_blocks_per_row.tolist(),
        "dirty": sorted(pt._dirty_rows),
    }


def test_traces_recorded_from_reference_replay_identically(golden_dir):
    traces = json.loads((golden_dir / "page_table_traces.json").read_text())
    assert len(traces) == 4
    n_ops = 0
    for tr in traces:
        pt = PageTable(n_pages=tr["n_pages"], page_size=tr["page_size"], max_batch_size=tr["rows"], device="cpu")
        for i, rec in enumerate(tr["ops"]):
            op = rec["op"]
            err = None
            ret = None
            try:
                if op == "allocate":
                    ret = pt.allocate()
                elif op == "reserve":
                    ret = pt.reserve(rec["b"], rec["n"])
                elif op == "erase":
                    pt.erase(rec["b"])
                elif op == "map":
                    pages = pt.allocate_pages(rec["count"])
                    pt.map_pages(rec["b"], len(pt.page_table_cpu[rec["b"]]), pages)
                    ret = pages
                elif op == "can":
                    ret = [pt.can_reserve(rec["n"], rec["b"]), pt.can_reserve_with_eviction(rec["n"], rec["b"]),
                           pt.can_reserve_pages(rec["n"])]
                elif op == "commit":
                    pt.commit_block_table()
                    assert pt.page_table.numpy().tolist() == rec["table"], (tr["seed"], i)
                elif op == "get":
                    ret = pt.get_pages(rec["b"], 0, len(pt.page_table_cpu[rec["b"]]))
            except RuntimeError as exc:
                err = str(exc)
            assert err == rec.get("error"), (tr["seed"], i, op)
            if "ret" in rec:
                assert ret == rec["ret"], (tr["seed"], i, op)
            assert _state(pt) == rec["state"], (tr["seed"], i, op)
            n_ops += 1
    assert n_ops > 300


def test_initial_layout_reserves_row0_and_page0():
    pt = PageTable(n_pages=6, page_size=2, max_batch_size=3, device="cpu")
    assert pt.page_table[0].tolist() == [0] * 6
    assert pt.page_table[1].tolist() == [-1] * 6
    assert pt.free_pages == [5, 4, 3, 2, 1] and pt.free_batch_idx == [2, 1]
    assert pt.allocate() == 1


def test_pool_accounting_budget_and_release():
    pool = KVMemoryPool(device="cpu")
    pt = PageTable(n_pages=4, page_size=1, max_batch_size=2, device="cpu")
    cache = PagedKVCache(pt, n_heads=2, head_dim=8, dtype=torch.float32, pool=pool)
    assert pool.allocated_bytes == 2 * 4 * 2 * 1 * 8 * 4
    assert tuple(cache.k_cache.shape) == (4, 2, 1, 8)
    assert pool.device == torch.device("cpu")
    del cache
    gc.collect()
    assert pool.allocated_bytes == 0
    small = KVMemoryPool(device="cpu", budget_bytes=128)
    with pytest.raises(MemoryError, match="budget exceeded"):
        PagedKVCache(pt, n_heads=4, head_dim=16, dtype=torch.float32, pool=small)
    assert small.allocated_bytes == 0
    with pytest.raises(ValueError, match="non-negative"):
        KVMemoryPool(device="cpu", budget_bytes=-1)


def test_pool_budget_is_thread_safe():
    pt = PageTable(n_pages=4, page_size=1, max_batch_size=2, device="cpu")
    per_layer = 2 * 4 * 2 * 1 * 8 * 4
    pool = KVMemoryPool(device="cpu", budget_bytes=3 * per_layer)
    keep, errors = [], []

    def work():
        try:
            keep.append(PagedKVCache(pt, n_heads=2, head_dim=8, dtype=torch.float32, pool=pool))
        except MemoryError:
            errors.append(1)

    threads = [threading.Thread(target=work) for _ in range(8)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert len(keep) == 3 and len(errors) == 5 and pool.allocated_bytes == 3 * per_layer


def test_fp8_cache_requires_scales_and_keeps_float_scales():
    pool = KVMemoryPool(device="cpu")
    pt = PageTable(n_pages=4, page_size=16, max_batch_size=2, device="cpu")
    with pytest.raises(ValueError, match="requires per-layer k/v scales"):
        PagedKVCache(pt, n_heads=2, head_dim=8, dtype=torch.float8_e4m3fn, pool=pool)
    c = PagedKVCache(pt, n_heads=2, head_dim=8, dtype=torch.float8_e4m3fn, pool=pool, k_scale=0.5, v_scale=0.25)
    assert c.quantized and c.k_scale == 0.5 and c.v_scale == 0.25
    assert c.k_scale_tensor.dtype == torch.float32 and c.k_scale_tensor.ndim == 0
    ph = PagedKVCache(pt, n_heads=2, head_dim=8, dtype=torch.float8_e4m3fn, pool=pool, k_scale=[0.5, 1.0],
                      v_scale=[0.25, 2.0])
    assert ph.k_scale_tensor.tolist() == [0.5, 1.0] and ph.k_scale is ph.k_scale_tensor
    plain = PagedKVCache(pt, n_heads=2, head_dim=8, dtype=torch.bfloat16, pool=pool)
    assert not plain.quantized and plain.k_scale == 1.0
    layers = allocate_paged_kv_layers(layer_specs=[PagedKVLayerSpec(2, 8), None], page_table=pt, pool=pool,
                                      dtype=torch.bfloat16)
    assert layers[1] is None and tuple(layers[0].v_cache.shape) == (4, 2, 16, 8)


def test_update_has_no_cpu_fallback():
    pool = KVMemoryPool(device="cpu")
    pt = PageTable(n_pages=3, page_size=4, max_batch_size=2, device="cpu")
    c = PagedKVCache(pt, n_heads=2, head_dim=4, dtype=torch.float32, pool=pool)
    k = torch.zeros(1, 1, 2, 4)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        c.update(torch.zeros(1, 1, dtype=torch.long), k, k, slot_mapping=torch.zeros(1, 1, dtype=torch.long))
    with pytest.raises(ValueError, match="slot_mapping must match input_pos shape"):
        c.update(torch.zeros(1, 1, dtype=torch.long), k, k, slot_mapping=torch.zeros(2, dtype=torch.long))
    # empty appends are a no-op and return their inputs
    e = torch.zeros(0, 1, 2, 4)
    assert c.update(torch.zeros(0, 1, dtype=torch.long), e, e, slot_mapping=torch.zeros(0, 1, dtype=torch.long))[0] is e
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        pt.build_slot_mapping(torch.tensor([1]), torch.zeros(1, 1, dtype=torch.long))


def test_flatten_accepts_fused_slices_and_rejects_gaps():
    fused = torch.arange(2 * 3 * 32, dtype=torch.float32).reshape(2, 3, 32)
    v = fused[..., 24:].reshape(2, 3, 2, 4)
    flat = _flatten_bshd_tokens("v", v)
    assert flat.shape == (6, 2, 4) and flat.stride() == (32, 4, 1)
    assert torch.equal(flat, v.reshape(6, 2, 4))
    dec = torch.arange(2 * 32, dtype=torch.float32).reshape(2, 1, 32)[..., 16:24].reshape(2, 1, 2, 4)
    assert _flatten_bshd_tokens("k", dec).stride(0) == 32
    with pytest.raises(ValueError, match="must have shape"):
        _flatten_bshd_tokens("k", torch.zeros(2, 3, 4))
    with pytest.raises(ValueError, match="compact across heads"):
        _flatten_bshd_tokens("k", torch.zeros(2, 3, 2, 8)[..., ::2])
    with pytest.raises(ValueError, match="cannot be flattened"):
        _flatten_bshd_tokens("k", torch.zeros(2, 4, 2, 4)[:, :3])


def test_map_pages_sequential_and_erase_with_cached_prefix():
    pt = PageTable(n_pages=100, page_size=1, max_batch_size=10, device="cpu")
    b = pt.allocate()
    pages = pt.allocate_pages(10)
    assert pages == list(range(10, 0, -1)) and pt.pages_available == 89
    pt.map_pages(b, 0, pages[:5])
    with pytest.raises(AssertionError, match="sequentially"):
        pt.map_pages(b, 3, pages[5:])
    pt.map_pages(b, 5, pages[5:])
    assert pt.capacity[b] == 10 and pt.page_table_cpu[b] == pages
    assert pt.get_pages(b, 2, 4) == pages[2:4] and pt.get_pages(b, 3, 3) == []
    pt.erase(b, cached_page_count=4)
    assert pt.pages_available == 89 + 6 and b in pt.free_batch_idx
    pt.free_pages_to_pool(tuple(pages[:4]))
    assert pt.pages_available == 99
    with pytest.raises(RuntimeError, match="Cannot allocate 200 pages: 99 available"):
        pt.allocate_pages(200)


def test_commit_uploads_only_when_dirty(monkeypatch):
    pt = PageTable(n_pages=16, page_size=4, max_batch_size=6, device="cpu")
    a, b = pt.allocate(), pt.allocate()
    pt.reserve(a, 5)
    pt.reserve(b, 9)
    assert pt._dirty_rows == {a, b}
    calls = []
    real = pt._page_table_buffer.copy_to_gpu
    monkeypatch.setattr(pt._page_table_buffer, "copy_to_gpu", lambda n=None: (calls.append(n), real(n))[1])
    pt.commit_block_table([a])
    assert calls == [a + 1] and pt._dirty_rows == {b}
    pt.commit_block_table([a])
    assert calls == [a + 1]
    pt.commit_block_table()
    assert calls == [a + 1, b + 1] and pt._dirty_rows == set()
    assert pt.page_table[b, :3].tolist() == pt.page_table_cpu[b]


class _FakeCache:
    """Prefix cache double: owns pages, evicts in insertion order."""

    def __init__(self, page_granular=False):
        self.page_granular = page_granular
        self.pages = []
        self.locked = False
        self._free_pages_sink = None

    def evict(self, needed):
        if self.locked:
            return 0
        out, self.pages = self.pages[:needed], self.pages[needed:]
        self._free_pages_sink(out)
        return len(out)

    def evictable_page_count(self):
        return 0 if self.locked else len(self.pages)

    def reclaimable_page_count(self):
        return self.evictable_page_count()


def test_prefix_cache_hookup_and_eviction():
    with pytest.raises(AssertionError, match="requires page_size=1"):
        PageTable(n_pages=8, page_size=16, max_batch_size=2, device="cpu", prefix_cache=_FakeCache())
    cache = _FakeCache()
    pt = PageTable(n_pages=8, page_size=1, max_batch_size=4, device="cpu", prefix_cache=cache)
    assert pt.prefix_cache is cache and cache._free_pages_sink == pt.free_pages_to_pool
    cache.pages = pt.allocate_pages(5)
    assert pt.pages_available == 2
    assert not pt.can_reserve(4) and pt.can_reserve_with_eviction(4) and pt.can_reserve_pages(7)
    assert not pt.can_reserve_pages(8)
    b = pt.allocate()
    assert pt.reserve(b, 4) and len(cache.pages) == 3
    cache.locked = True
    with pytest.raises(RuntimeError, match="All cached prefixes are locked"):
        pt.reserve(b, 9)
    with pytest.raises(RuntimeError, match="all cached prefixes are locked"):
        pt.allocate_pages(3)


def test_cow_page_remaps_row_and_queues_copy():
    cache = _FakeCache(page_granular=True)
    pt = PageTable(n_pages=12, page_size=16, max_batch_size=4, device="cpu", prefix_cache=cache)
    shared = pt.allocate_pages(3)
    cache.pages = list(shared)
    r1, r2 = pt.allocate(), pt.allocate()
    for r in (r1, r2):
        pt.map_pages(r, 0, shared)
    pt.commit_block_table()
    src, dst = pt.cow_page(r1, 2)
    assert src == shared[2] and dst not in shared
    assert pt.page_table_cpu[r1] == shared[:2] + [dst] and pt.page_table_cpu[r2] == shared
    assert r1 in pt._dirty_rows and r2 not in pt._dirty_rows
    pt.reserve(r1, 3 * 16 + 5)
    assert len(pt.page_table_cpu[r1]) == 4
    assert pt.take_pending_page_copies() == ([src], [dst]) and pt.take_pending_page_copies() == ([], [])
    before = pt.pages_available
    pt.erase(r1, cached_page_count=2)
    assert pt.pages_available == before + 2  # the private copy and the suffix page
    pt.erase(r2, cached_page_count=3)
    assert pt.pages_available == before + 2
    with pytest.raises(IndexError):
        pt.cow_page(r1, 0)


def test_common_prefix_pages_counts_the_shared_leading_pages():
    """Rows attached to one cached prefix map the same leading pages; the count feeds flash_attn_fwd's
    shared_prefix_pages."""
    pt = PageTable(n_pages=256, page_size=16, max_batch_size=8, device="cpu")
    owner = pt.allocate()
    pt.reserve(owner, 729)
    shared = list(pt.page_table_cpu[owner])[:45]
    rows = []
    for extra in (10, 40, 100):
        r = pt.allocate()
        pt.map_pages(r, 0, shared)
        pt.reserve(r, 729 + extra)
        rows.append(r)
    assert pt.common_prefix_pages(rows) == 45
    assert pt.common_prefix_pages(rows, min_tokens=700) == 43   # only pages entirely below 700 tokens
    assert pt.common_prefix_pages(rows, min_tokens=0) == 0
    assert pt.common_prefix_pages(rows[:1]) == 0                # one row shares with nobody
    assert pt.common_prefix_pages([]) == 0
    other = pt.allocate()
    pt.reserve(other, 100)
    assert pt.common_prefix_pages(rows + [other]) == 0
    # rows that agree on the first pages only
    a, b = pt.allocate(), pt.allocate()
    pt.map_pages(a, 0, shared[:10])
    pt.map_pages(b, 0, shared[:7])
    pt.reserve(a, 400)
    pt.reserve(b, 400)
    assert pt.common_prefix_pages([a, b]) == 7


def test_layer_cache_adapter_checks_shapes_before_the_append():
    """The checks of _LayerPagedCache.update (kestrel/models/moondream/runtime.py:451-481), on CPU tensors:
    they fire before any kernel is reached."""
    pt = PageTable(n_pages=8, page_size=4, max_batch_size=2, device="cpu")
    layer = LayerPagedCache(pt, n_kv_heads=2, head_dim=8, dtype=torch.float32, pool=KVMemoryPool(device="cpu"))
    assert layer.cache.k_cache.shape == (8, 2, 4, 8)
    k = torch.zeros(2, 3, 2, 8)
    slots = torch.zeros(2, 3, dtype=torch.int64)
    with pytest.raises(ValueError, match="k_val and v_val must match shape"):
        layer.update(torch.arange(3), k, torch.zeros(2, 3, 2, 4), slot_mapping=slots)
    with pytest.raises(ValueError, match="Unsupported position shape"):
        layer.update(torch.zeros(3, 3, dtype=torch.int64), k, k, slot_mapping=slots)
    with pytest.raises(ValueError, match="does not match position tensor"):
        layer.update(torch.arange(4), k, k, slot_mapping=slots)
    # well-formed arguments get as far as the kernel, which refuses CPU tensors (no fallback)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        layer.update(torch.arange(3).expand(2, 3), k, k, slot_mapping=slots)


def test_allocating_zero_pages_takes_nothing():
    pt = PageTable(n_pages=8, page_size=4, max_batch_size=3, device="cpu")
    before = list(pt.free_pages)
    assert pt.allocate_pages(0) == []
    assert pt.free_pages == before


def test_page_granular_cache_must_use_the_tables_page_size():
    from kestrel_b200.prefix_cache import PagedRadixCache
    with pytest.raises(AssertionError):
        PageTable(n_pages=8, page_size=16, max_batch_size=3, device="cpu", prefix_cache=PagedRadixCache(page_size=4))
    PageTable(n_pages=8, page_size=16, max_batch_size=3, device="cpu", prefix_cache=PagedRadixCache(page_size=16))
