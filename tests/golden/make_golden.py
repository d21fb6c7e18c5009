"""Generates the golden fixtures in this directory from the reference's own torch path.

Run once, in a container that has the reference tree:

    python tests/golden/make_golden.py --reference /path/to/kestrel

It imports the UNMODIFIED ``kestrel/kv_cache.py`` of the reference with a stub
``kestrel_kernels`` whose kernels are ``None`` -- which makes ``PagedKVCache.update``
take its torch path (``kestrel/kv_cache.py:216-220``) -- and records:

* ``append_*``        inputs and resulting pools of ``PagedKVCache.update`` (fp32 / bf16,
                      contiguous and fused-QKV-slice inputs, the two cases of the
                      reference's ``tests/test_kv_pool.py:77-178`` included);
* ``slots_*``         ``PageTable.build_slot_mapping`` results;
* ``meta_*``          the vector of ``tests/test_page_table.py:48-79`` with the outputs its
                      assertions require (checked here against the torch restatement in
                      ``kestrel/models/qwen35/runtime.py:1161-1166``);
* ``rope_vectors.npz``  the cos/sin table of ``kestrel/models/moondream/rope.py`` (Moondream's
                      geometry: 32 rotated of 64 head dims, theta 1.5e6) and fp32 rows rotated with
                      ``kestrel/ops/rotary.py:apply_rotary`` (both files loaded by path, unmodified);
* ``pool_image.npz``   raw bytes of a small bf16 pool (reference torch path) and FP8 pool (oracle codes on the
                      reference's slots) after a fixed append sequence: the pool layout / FP8 code contract;
* ``page_table_traces.json``   random op sequences on the reference ``PageTable`` with every
                      return value and the resulting host state.

The test-suite only reads the files written here; it never imports the reference.
"""

from __future__ import annotations

import argparse
import json
import random
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def import_reference(root: str):
    stub = types.ModuleType("kestrel_kernels")

    class _NS:
        pass

    rt = _NS()
    rt.cache = _NS()
    rt.cache.reshape_and_cache_flash = None
    rt.cache.build_paged_kv_metadata = None
    stub.get_runtime = lambda: rt
    sys.modules["kestrel_kernels"] = stub
    pkg = types.ModuleType("kestrel")
    pkg.__path__ = [str(Path(root) / "kestrel")]
    sys.modules["kestrel"] = pkg
    import kestrel.kv_cache as kc  # noqa: WPS433

    return kc


def to_np(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().copy()
    return t.numpy().copy()


def append_case(kc, name, *, dtype, n_pages, page_size, heads, dim, batch, seq, fused, seed, out):
    g = torch.Generator().manual_seed(seed)
    pool = kc.KVMemoryPool(device="cpu")
    pt = kc.PageTable(n_pages=n_pages, page_size=page_size, max_batch_size=batch + 1, device="cpu")
    cache = kc.PagedKVCache(pt, n_heads=heads, head_dim=dim, dtype=dtype, pool=pool)
    kv = heads * dim
    if fused:
        qsz = 2 * kv
        buf = torch.randn(batch, seq, qsz + 2 * kv, generator=g).to(dtype)
        k = buf[..., qsz:qsz + kv].reshape(batch, seq, heads, dim) if seq == 1 else buf[..., qsz:qsz + kv].unflatten(-1, (heads, dim))
        v = buf[..., qsz + kv:].unflatten(-1, (heads, dim))
    else:
        buf = None
        k = torch.randn(batch, seq, heads, dim, generator=g).to(dtype)
        v = torch.randn(batch, seq, heads, dim, generator=g).to(dtype)
    total = n_pages * page_size
    perm = torch.randperm(total - page_size, generator=g)[: batch * seq] + page_size  # page 0 stays untouched
    slots = perm.view(batch, seq).to(torch.int64)
    pos = torch.arange(batch * seq).view(batch, seq)
    cache.update(input_pos=pos, k_val=k, v_val=v, slot_mapping=slots)
    out[f"append_{name}_k"] = to_np(k.contiguous())
    out[f"append_{name}_v"] = to_np(v.contiguous())
    out[f"append_{name}_slots"] = slots.numpy()
    out[f"append_{name}_kcache"] = to_np(cache.k_cache)
    out[f"append_{name}_vcache"] = to_np(cache.v_cache)
    return {"name": name, "dtype": str(dtype).split(".")[-1], "n_pages": n_pages, "page_size": page_size,
            "heads": heads, "dim": dim, "batch": batch, "seq": seq, "fused": fused}


def reference_test_cases(kc, out):
    """The two append cases of the reference's tests/test_kv_pool.py, inputs as written there."""
    metas = []
    for name, batch, seq, slots in (("ref_fused_slice", 2, 3, [[0, 1, 2], [4, 5, 6]]),
                                    ("ref_decode_slice", 2, 1, [[2], [5]])):
        pool = kc.KVMemoryPool(device="cpu")
        pt = kc.PageTable(n_pages=3, page_size=4, max_batch_size=2, device="cpu")
        cache = kc.PagedKVCache(pt, n_heads=2, head_dim=4, dtype=torch.float32, pool=pool)
        q_size, kv_size = 16, 8
        fused = torch.arange(batch * seq * (q_size + 2 * kv_size), dtype=torch.float32).reshape(
            batch, seq, q_size + 2 * kv_size)
        if seq == 3:
            key = torch.arange(batch * seq * kv_size, dtype=torch.float32).reshape(batch, seq, 2, 4)
        else:
            key = fused[..., q_size:q_size + kv_size].reshape(batch, seq, 2, 4)
        value = fused[..., q_size + kv_size:].reshape(batch, seq, 2, 4)
        slot_mapping = torch.tensor(slots, dtype=torch.int64)
        cache.update(input_pos=torch.zeros_like(slot_mapping), k_val=key, v_val=value, slot_mapping=slot_mapping)
        out[f"append_{name}_k"] = to_np(key.contiguous())
        out[f"append_{name}_v"] = to_np(value.contiguous())
        out[f"append_{name}_slots"] = slot_mapping.numpy()
        out[f"append_{name}_kcache"] = to_np(cache.k_cache)
        out[f"append_{name}_vcache"] = to_np(cache.v_cache)
        metas.append({"name": name, "dtype": "float32", "n_pages": 3, "page_size": 4, "heads": 2, "dim": 4,
                      "batch": batch, "seq": seq, "fused": True})
    return metas


def slot_cases(kc, out):
    metas = []
    for name, page_size, n_pages, rows, lens, seed in (("p1", 1, 64, 4, [10, 3, 7, 1], 1),
                                                       ("p4", 4, 32, 3, [9, 17, 5], 2),
                                                       ("p16", 16, 40, 4, [100, 33, 16, 1], 3)):
        rng = random.Random(seed)
        pt = kc.PageTable(n_pages=n_pages, page_size=page_size, max_batch_size=rows + 2, device="cpu")
        rows_idx = []
        for L in lens:
            b = pt.allocate()
            pt.reserve(b, L)
            rows_idx.append(b)
        pt.commit_block_table()
        S = 5
        batch_idx = torch.tensor(rows_idx, dtype=torch.int64)
        positions = torch.tensor([[rng.randrange(L) for _ in range(S)] for L in lens], dtype=torch.int32)
        slots = pt.build_slot_mapping(batch_idx, positions)
        flat_b = batch_idx.view(-1, 1).expand_as(positions).contiguous()
        slots2 = pt.build_slot_mapping(flat_b, positions)
        assert torch.equal(slots, slots2)
        out[f"slots_{name}_table"] = pt.page_table.numpy().copy()
        out[f"slots_{name}_batch"] = batch_idx.numpy()
        out[f"slots_{name}_pos"] = positions.numpy()
        out[f"slots_{name}_out"] = slots.numpy()
        metas.append({"name": name, "page_size": page_size})
    return metas


def metadata_case(kc, out):
    pt = kc.PageTable(n_pages=16, page_size=4, max_batch_size=8, device="cpu")
    pt.reserve(1, 9)
    pt.reserve(2, 17)
    pt.commit_block_table([1, 2])
    batch_idx = torch.tensor([2, 1], dtype=torch.int64)
    input_pos = torch.tensor([7, 8], dtype=torch.int32)
    table = pt.page_table.clone()
    # torch restatement in the reference (qwen35 runtime): whole-row copy + input_pos + 1
    full = torch.stack([table[int(b)] for b in batch_idx.tolist()])
    seqused = input_pos + 1
    # what the reference's test requires: live prefix copied, tail keeps the sentinel
    expect = torch.full((2, 16), -99, dtype=torch.int32)
    for r in range(2):
        n = -(-int(seqused[r]) // 4)
        expect[r, :n] = full[r, :n]
    assert expect[0, :2].tolist() == table[2, :2].tolist() and expect[1, :3].tolist() == table[1, :3].tolist()
    out["meta_table"] = table.numpy()
    out["meta_batch"] = batch_idx.numpy()
    out["meta_pos"] = input_pos.numpy()
    out["meta_out_table"] = expect.numpy()
    out["meta_out_seqused"] = seqused.numpy()


def page_table_traces(kc):
    traces = []
    for seed, page_size, n_pages, rows in ((11, 1, 24, 5), (12, 4, 20, 4), (13, 16, 48, 6), (14, 16, 12, 3)):
        rng = random.Random(seed)
        pt = kc.PageTable(n_pages=n_pages, page_size=page_size, max_batch_size=rows, device="cpu")
        live: dict[int, int] = {}
        ops = []
        for _ in range(120):
            kind = rng.choice(["allocate", "reserve", "reserve", "erase", "map", "can", "commit", "get"])
            rec = {"op": kind}
            try:
                if kind == "allocate":
                    if not pt.free_batch_idx:
                        continue
                    b = pt.allocate()
                    live[b] = 0
                    rec["ret"] = b
                elif kind == "reserve":
                    if not live:
                        continue
                    b = rng.choice(sorted(live))
                    want = live[b] + rng.randrange(0, 3 * page_size + 1)
                    rec.update(b=b, n=want)
                    rec["ret"] = pt.reserve(b, want)
                    live[b] = max(live[b], want)
                elif kind == "erase":
                    if not live:
                        continue
                    b = rng.choice(sorted(live))
                    rec.update(b=b)
                    pt.erase(b)
                    del live[b]
                elif kind == "map":
                    if not live:
                        continue
                    b = rng.choice(sorted(live))
                    # 1 or 2 pages.  A count of 0 is left out on purpose: the reference's
                    # allocate_pages(0) hands out the whole free list (free_pages[-0:]), a defect
                    # the mirror does not reproduce (it returns no pages).
                    cnt = rng.randrange(1, 3)
                    rec.update(b=b, count=cnt)
                    pages = pt.allocate_pages(cnt)
                    pt.map_pages(b, len(pt.page_table_cpu[b]), pages)
                    live[b] = pt.capacity[b]
                    rec["ret"] = pages
                elif kind == "can":
                    n = rng.randrange(0, n_pages * page_size)
                    b = rng.choice([None] + sorted(live))
                    rec.update(b=b, n=n)
                    rec["ret"] = [pt.can_reserve(n, b), pt.can_reserve_with_eviction(n, b), pt.can_reserve_pages(n)]
                elif kind == "commit":
                    pt.commit_block_table()
                    rec["table"] = pt.page_table.numpy().tolist()
                elif kind == "get":
                    if not live:
                        continue
                    b = rng.choice(sorted(live))
                    rec.update(b=b)
                    rec["ret"] = pt.get_pages(b, 0, len(pt.page_table_cpu[b]))
            except RuntimeError as exc:
                rec["error"] = str(exc)
            rec["state"] = {
                "free_pages": list(pt.free_pages),
                "free_batch_idx": list(pt.free_batch_idx),
                "capacity": list(pt.capacity),
                "rows": [list(r) for r in pt.page_table_cpu],
                "blocks": pt.num_blocks_per_row.tolist(),
                "dirty": sorted(pt._dirty_rows),
            }
            ops.append(rec)
        traces.append({"seed": seed, "page_size": page_size, "n_pages": n_pages, "rows": rows, "ops": ops})
    return traces


class Tok:
    """Token double with the interface the caches key on."""

    def __init__(self, ident: int, kv: int = 1):
        self.ident, self.kv = ident, kv

    def cache_key(self):
        return (0, self.ident, self.kv)

    def kv_length(self):
        return self.kv


def radix_traces(root: str):
    """Random op sequences on the reference RadixPrefixCache (one KV position per page)."""
    from kestrel.prefix_cache import CacheNamespace, RadixPrefixCache

    traces = []
    for seed in (21, 22, 23, 24, 25):
        rng = random.Random(seed)
        freed: list[int] = []
        cache = RadixPrefixCache(free_pages_sink=lambda pages: freed.extend(pages))
        namespaces = [None, CacheNamespace(lora_id="a"), CacheNamespace(image_hash=7)]
        next_page = [100]
        handles = []      # nodes returned so far
        locks = []        # (kind, handle index) currently held
        ops = []

        def seq():
            n = rng.randrange(1, 7)
            base = rng.choice([[1, 2, 3, 4, 5, 6, 7], [1, 2, 9, 9, 9, 9, 9], [5, 5, 5, 5, 5, 5, 5]])
            ids = base[:n] if rng.random() < 0.7 else [rng.randrange(1, 6) for _ in range(n)]
            return [(i, 3 if i == 9 else 1) for i in ids]

        for _ in range(260):
            kind = rng.choice(["insert", "insert", "match", "match", "lock", "unlock", "evict", "lock_prefill"])
            rec = {"op": kind}
            if kind in ("insert", "match"):
                toks = seq()
                ns_i = rng.randrange(len(namespaces))
                objs = [Tok(i, k) for i, k in toks]
                rec.update(tokens=toks, ns=ns_i)
                if kind == "match":
                    m = cache.match_prefix(objs, namespaces[ns_i])
                    handles.append(m.last_node)
                    rec["ret"] = [list(m.matched_pages), m.matched_kv_length, m.matched_token_count,
                                  len(m.unmatched_tokens), m.last_node is not None]
                else:
                    m = cache.match_prefix(objs, namespaces[ns_i])
                    handles.append(m.last_node)
                    total = sum(k for _, k in toks)
                    reuse = rng.random() < 0.85
                    pages = list(m.matched_pages) if reuse else []
                    while len(pages) < total:
                        pages.append(next_page[0])
                        next_page[0] += 1
                    rec.update(pages=pages, reuse=reuse)
                    r = cache.insert(objs, pages, namespaces[ns_i])
                    handles.append(r.node)
                    rec["ret"] = [r.inserted_pages]
            elif kind in ("lock", "lock_prefill"):
                live = [i for i, h in enumerate(handles) if h is not None]
                if not live:
                    continue
                i = rng.choice(live)
                # only lock nodes that are still attached to a tree
                node = handles[i]
                if node.parent is None:   # a namespace root: callers never lock it
                    continue
                top = node
                while top.parent is not None:
                    top = top.parent
                if top.namespace is None or cache._trees.get(top.namespace) is not top:
                    continue
                p = node.parent
                if p is not None and node.tokens and p.children.get(node.tokens[0].cache_key()) is not node:
                    continue
                (cache.lock if kind == "lock" else cache.lock_prefill)(node)
                locks.append((kind, i))
                rec.update(h=i)
            elif kind == "unlock":
                if not locks:
                    continue
                k, i = locks.pop(rng.randrange(len(locks)))
                (cache.unlock if k == "lock" else cache.unlock_prefill)(handles[i])
                rec.update(h=i, kind=k)
            elif kind == "evict":
                n = rng.randrange(1, 6)
                del freed[:]
                got = cache.evict(n)
                rec.update(n=n, ret=[got, sorted(freed)])
            rec["counts"] = [cache.total_cached_pages, cache.evictable_page_count(), cache.reclaimable_page_count()]
            ops.append(rec)
        traces.append({"seed": seed, "ops": ops})
    return traces


def rope_vectors(root: str) -> dict[str, np.ndarray]:
    import importlib.util

    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, str(Path(root) / rel))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod

    rope = load("_ref_rope", "kestrel/models/moondream/rope.py")
    rotary = load("_ref_rotary", "kestrel/ops/rotary.py")
    out: dict[str, np.ndarray] = {}
    rot, end, theta = 32, 96, 1_500_000.0
    table = rope.precompute_freqs_cis(rot, end, theta)
    out["table"] = table.numpy()
    out["table_args"] = np.array([rot, end, theta], dtype=np.float64)
    g = torch.Generator().manual_seed(301)
    T, H, D = 7, 3, 64
    x = torch.randn(T, H, D, generator=g)
    pos = torch.randint(0, end, (T,), generator=g)
    half = rot // 2
    cos = torch.cat([table[pos, :half], table[pos, :half]], dim=-1)   # [T, rot], the cat(freqs, freqs) layout
    sin = torch.cat([table[pos, half:], table[pos, half:]], dim=-1)
    y = x.clone()
    y[..., :rot] = rotary.apply_rotary(x[..., :rot], cos, sin, unsqueeze_dim=1)
    out["x"] = x.numpy()
    out["pos"] = pos.numpy()
    out["y"] = y.numpy()
    return out


def pool_image(kc) -> dict[str, np.ndarray]:
    """The byte image of a small pool after a fixed append sequence: the contract a whole-model decode
    kernel that reads and appends the same pool relies on (``kestrel/models/moondream/runtime.py:638-644``).

    A 37-token and a 5-token prompt are appended out of fused q/k/v projections, then three batched decode
    steps follow.  bf16: slots and pool bytes come from the reference's own ``PageTable.build_slot_mapping``
    and ``PagedKVCache.update`` torch path.  FP8 e4m3: the reference's torch path refuses FP8
    (``kestrel/kv_cache.py:212-215``), so the code image is the oracle's (``satfinite(rn(x / scale))`` with the
    per-layer scalar scales the reference passes) on the reference's slots -- defined here, not pinned there.
    """
    sys.path.insert(0, str(HERE.parent.parent))
    from oracle import paged_kv_oracle as O

    n_pages, P, H, D, hq = 8, 16, 2, 64, 4
    g = torch.Generator().manual_seed(404)
    pt = kc.PageTable(n_pages=n_pages, page_size=P, max_batch_size=3, device="cpu")
    pt.free_pages = [pt.free_pages[i] for i in torch.randperm(len(pt.free_pages), generator=g).tolist()]
    cache = kc.PagedKVCache(pt, n_heads=H, head_dim=D, dtype=torch.bfloat16, pool=kc.KVMemoryPool(device="cpu"))
    k8 = torch.zeros(n_pages, H, P, D, dtype=torch.uint8)
    v8 = torch.zeros_like(k8)
    ks, vs = 0.02, 0.03
    out: dict[str, np.ndarray] = {"geometry": np.array([n_pages, P, H, D, hq], dtype=np.int64),
                                  "scales": np.array([ks, vs], dtype=np.float32)}
    rows = [pt.allocate(), pt.allocate()]
    pt.reserve(rows[0], 40)
    pt.reserve(rows[1], 8)
    pt.commit_block_table(rows)
    step = 0

    def append(batch_rows, positions):
        nonlocal step
        B, S = positions.shape
        fused = torch.randn(B, S, (hq + 2 * H) * D, generator=g).to(torch.bfloat16)
        k = fused[..., hq * D:(hq + H) * D].unflatten(-1, (H, D))
        v = fused[..., (hq + H) * D:].unflatten(-1, (H, D))
        slots = pt.build_slot_mapping(torch.tensor(batch_rows), positions)
        cache.update(input_pos=positions, k_val=k, v_val=v, slot_mapping=slots)
        O.append(k8, v8, k.reshape(-1, H, D), v.reshape(-1, H, D), slots.reshape(-1),
                 k_scale=torch.tensor([ks]), v_scale=torch.tensor([vs]))
        out[f"step{step}_rows"] = np.array(batch_rows, dtype=np.int64)
        out[f"step{step}_pos"] = positions.numpy().copy()
        out[f"step{step}_fused"] = to_np(fused)
        out[f"step{step}_slots"] = slots.numpy().copy()
        step += 1

    append([rows[0]], torch.arange(37).view(1, 37))
    append([rows[1]], torch.arange(5).view(1, 5))
    lens = [37, 5]
    for _ in range(3):
        for i, r in enumerate(rows):
            pt.reserve(r, lens[i] + 1)
        pt.commit_block_table(rows)
        append(rows, torch.tensor(lens).view(2, 1))
        lens = [n + 1 for n in lens]
    out["n_steps"] = np.array([step], dtype=np.int64)
    out["page_table"] = pt.page_table.numpy().copy()
    out["k_bf16"] = cache.k_cache.contiguous().view(torch.uint8).numpy().copy()   # raw bytes, [n_pages, H, P, D * 2]
    out["v_bf16"] = cache.v_cache.contiguous().view(torch.uint8).numpy().copy()
    out["k_e4m3"] = k8.numpy().copy()
    out["v_e4m3"] = v8.numpy().copy()
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the m87-labs/kestrel source tree")
    args = ap.parse_args()
    kc = import_reference(args.reference)
    out: dict[str, np.ndarray] = {}
    metas = {"append": [], "slots": []}
    metas["append"] += reference_test_cases(kc, out)
    metas["append"].append(append_case(kc, "f32_p4", dtype=torch.float32, n_pages=6, page_size=4, heads=2, dim=8,
                                       batch=3, seq=2, fused=False, seed=101, out=out))
    metas["append"].append(append_case(kc, "bf16_p16", dtype=torch.bfloat16, n_pages=9, page_size=16, heads=8, dim=64,
                                       batch=4, seq=1, fused=True, seed=102, out=out))
    metas["append"].append(append_case(kc, "bf16_p16_prefill", dtype=torch.bfloat16, n_pages=12, page_size=16, heads=2,
                                       dim=128, batch=2, seq=37, fused=True, seed=103, out=out))
    metas["append"].append(append_case(kc, "f32_p1", dtype=torch.float32, n_pages=40, page_size=1, heads=4, dim=16,
                                       batch=5, seq=3, fused=False, seed=104, out=out))
    metas["slots"] = slot_cases(kc, out)
    metadata_case(kc, out)
    np.savez_compressed(HERE / "reference_vectors.npz", **out)
    (HERE / "reference_vectors.json").write_text(json.dumps(metas, indent=1))
    (HERE / "page_table_traces.json").write_text(json.dumps(page_table_traces(kc)))
    (HERE / "radix_traces.json").write_text(json.dumps(radix_traces(args.reference)))
    np.savez_compressed(HERE / "rope_vectors.npz", **rope_vectors(args.reference))
    np.savez_compressed(HERE / "pool_image.npz", **pool_image(kc))
    print("wrote", sorted(p.name for p in HERE.iterdir()))


if __name__ == "__main__":
    main()
