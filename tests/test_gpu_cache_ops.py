"""GPU parity (bit-exact) of append, FP8 quantise-on-append, slot mapping, decode metadata and
copy-on-write page copies, through the public API / C ABI, against the CPU oracle and the
fixtures recorded from the reference's torch path."""

import json

import numpy as np
import pytest
import torch

from helpers import from_np
from kestrel_b200 import _native, kernels
from kestrel_b200.kv_cache import KVMemoryPool, LayerPagedCache, PagedKVCache, PageTable, copy_kv_pages
from oracle import paged_kv_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _clean_status():
    _native.device_status(torch.cuda.current_device(), clear=True)
    yield
    flags = _native.device_status(torch.cuda.current_device(), clear=True)
    assert flags[0] == 0, f"kernel diagnostics: {flags}"


def _bits(t):
    return t.contiguous().view(torch.uint8)


def test_append_golden_cases_from_reference(golden_dir):
    vec = np.load(golden_dir / "reference_vectors.npz")
    meta = json.loads((golden_dir / "reference_vectors.json").read_text())
    for m in meta["append"]:
        n, dt = m["name"], m["dtype"]
        tdt = getattr(torch, dt)
        pool = KVMemoryPool(device=DEV)
        pt = PageTable(n_pages=m["n_pages"], page_size=m["page_size"], max_batch_size=2, device=DEV)
        cache = PagedKVCache(pt, n_heads=m["heads"], head_dim=m["dim"], dtype=tdt, pool=pool)
        k = from_np(vec[f"append_{n}_k"], dt).to(DEV)
        v = from_np(vec[f"append_{n}_v"], dt).to(DEV)
        if m["fused"]:  # rebuild the strided slices of a fused projection
            B, S, H, D = k.shape
            buf = torch.zeros(B, S, 4 * H * D, dtype=tdt, device=DEV)
            buf[..., 2 * H * D:3 * H * D] = k.reshape(B, S, H * D)
            buf[..., 3 * H * D:] = v.reshape(B, S, H * D)
            k = buf[..., 2 * H * D:3 * H * D].unflatten(-1, (H, D))
            v = buf[..., 3 * H * D:].unflatten(-1, (H, D))
            assert not k.is_contiguous()
        slots = torch.from_numpy(vec[f"append_{n}_slots"]).to(DEV)
        rk, rv = cache.update(torch.zeros_like(slots), k, v, slot_mapping=slots)
        assert rk is k and rv is v
        assert torch.equal(_bits(cache.k_cache).cpu(), _bits(from_np(vec[f"append_{n}_kcache"], dt))), n
        assert torch.equal(_bits(cache.v_cache).cpu(), _bits(from_np(vec[f"append_{n}_vcache"], dt))), n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("page_size,heads,dim,tokens", [(16, 8, 128, 300), (16, 8, 64, 77), (1, 2, 8, 33), (4, 3, 6, 19)])
def test_append_matches_oracle_and_leaves_other_slots_alone(dtype, page_size, heads, dim, tokens):
    g = torch.Generator().manual_seed(tokens)
    n_pages = tokens // page_size + 6
    pool = KVMemoryPool(device=DEV)
    pt = PageTable(n_pages=n_pages, page_size=page_size, max_batch_size=2, device=DEV)
    cache = PagedKVCache(pt, n_heads=heads, head_dim=dim, dtype=dtype, pool=pool)
    poison = torch.randn(n_pages, heads, page_size, dim, generator=g).to(dtype)
    cache.k_cache.copy_(poison)
    cache.v_cache.copy_(-poison)
    k = torch.randn(tokens, 1, heads, dim, generator=g).to(dtype)
    v = torch.randn(tokens, 1, heads, dim, generator=g).to(dtype)
    slots = (torch.randperm((n_pages - 1) * page_size, generator=g)[:tokens] + page_size).view(tokens, 1)
    slots[::7] = -1  # padding rows are skipped
    want_k, want_v = poison.clone(), (-poison).clone()
    O.append(want_k, want_v, k.view(tokens, heads, dim), v.view(tokens, heads, dim), slots)
    cache.update(slots, k.to(DEV), v.to(DEV), slot_mapping=slots.to(DEV))
    assert torch.equal(_bits(cache.k_cache).cpu(), _bits(want_k))
    assert torch.equal(_bits(cache.v_cache).cpu(), _bits(want_v))


@pytest.mark.parametrize("in_dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("per_head", [False, True])
@pytest.mark.parametrize("dim", [128, 64, 10])
def test_fp8_quantise_on_append_is_code_exact(in_dtype, per_head, dim):
    g = torch.Generator().manual_seed(17 + dim)
    heads, page_size, tokens, n_pages = 8, 16, 257, 20
    x = torch.randn(2, tokens, heads, dim, generator=g)
    x = torch.where(torch.rand(x.shape, generator=g) < 0.01, x * 20, x)  # 1 % outliers x20
    x[0, 0, 0, :4] = torch.tensor([6e4, -6e4, 0.0, 1e-9])  # saturation and underflow (finite in fp16 too)
    k, v = x[0].to(in_dtype), x[1].to(in_dtype)
    if per_head:
        ks = (k.float().abs().amax(dim=(0, 2)) / 448).tolist()
        vs = (v.float().abs().amax(dim=(0, 2)) / 448).tolist()
    else:
        ks = float(k.float().abs().max() / 448)
        vs = float(v.float().abs().max() / 448)
    pool = KVMemoryPool(device=DEV)
    pt = PageTable(n_pages=n_pages, page_size=page_size, max_batch_size=2, device=DEV)
    cache = PagedKVCache(pt, n_heads=heads, head_dim=dim, dtype=torch.float8_e4m3fn, pool=pool, k_scale=ks, v_scale=vs)
    slots = (torch.randperm((n_pages - 1) * page_size, generator=g)[:tokens] + page_size).view(1, tokens)
    want_k = torch.zeros(n_pages, heads, page_size, dim, dtype=torch.uint8)
    want_v = torch.zeros_like(want_k)
    O.append(want_k, want_v, k, v, slots, k_scale=cache.k_scale_tensor.cpu(), v_scale=cache.v_scale_tensor.cpu())
    cache.update(slots, k.unsqueeze(0).to(DEV), v.unsqueeze(0).to(DEV), slot_mapping=slots.to(DEV))
    got_k = cache.k_cache.view(torch.uint8).cpu()
    got_v = cache.v_cache.view(torch.uint8).cpu()
    assert torch.equal(got_k, want_k), (got_k != want_k).sum()
    assert torch.equal(got_v, want_v)
    # independent check against torch's own cast of the same quotient
    t = (k.float() / cache.k_scale_tensor.cpu().view(-1, 1)).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    page, off = divmod(int(slots[0, 5]), page_size)
    assert torch.equal(got_k[page, :, off], t[5])


@pytest.mark.parametrize("path", ["append", "rope_append"])
def test_fp8_codes_of_every_finite_bf16_value_through_the_kernel(path):
    """All 65 280 finite bf16 values, each divided by a handful of scales (powers of two, where the quotient
    is exact, and others, where it lands on and next to rounding ties), through the append kernels: the
    codes must equal the oracle's -- and torch's own cast of the clamped fp32 quotient -- byte for byte."""
    bits = torch.arange(0x10000, dtype=torch.int32)
    bits = bits[(bits & 0x7F80) != 0x7F80]                     # drop Inf / NaN
    assert bits.numel() == 65280
    vals = bits.to(torch.int16).view(torch.bfloat16)
    heads, dim, page_size = 8, 64, 16
    per_token = heads * dim
    tokens = -(-vals.numel() // per_token)
    x = torch.zeros(tokens * per_token, dtype=torch.bfloat16)
    x[: vals.numel()] = vals
    x = x.view(tokens, heads, dim)
    n_pages = tokens // page_size + 3
    slots = torch.arange(page_size, page_size + tokens, dtype=torch.int64).view(1, tokens)
    scale_sets = [
        [1.0] * heads, [0.5] * heads, [2.0 ** -7] * heads,
        [0.0123, 1.0 / 3.0, 0.3, 7.7, 1.0 / 448.0, 3.0, 0.0491, 123.456],   # per KV head
        [5.0 / 448.0] * heads, [20.0 / 448.0] * heads,
    ]
    table = O.precompute_freqs_cis(32, 4, 1.5e6)               # Moondream: 32 of 64 dims rotated
    pos = torch.zeros(tokens, dtype=torch.int64)
    for scales in scale_sets:
        pool = KVMemoryPool(device=DEV)
        pt = PageTable(n_pages=n_pages, page_size=page_size, max_batch_size=2, device=DEV)
        cache = PagedKVCache(pt, n_heads=heads, head_dim=dim, dtype=torch.float8_e4m3fn, pool=pool,
                             k_scale=scales, v_scale=scales[::-1])
        xk = x.unsqueeze(0).to(DEV)
        xv = x.flip(0).contiguous().unsqueeze(0).to(DEV)
        if path == "append":
            cache.update(slots, xk, xv, slot_mapping=slots.to(DEV))
        else:
            # position 0 rotates by angle 0 (cos 1, sin 0): the values survive, only the sign of a zero may
            # change, so the expectation below goes through the oracle's rotary as well
            kernels.rope_reshape_and_cache(pos.to(DEV), None, xk.clone(), xv, table.to(DEV),
                                           cache.k_cache.permute(0, 2, 1, 3), cache.v_cache.permute(0, 2, 1, 3),
                                           slots.view(-1).to(DEV), "fp8_e4m3", cache.k_scale_tensor, cache.v_scale_tensor)
        want_k = torch.zeros(n_pages, heads, page_size, dim, dtype=torch.uint8)
        want_v = torch.zeros_like(want_k)
        ks, vs = torch.tensor(scales), torch.tensor(scales[::-1])
        x_k = x if path == "append" else O.rotary_embedding(pos, x, table)
        O.append(want_k, want_v, x_k, x.flip(0), slots, k_scale=ks, v_scale=vs)
        got_k = cache.k_cache.view(torch.uint8).cpu()
        got_v = cache.v_cache.view(torch.uint8).cpu()
        assert torch.equal(got_k, want_k), (scales[0], int((got_k != want_k).sum()))
        assert torch.equal(got_v, want_v), (scales[0], int((got_v != want_v).sum()))
        cast = (x_k.float() / ks.view(1, heads, 1)).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
        flat = got_k[1:1 + -(-tokens // page_size)].permute(0, 2, 1, 3).reshape(-1, heads, dim)[:tokens]
        assert torch.equal(flat, cast)


def test_append_reports_out_of_range_slot_without_faulting():
    pool = KVMemoryPool(device=DEV)
    pt = PageTable(n_pages=4, page_size=4, max_batch_size=2, device=DEV)
    cache = PagedKVCache(pt, n_heads=2, head_dim=8, dtype=torch.bfloat16, pool=pool)
    k = torch.ones(2, 1, 2, 8, dtype=torch.bfloat16, device=DEV)
    slots = torch.tensor([[5], [4 * 4 + 3]], device=DEV)
    cache.update(slots, k, k, slot_mapping=slots)
    flags = _native.device_status(torch.cuda.current_device(), clear=True)
    assert flags[0] == _native.STATUS_BAD_SLOT and flags[1] == 19
    assert cache.k_cache.float().sum().item() == 16.0


def test_slot_mapping_golden_and_oracle(golden_dir):
    vec = np.load(golden_dir / "reference_vectors.npz")
    meta = json.loads((golden_dir / "reference_vectors.json").read_text())
    for m in meta["slots"]:
        n = m["name"]
        table = torch.from_numpy(vec[f"slots_{n}_table"]).to(DEV)
        batch = torch.from_numpy(vec[f"slots_{n}_batch"]).to(DEV)
        pos = torch.from_numpy(vec[f"slots_{n}_pos"]).to(DEV)
        want = torch.from_numpy(vec[f"slots_{n}_out"])
        got = kernels.build_slot_mapping(table, batch, pos, m["page_size"])
        assert got.dtype == torch.int64 and torch.equal(got.cpu(), want)
        both = kernels.build_slot_mapping(table, batch.view(-1, 1).expand_as(pos).to(torch.int32), pos.long(), m["page_size"])
        assert torch.equal(both.cpu(), want)


def test_page_table_slot_mapping_and_metadata_through_host_api(golden_dir):
    vec = np.load(golden_dir / "reference_vectors.npz")
    pt = PageTable(n_pages=16, page_size=4, max_batch_size=8, device=DEV)
    pt.reserve(1, 9)
    pt.reserve(2, 17)
    pt.commit_block_table([1, 2])
    torch.cuda.synchronize()
    assert torch.equal(pt.page_table.cpu(), torch.from_numpy(vec["meta_table"]))
    out_pt = torch.full((2, 16), -99, dtype=torch.int32, device=DEV)
    out_sk = torch.full((2,), -1, dtype=torch.int32, device=DEV)
    pt.populate_paged_kv_metadata(batch_idx=torch.from_numpy(vec["meta_batch"]).to(DEV),
                                  input_pos=torch.from_numpy(vec["meta_pos"]).to(DEV),
                                  out_page_table=out_pt, out_seqused_k=out_sk)
    assert torch.equal(out_pt.cpu(), torch.from_numpy(vec["meta_out_table"]))
    assert torch.equal(out_sk.cpu(), torch.from_numpy(vec["meta_out_seqused"]))
    pos = torch.tensor([[0, 3, 4, 8], [16, 15, 1, 7]], dtype=torch.int32, device=DEV)
    slots = pt.build_slot_mapping(torch.tensor([1, 2], device=DEV), pos)
    want = O.build_slot_mapping(pt.page_table.cpu(), torch.tensor([1, 2]), pos.cpu(), 4)
    assert torch.equal(slots.cpu(), want)
    # int32 batch_idx, strided output rows, and a row stride wider than the live prefix
    wide = torch.full((4, 40), -7, dtype=torch.int32, device=DEV)
    sk = torch.zeros(4, dtype=torch.int32, device=DEV)
    pt.populate_paged_kv_metadata(batch_idx=torch.tensor([2, 1, 0], dtype=torch.int32, device=DEV),
                                  input_pos=torch.tensor([16, 0, 3], dtype=torch.int32, device=DEV),
                                  out_page_table=wide, out_seqused_k=sk)
    want_pt = torch.full((4, 40), -7, dtype=torch.int32)
    want_sk = torch.zeros(4, dtype=torch.int32)
    O.build_paged_kv_metadata(pt.page_table.cpu(), torch.tensor([2, 1, 0]), torch.tensor([16, 0, 3]), want_pt, want_sk, 4)
    assert torch.equal(wide.cpu(), want_pt) and torch.equal(sk.cpu(), want_sk)
    with pytest.raises(ValueError, match="insufficient page capacity"):
        pt.populate_paged_kv_metadata(batch_idx=torch.tensor([1], device=DEV),
                                      input_pos=torch.tensor([1], dtype=torch.int32, device=DEV),
                                      out_page_table=torch.zeros(1, 8, dtype=torch.int32, device=DEV), out_seqused_k=sk)
    with pytest.raises(ValueError, match="input_pos must be int32"):
        pt.populate_paged_kv_metadata(batch_idx=torch.tensor([1], device=DEV), input_pos=torch.tensor([1], device=DEV),
                                      out_page_table=wide, out_seqused_k=sk)


def test_metadata_large_rows_at_config3_width():
    """256 rows, up to 2048 live pages each (32k tokens at page 16): only the live prefix moves."""
    g = torch.Generator().manual_seed(3)
    rows, cols, P = 258, 2048, 16
    table = torch.randint(0, 1 << 20, (rows, cols), generator=g, dtype=torch.int32)
    batch = torch.randperm(rows - 1, generator=g)[:256] + 1
    pos = torch.randint(4096, 32768, (256,), generator=g, dtype=torch.int32) - 1
    out = torch.full((256, cols), -5, dtype=torch.int32)
    sk = torch.zeros(256, dtype=torch.int32)
    O.build_paged_kv_metadata(table, batch, pos, out, sk, P)
    d_out = torch.full((256, cols), -5, dtype=torch.int32, device=DEV)
    d_sk = torch.zeros(256, dtype=torch.int32, device=DEV)
    kernels.build_paged_kv_metadata(table.to(DEV), batch.to(DEV), pos.to(DEV), d_out, d_sk, P)
    assert torch.equal(d_out.cpu(), out) and torch.equal(d_sk.cpu(), sk)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float8_e4m3fn])
def test_cow_copies_pages_across_all_layers_bit_exactly(dtype):
    g = torch.Generator().manual_seed(5)
    n_layers, n_pages, heads, P, D = 5, 40, 8, 16, 64
    pool = KVMemoryPool(device=DEV)
    pt = PageTable(n_pages=n_pages, page_size=P, max_batch_size=4, device=DEV)
    kw = dict(k_scale=1.0, v_scale=1.0) if dtype == torch.float8_e4m3fn else {}
    layers = [PagedKVCache(pt, n_heads=heads, head_dim=D, dtype=dtype, pool=pool, **kw) for _ in range(n_layers)]
    for l in layers:
        for t in (l.k_cache, l.v_cache):
            raw = t.view(torch.uint8)
            raw.copy_(torch.randint(0, 255, raw.shape, generator=g, dtype=torch.uint8))
    want = [t.view(torch.uint8).cpu().clone() for l in layers for t in (l.k_cache, l.v_cache)]
    src, dst = [3, 7, 7, 30], [10, 11, 12, 39]
    O.copy_pages(want, src, dst)
    copy_kv_pages(layers + [None], src, dst)
    got = [t.view(torch.uint8).cpu() for l in layers for t in (l.k_cache, l.v_cache)]
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    with pytest.raises(ValueError, match="distinct and disjoint"):
        copy_kv_pages(layers, [1, 2], [2, 3])
    with pytest.raises(ValueError, match="out of range"):
        copy_kv_pages(layers, [1], [n_pages])


def test_cow_through_page_table_then_private_append():
    """A shared, partly filled prefix page is copied before the first private append; the
    shared page keeps its contents, the copy gets the new row."""
    P, heads, D = 16, 2, 64
    pool = KVMemoryPool(device=DEV)

    class Cache:  # minimal page-granular owner
        page_granular = True
        _free_pages_sink = None

        def evict(self, n): return 0
        def evictable_page_count(self): return 0
        def reclaimable_page_count(self): return 0

    pt = PageTable(n_pages=16, page_size=P, max_batch_size=4, device=DEV, prefix_cache=Cache())
    layer = PagedKVCache(pt, n_heads=heads, head_dim=D, dtype=torch.bfloat16, pool=pool)
    g = torch.Generator().manual_seed(1)
    prefix_len = 25  # one full page + 9 tokens
    first = pt.allocate()
    pt.reserve(first, prefix_len)
    pt.commit_block_table()
    pos = torch.arange(prefix_len, device=DEV).view(1, -1)
    k = torch.randn(1, prefix_len, heads, D, generator=g).to(torch.bfloat16).to(DEV)
    layer.update(pos, k, k, slot_mapping=pt.build_slot_mapping(torch.tensor([first], device=DEV), pos))
    shared = list(pt.page_table_cpu[first])
    second = pt.allocate()
    pt.map_pages(second, 0, shared)
    src, dst = pt.cow_page(second, 1)
    pt.commit_block_table()
    copy_kv_pages([layer], *pt.take_pending_page_copies())
    before = layer.k_cache[src].clone()
    new = torch.full((1, 1, heads, D), 3.0, dtype=torch.bfloat16, device=DEV)
    p = torch.tensor([[prefix_len]], device=DEV)
    layer.update(p, new, new, slot_mapping=pt.build_slot_mapping(torch.tensor([second], device=DEV), p))
    assert torch.equal(layer.k_cache[src], before)
    assert torch.equal(layer.k_cache[dst][:, :9], before[:, :9])
    assert (layer.k_cache[dst][:, 9] == 3.0).all()


@pytest.mark.parametrize("B,pos_1d", [(1, True), (3, False)])
def test_layer_cache_adapter_appends_like_the_cache_itself(B, pos_1d):
    """LayerPagedCache.update (the adapter of kestrel/models/moondream/runtime.py:426-481): positions given as
    [S] (one sequence) or as [B, S]; the pool bytes equal the oracle's append."""
    S, H, D, P = 5, 4, 64, 16
    pt = PageTable(n_pages=32, page_size=P, max_batch_size=B + 1, device=DEV)
    rows = [pt.allocate() for _ in range(B)]
    for r in rows:
        pt.reserve(r, 40)
    pt.commit_block_table()
    layer = LayerPagedCache(pt, n_kv_heads=H, head_dim=D, dtype=torch.bfloat16, pool=KVMemoryPool(device=DEV))
    g = torch.Generator().manual_seed(5)
    k = torch.randn(B, S, H, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, H, D, generator=g).to(torch.bfloat16)
    pos = torch.arange(7, 7 + S)
    pos_b = pos.expand(B, S).contiguous()
    slots = pt.build_slot_mapping(torch.tensor(rows, device=DEV).view(B, 1).expand(B, S).contiguous(), pos_b.to(DEV))
    got_k, got_v = layer.update(pos.to(DEV) if pos_1d else pos_b.to(DEV), k.to(DEV), v.to(DEV), slot_mapping=slots)
    want_k = torch.zeros(32, H, P, D, dtype=torch.bfloat16)
    want_v = torch.zeros_like(want_k)
    O.append(want_k, want_v, k.reshape(B * S, H, D), v.reshape(B * S, H, D), slots.cpu().reshape(-1))
    assert torch.equal(_bits(layer.cache.k_cache.cpu()), _bits(want_k))
    assert torch.equal(_bits(layer.cache.v_cache.cpu()), _bits(want_v))
    assert got_k.shape == k.shape and got_v.shape == v.shape
