"""The drop-in claim, executed: the reference's UNMODIFIED ``kestrel/kv_cache.py``, ``kestrel/ops/attention.py``
and ``kestrel/prefix_cache`` (staged byte copies, ``oracle/stage_reference.py``) run on this library through
``install_as_kestrel_kernels()`` -- their ``KVMemoryPool``, ``PagedKVCache.update``,
``PageTable.populate_paged_kv_metadata`` / ``build_slot_mapping`` / ``commit_block_table``, ``paged_attention``
and ``RadixPrefixCache`` -- and every result is compared with the CPU oracle.  Nothing of
``kestrel_b200.kv_cache`` / ``attention`` / ``prefix_cache`` (the hand-written mirror) is used here.
"""

from __future__ import annotations

import math

import pytest
import torch

from oracle import paged_kv_oracle as O
from tests.helpers import import_staged_reference

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    mods = import_staged_reference()
    if mods is None:
        pytest.skip("reference modules are not staged (python oracle/stage_reference.py)")
    kc, attn, pc = mods
    import kestrel_b200.kernels as shim

    # the reference bound OUR entry points at import time
    assert kc.reshape_and_cache_flash_cuda is shim.reshape_and_cache_flash
    assert kc.build_paged_kv_metadata_runtime is shim.build_paged_kv_metadata
    assert "oracle/_ref/kestrel" in kc.__file__.replace("\\", "/")
    return kc, attn, pc


DEV = "cuda"


def _status_clean():
    from kestrel_b200 import _native
    flags = _native.device_status(torch.cuda.current_device(), clear=True)
    assert flags[0] == 0, flags


def test_reference_append_cases_on_cuda(ref):
    """The two append vectors of the reference's tests/test_kv_pool.py:77-178 (strided V out of a fused
    projection; batched decode rows with stride(0) > stride(1)), on the GPU through the reference's class."""
    kc, _, _ = ref
    q_size, kv_size = 16, 8
    for batch, seq_len, slots in ((2, 3, [[0, 1, 2], [4, 5, 6]]), (2, 1, [[2], [5]])):
        pool = kc.KVMemoryPool(device=DEV)
        pt = kc.PageTable(n_pages=3, page_size=4, max_batch_size=2, device=DEV)
        cache = kc.PagedKVCache(pt, n_heads=2, head_dim=4, dtype=torch.float32, pool=pool)
        fused = torch.arange(batch * seq_len * (q_size + 2 * kv_size), dtype=torch.float32, device=DEV).reshape(
            batch, seq_len, q_size + 2 * kv_size)
        if seq_len == 3:
            key = torch.arange(batch * seq_len * kv_size, dtype=torch.float32, device=DEV).reshape(batch, seq_len, 2, 4)
        else:
            key = fused[..., q_size:q_size + kv_size].reshape(batch, seq_len, 2, 4)
        value = fused[..., q_size + kv_size:].reshape(batch, seq_len, 2, 4)
        assert value.stride(2) == 4 and value.stride(3) == 1 and max(value.stride(0), value.stride(1)) > 8
        slot_mapping = torch.tensor(slots, dtype=torch.int64, device=DEV)
        out = cache.update(input_pos=torch.zeros_like(slot_mapping), k_val=key, v_val=value, slot_mapping=slot_mapping)
        assert out[0] is key and out[1] is value
        exp_k = torch.zeros(3, 2, 4, 4)
        exp_v = torch.zeros(3, 2, 4, 4)
        O.append(exp_k, exp_v, key.cpu().reshape(-1, 2, 4), value.cpu().reshape(-1, 2, 4), slot_mapping.cpu().view(-1))
        assert torch.equal(cache.k_cache.cpu(), exp_k) and torch.equal(cache.v_cache.cpu(), exp_v)
    _status_clean()


def test_reference_metadata_vector_on_cuda(ref):
    """tests/test_page_table.py:48-79 through the reference's PageTable: seqused_k = input_pos + 1, live
    prefix copied, tail untouched (sentinel -99)."""
    kc, _, _ = ref
    pt = kc.PageTable(n_pages=16, page_size=4, max_batch_size=8, device=DEV)
    pt.reserve(1, 9)
    pt.reserve(2, 17)
    pt.commit_block_table([1, 2])
    batch_idx = torch.tensor([2, 1], dtype=torch.int64, device=DEV)
    input_pos = torch.tensor([7, 8], dtype=torch.int32, device=DEV)
    out_pt = torch.full((2, pt.n_pages), -99, dtype=torch.int32, device=DEV)
    out_sk = torch.full((2,), -1, dtype=torch.int32, device=DEV)
    pt.populate_paged_kv_metadata(batch_idx=batch_idx, input_pos=input_pos, out_page_table=out_pt, out_seqused_k=out_sk)
    table = pt.page_table.cpu()
    assert out_sk.cpu().tolist() == [8, 9]
    got = out_pt.cpu()
    assert torch.equal(got[0, :2], table[2, :2]) and torch.equal(got[1, :3], table[1, :3])
    assert (got[0, 2:] == -99).all() and (got[1, 3:] == -99).all()
    exp_pt = torch.full((2, pt.n_pages), -99, dtype=torch.int32)
    exp_sk = torch.full((2,), -1, dtype=torch.int32)
    O.build_paged_kv_metadata(table, batch_idx.cpu(), input_pos.cpu(), exp_pt, exp_sk, 4)
    assert torch.equal(got, exp_pt) and torch.equal(out_sk.cpu(), exp_sk)
    _status_clean()


def _decode_problem(kc, *, kv_dtype, P, D, hq, hkv, lengths, seed, k_scale=None, v_scale=None, sq=1):
    """Contexts appended through the reference's PagedKVCache.update, then one step of ``sq`` new tokens."""
    g = torch.Generator().manual_seed(seed)
    B = len(lengths)
    n_pages = sum(-(-(L + sq) // P) for L in lengths) + 8
    pool = kc.KVMemoryPool(device=DEV)
    pt = kc.PageTable(n_pages=n_pages, page_size=P, max_batch_size=B + 1, device=DEV)
    order = torch.randperm(len(pt.free_pages), generator=g).tolist()
    pt.free_pages = [pt.free_pages[i] for i in order]         # scattered pages
    kw = dict(k_scale=k_scale, v_scale=v_scale) if kv_dtype == torch.float8_e4m3fn else {}
    cache = kc.PagedKVCache(pt, n_heads=hkv, head_dim=D, dtype=kv_dtype, pool=pool, **kw)
    fp8 = kv_dtype == torch.float8_e4m3fn
    mk = torch.zeros(n_pages, hkv, P, D, dtype=torch.uint8 if fp8 else torch.float32)
    mv = torch.zeros_like(mk)
    ks = torch.full((hkv,), float(k_scale)) if fp8 else None
    vs = torch.full((hkv,), float(v_scale)) if fp8 else None
    rows = [pt.allocate() for _ in lengths]
    for r, L in zip(rows, lengths):
        pt.reserve(r, L + sq)
    pt.commit_block_table(rows)
    table = pt._page_table_cpu_tensor.clone()
    for r, L in zip(rows, lengths):
        k = torch.randn(1, L, hkv, D, generator=g).to(torch.bfloat16)
        v = torch.randn(1, L, hkv, D, generator=g).to(torch.bfloat16)
        pos = torch.arange(L).view(1, L)
        slots = pt.build_slot_mapping(torch.tensor([r], device=DEV), pos.to(DEV))     # the reference's torch ops
        ref_slots = O.build_slot_mapping(table, torch.tensor([r]), pos, P)
        assert torch.equal(slots.cpu(), ref_slots)
        cache.update(input_pos=pos.to(DEV), k_val=k.to(DEV), v_val=v.to(DEV), slot_mapping=slots)
        O.append(mk, mv, k[0], v[0], ref_slots.view(-1), k_scale=ks, v_scale=vs)
    # the step: sq new tokens per sequence out of a fused projection
    fused = torch.randn(B, sq, (hq + 2 * hkv) * D, generator=g).to(torch.bfloat16).to(DEV)
    q, k, v = fused.split([hq * D, hkv * D, hkv * D], dim=-1)
    q, k, v = q.view(B, sq, hq, D), k.view(B, sq, hkv, D), v.view(B, sq, hkv, D)
    pos = torch.tensor(lengths).view(B, 1) + torch.arange(sq).view(1, sq)
    batch_idx = torch.tensor(rows, device=DEV)
    slots = pt.build_slot_mapping(batch_idx, pos.to(DEV))
    cache.update(input_pos=pos.to(DEV), k_val=k, v_val=v, slot_mapping=slots)
    ref_slots = O.build_slot_mapping(table, torch.tensor(rows), pos, P)
    assert torch.equal(slots.cpu(), ref_slots)
    O.append(mk, mv, k.cpu().reshape(B * sq, hkv, D), v.cpu().reshape(B * sq, hkv, D), ref_slots.view(-1),
             k_scale=ks, v_scale=vs)
    meta_pt = torch.zeros(B, n_pages, dtype=torch.int32, device=DEV)
    meta_sk = torch.zeros(B, dtype=torch.int32, device=DEV)
    pt.populate_paged_kv_metadata(batch_idx=batch_idx, input_pos=pos[:, -1].to(torch.int32).to(DEV),
                                  out_page_table=meta_pt, out_seqused_k=meta_sk)
    got_k = cache.k_cache.view(torch.uint8).cpu() if fp8 else cache.k_cache.float().cpu()
    got_v = cache.v_cache.view(torch.uint8).cpu() if fp8 else cache.v_cache.float().cpu()
    assert torch.equal(got_k, mk) and torch.equal(got_v, mv), "pool bytes differ from the oracle"
    return dict(cache=cache, pt=pt, q=q, meta_pt=meta_pt, meta_sk=meta_sk, mk=mk, mv=mv, ks=ks, vs=vs, rows=rows)


def _check(out, want):
    err = (out.float().cpu() - want).abs().max().item()
    assert err <= 2e-2, f"max abs error {err}"


@pytest.mark.parametrize("P,D", [(16, 128), (1, 64), (16, 64)])
def test_reference_bf16_decode_step(ref, P, D):
    kc, attn, _ = ref
    pr = _decode_problem(kc, kv_dtype=torch.bfloat16, P=P, D=D, hq=32, hkv=8, lengths=[300, 17, 64, 129, 1], seed=3)
    out = attn.paged_attention(pr["q"].transpose(1, 2), paged_kv_layer=pr["cache"], page_table=pr["meta_pt"],
                               paged_kv_seqlens_k=pr["meta_sk"], scaling=1.0 / math.sqrt(D))
    assert out.shape == pr["q"].shape and out.dtype == torch.bfloat16
    want = O.paged_attention(pr["q"].cpu().float(), pr["mk"], pr["mv"], pr["meta_pt"].cpu(), pr["meta_sk"].cpu())
    _check(out, want)
    _status_clean()


def test_reference_fp8_decode_step_with_per_layer_scalar_scales(ref):
    """FP8 pools as the reference builds them: python-float per-layer scales, 0-dim fp32 scale tensors for the
    append, ``k_scale`` / ``v_scale`` floats read by paged_attention (kestrel/kv_cache.py:164-181)."""
    kc, attn, _ = ref
    pr = _decode_problem(kc, kv_dtype=torch.float8_e4m3fn, P=16, D=128, hq=32, hkv=8, lengths=[257, 40, 16, 1023],
                         seed=5, k_scale=0.0123, v_scale=0.0171)
    cache = pr["cache"]
    assert cache.quantized and isinstance(cache.k_scale, float) and cache.k_scale_tensor.ndim == 0
    out = attn.paged_attention(pr["q"].transpose(1, 2), paged_kv_layer=cache, page_table=pr["meta_pt"],
                               paged_kv_seqlens_k=pr["meta_sk"], scaling=1.0 / math.sqrt(128))
    want = O.paged_attention(pr["q"].cpu().float(), pr["mk"], pr["mv"], pr["meta_pt"].cpu(), pr["meta_sk"].cpu(),
                             k_scale=pr["ks"], v_scale=pr["vs"])
    _check(out, want)
    _status_clean()


def test_reference_fp8_decode_step_in_the_references_own_fp8_geometry(ref):
    """FP8 KV exists in the reference only with page size 1 (kestrel/models/moondream/runtime.py:645-663), on
    Moondream's MHA 32/32 heads of 64: rows of 64 bytes.  Same flow as above through the reference's classes."""
    kc, attn, _ = ref
    pr = _decode_problem(kc, kv_dtype=torch.float8_e4m3fn, P=1, D=64, hq=32, hkv=32, lengths=[130, 17, 64, 700],
                         seed=6, k_scale=0.0141, v_scale=0.0113)
    out = attn.paged_attention(pr["q"].transpose(1, 2), paged_kv_layer=pr["cache"], page_table=pr["meta_pt"],
                               paged_kv_seqlens_k=pr["meta_sk"], scaling=1.0 / math.sqrt(64))
    want = O.paged_attention(pr["q"].cpu().float(), pr["mk"], pr["mv"], pr["meta_pt"].cpu(), pr["meta_sk"].cpu(),
                             k_scale=pr["ks"], v_scale=pr["vs"])
    _check(out, want)
    _status_clean()


def test_reference_multi_query_seqlens_q_packed_and_window_calls(ref):
    kc, attn, _ = ref
    D, sq = 128, 4
    pr = _decode_problem(kc, kv_dtype=torch.bfloat16, P=16, D=D, hq=32, hkv=8, lengths=[90, 300, 33], seed=7, sq=sq)
    q, B = pr["q"], 3
    args = dict(paged_kv_layer=pr["cache"], page_table=pr["meta_pt"], paged_kv_seqlens_k=pr["meta_sk"],
                scaling=1.0 / math.sqrt(D))
    ref_args = (pr["mk"], pr["mv"], pr["meta_pt"].cpu(), pr["meta_sk"].cpu())
    # padded verify step
    _check(attn.paged_attention(q.transpose(1, 2), **args), O.paged_attention(q.cpu().float(), *ref_args))
    # fewer valid query rows in some sequences
    sq_used = torch.tensor([4, 2, 3], dtype=torch.int32)
    out = attn.paged_attention(q.transpose(1, 2), paged_kv_seqlens_q=sq_used.to(DEV), **args)
    want = O.paged_attention(q.cpu().float(), *ref_args, seqused_q=sq_used)
    for b in range(B):
        _check(out[b, : int(sq_used[b])], want[b, : int(sq_used[b])])
    # packed rows: the reference flattens [B, Hq, S, D] -> [B*S, Hq, D] and passes cu_seqlens_q only
    cu = torch.arange(0, (B + 1) * sq, sq, dtype=torch.int32, device=DEV)
    out = attn.paged_attention(q.transpose(1, 2), cu_seqlens_q=cu, **args)
    assert out.shape == q.shape
    _check(out, O.paged_attention(q.cpu().float(), *ref_args))
    # sliding window (kestrel/ops/attention.py:78-82: window_size_left = W - 1, right = 0, causal False)
    out = attn.paged_attention(q.transpose(1, 2), sliding_window=24, **args)
    _check(out, O.paged_attention(q.cpu().float(), *ref_args, window_left=23))
    _status_clean()


def test_reference_packed_single_row_sequences_stay_correct(ref):
    """A packed batch of one-row sequences (what a decode step looks like through ``cu_seqlens_q``): the
    shim gets no ``max_seqlen_q`` from the reference's call."""
    kc, attn, _ = ref
    D = 128
    lengths = [50 + 37 * i for i in range(12)]
    pr = _decode_problem(kc, kv_dtype=torch.bfloat16, P=16, D=D, hq=32, hkv=8, lengths=lengths, seed=11)
    cu = torch.arange(0, len(lengths) + 1, dtype=torch.int32, device=DEV)
    out = attn.paged_attention(pr["q"].transpose(1, 2), paged_kv_layer=pr["cache"], page_table=pr["meta_pt"],
                               paged_kv_seqlens_k=pr["meta_sk"], scaling=1.0 / math.sqrt(D), cu_seqlens_q=cu)
    want = O.paged_attention(pr["q"].cpu().float(), pr["mk"], pr["mv"], pr["meta_pt"].cpu(), pr["meta_sk"].cpu())
    _check(out, want)
    _status_clean()


def test_reference_radix_cache_drives_the_kernels_at_page_size_one(ref):
    """The reference's RadixPrefixCache + PageTable (page size 1, its only mode) share a cached prompt between
    two requests; the second request's attention over mapped + own pages matches the oracle."""
    kc, attn, pc = ref
    hq, hkv, D, P = 8, 8, 64, 1
    g = torch.Generator().manual_seed(13)

    class Tok:
        def __init__(self, i): self.i = i
        def cache_key(self): return (0, self.i)
        def kv_length(self): return 1

    cache_tree = pc.RadixPrefixCache()
    n_pages = 256
    pool = kc.KVMemoryPool(device=DEV)
    pt = kc.PageTable(n_pages=n_pages, page_size=P, max_batch_size=4, device=DEV, prefix_cache=cache_tree)
    layer = kc.PagedKVCache(pt, n_heads=hkv, head_dim=D, dtype=torch.bfloat16, pool=pool)
    mk = torch.zeros(n_pages, hkv, P, D)
    mv = torch.zeros_like(mk)

    def prefill(row, start, n):
        k = torch.randn(1, n, hkv, D, generator=g).to(torch.bfloat16)
        v = torch.randn(1, n, hkv, D, generator=g).to(torch.bfloat16)
        pos = torch.arange(start, start + n).view(1, n)
        pt.commit_block_table([row])
        slots = pt.build_slot_mapping(torch.tensor([row], device=DEV), pos.to(DEV))
        layer.update(input_pos=pos.to(DEV), k_val=k.to(DEV), v_val=v.to(DEV), slot_mapping=slots)
        O.append(mk, mv, k[0], v[0], slots.cpu().view(-1))

    prompt = [Tok(i) for i in range(40)]
    a = pt.allocate()
    pt.reserve(a, 40)
    prefill(a, 0, 40)
    ins = cache_tree.insert(prompt, pt.get_pages(a, 0, 40))
    assert ins.inserted_pages == 40
    # second request: same first 30 tokens, then its own
    b = pt.allocate()
    m = cache_tree.match_prefix(prompt[:30] + [Tok(1000 + i) for i in range(10)])
    assert m.matched_kv_length == 30
    pt.map_pages(b, 0, list(m.matched_pages))
    cache_tree.lock(m.last_node)
    pt.reserve(b, 41)
    prefill(b, 30, 10)
    assert pt.get_pages(b, 0, 30) == pt.get_pages(a, 0, 30)
    q = torch.randn(1, 1, hq, D, generator=g).to(torch.bfloat16).to(DEV)
    meta_pt = torch.zeros(1, n_pages, dtype=torch.int32, device=DEV)
    meta_sk = torch.zeros(1, dtype=torch.int32, device=DEV)
    pt.populate_paged_kv_metadata(batch_idx=torch.tensor([b], device=DEV),
                                  input_pos=torch.tensor([39], dtype=torch.int32, device=DEV),
                                  out_page_table=meta_pt, out_seqused_k=meta_sk)
    out = attn.paged_attention(q.transpose(1, 2), paged_kv_layer=layer, page_table=meta_pt,
                               paged_kv_seqlens_k=meta_sk, scaling=1.0 / math.sqrt(D))
    _check(out, O.paged_attention(q.cpu().float(), mk, mv, meta_pt.cpu(), meta_sk.cpu()))
    cache_tree.unlock(m.last_node)
    pt.erase(b, 30)
    _status_clean()


def test_reference_rejects_what_it_rejected_before(ref):
    """Error behaviour of the reference's own checks stays in front of the kernels."""
    kc, attn, _ = ref
    pool = kc.KVMemoryPool(device=DEV)
    pt = kc.PageTable(n_pages=8, page_size=4, max_batch_size=2, device=DEV)
    with pytest.raises(ValueError, match="FP8 KV cache requires"):
        kc.PagedKVCache(pt, n_heads=2, head_dim=64, dtype=torch.float8_e4m3fn, pool=pool)
    cache = kc.PagedKVCache(pt, n_heads=2, head_dim=64, dtype=torch.bfloat16, pool=pool)
    q32 = torch.zeros(1, 4, 1, 64, device=DEV)
    with pytest.raises(RuntimeError, match="fp16/bf16"):
        attn.paged_attention(q32, paged_kv_layer=cache, page_table=pt.page_table[:1],
                             paged_kv_seqlens_k=torch.ones(1, dtype=torch.int32, device=DEV), scaling=0.125)
