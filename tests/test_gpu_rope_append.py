"""GPU parity (bit-exact) of the rotary embedding, the rotary + append fusion and the fused
per-step decode metadata, through the public API / C ABI, against the CPU oracle."""

import numpy as np
import pytest
import torch

from kestrel_b200 import _native, kernels
from kestrel_b200.kv_cache import KVMemoryPool, PagedKVCache, PageTable
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


def _fused_qkv(g, B, S, hq, hkv, D, dtype):
    """q, k, v as the strided slices of one fused projection buffer (how the models pass them)."""
    buf = torch.randn(B, S, (hq + 2 * hkv) * D, generator=g).to(dtype).to(DEV)
    q, k, v = buf.split([hq * D, hkv * D, hkv * D], dim=-1)
    return buf, q.unflatten(-1, (hq, D)), k.unflatten(-1, (hkv, D)), v.unflatten(-1, (hkv, D))


def test_rotary_golden_vectors_from_reference(golden_dir):
    vec = np.load(golden_dir / "rope_vectors.npz")
    x = torch.from_numpy(vec["x"]).to(DEV)
    pos = torch.from_numpy(vec["pos"]).to(DEV)
    table = torch.from_numpy(vec["table"]).to(DEV)
    q = x.clone().unsqueeze(0)
    k = x.clone().unsqueeze(0)
    kernels.get_runtime().rotary.rotary_embedding(pos.view(1, -1), q, k, 64, table)
    want = torch.from_numpy(vec["y"])
    assert torch.equal(q[0].cpu().view(torch.int32), want.view(torch.int32))
    assert torch.equal(k[0].cpu().view(torch.int32), want.view(torch.int32))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("B,S,hq,hkv,D,rot", [(5, 1, 32, 8, 64, 32), (2, 37, 32, 32, 64, 32), (3, 4, 8, 2, 128, 128),
                                               (2, 3, 4, 2, 24, 6), (1, 9, 6, 3, 16, 16)])
def test_rotary_in_place_matches_oracle(dtype, B, S, hq, hkv, D, rot):
    g = torch.Generator().manual_seed(B * 100 + S)
    table = O.precompute_freqs_cis(rot, 512, 1.5e6)
    buf, q, k, v = _fused_qkv(g, B, S, hq, hkv, D, dtype)
    before = buf.clone()
    pos = torch.randint(0, 512, (B, S), generator=g)
    want_q = O.rotary_embedding(pos, q.cpu().reshape(B * S, hq, D), table)
    want_k = O.rotary_embedding(pos, k.cpu().reshape(B * S, hkv, D), table)
    kernels.rotary_embedding(pos.to(DEV), q, k, D, table.to(DEV))
    assert torch.equal(_bits(q.reshape(B * S, hq, D)).cpu(), _bits(want_q))
    assert torch.equal(_bits(k.reshape(B * S, hkv, D)).cpu(), _bits(want_k))
    assert torch.equal(_bits(v).cpu(), _bits(before.split([hq * D, hkv * D, hkv * D], dim=-1)[2].unflatten(-1, (hkv, D))).cpu())


@pytest.mark.parametrize("kv_dtype", [torch.bfloat16, torch.float8_e4m3fn])
@pytest.mark.parametrize("B,S,hq,hkv,D,rot,P", [(6, 1, 32, 8, 128, 128, 16), (2, 50, 32, 32, 64, 32, 16),
                                                 (3, 5, 8, 2, 64, 32, 1), (2, 7, 4, 2, 24, 6, 4)])
@pytest.mark.parametrize("write_k", [True, False])
def test_rope_append_equals_rotary_then_append(kv_dtype, B, S, hq, hkv, D, rot, P, write_k):
    g = torch.Generator().manual_seed(7 + S)
    n_pages = -(-B * S // P) * 2 + 3
    table = O.precompute_freqs_cis(rot, 256, 1.5e6)
    kw = {}
    ks = vs = None
    if kv_dtype == torch.float8_e4m3fn:
        ks = (torch.rand(hkv, generator=g) * 0.02 + 0.005).tolist()
        vs = (torch.rand(hkv, generator=g) * 0.02 + 0.005).tolist()
        kw = dict(k_scale=ks, v_scale=vs)
    pool = KVMemoryPool(device=DEV)
    pt = PageTable(n_pages=n_pages, page_size=P, max_batch_size=2, device=DEV)
    fused_layer = PagedKVCache(pt, n_heads=hkv, head_dim=D, dtype=kv_dtype, pool=pool, **kw)
    plain_layer = PagedKVCache(pt, n_heads=hkv, head_dim=D, dtype=kv_dtype, pool=pool, **kw)
    buf, q, k, v = _fused_qkv(g, B, S, hq, hkv, D, torch.bfloat16)
    buf2 = buf.clone()
    ref_buf = buf.cpu().clone()   # untouched copy for the oracle (q and k are rotated in place)
    q2, k2, v2 = (t.unflatten(-1, (h, D)) for t, h in zip(buf2.split([hq * D, hkv * D, hkv * D], dim=-1), (hq, hkv, hkv)))
    pos = torch.randint(0, 256, (B, S), generator=g).to(DEV)
    slots = (torch.randperm(n_pages * P - P, generator=g)[: B * S] + P).view(B, S)
    slots[0, 0] = -1   # a padding row: rotated, not stored
    slots = slots.to(DEV)

    fused_layer.rope_update(pos, q, k, v, table.to(DEV), slot_mapping=slots, write_k=write_k)
    kernels.rotary_embedding(pos, q2, k2, D, table.to(DEV))
    plain_layer.update(pos, k2, v2, slot_mapping=slots)

    assert torch.equal(_bits(fused_layer.k_cache), _bits(plain_layer.k_cache))
    assert torch.equal(_bits(fused_layer.v_cache), _bits(plain_layer.v_cache))
    assert torch.equal(_bits(q), _bits(q2))
    if write_k:
        assert torch.equal(_bits(k), _bits(k2))
    # and against the oracle: rotate, then append (quantising when the pool is FP8)
    mirror_dt = torch.uint8 if kv_dtype == torch.float8_e4m3fn else torch.float32
    mk = torch.zeros(n_pages, hkv, P, D, dtype=mirror_dt)
    mv = torch.zeros_like(mk)
    rq, rk, rv = ref_buf.split([hq * D, hkv * D, hkv * D], dim=-1)
    rk = O.rotary_embedding(pos.cpu(), rk.reshape(B * S, hkv, D), table)
    O.append(mk, mv, rk, rv.reshape(B * S, hkv, D), slots.cpu(),
             k_scale=None if ks is None else torch.tensor(ks), v_scale=None if vs is None else torch.tensor(vs))
    got_k = fused_layer.k_cache.view(torch.uint8).cpu() if mirror_dt == torch.uint8 else fused_layer.k_cache.float().cpu()
    got_v = fused_layer.v_cache.view(torch.uint8).cpu() if mirror_dt == torch.uint8 else fused_layer.v_cache.float().cpu()
    assert torch.equal(got_k, mk) and torch.equal(got_v, mv)
    want_q = O.rotary_embedding(pos.cpu(), rq.reshape(B * S, hq, D), table)
    assert torch.equal(_bits(q.reshape(B * S, hq, D)).cpu(), _bits(want_q))


def test_rotary_reports_positions_outside_the_table():
    table = O.precompute_freqs_cis(32, 16, 1.5e6).to(DEV)
    q = torch.randn(1, 2, 4, 64, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(1, 2, 2, 64, device=DEV, dtype=torch.bfloat16)
    kernels.rotary_embedding(torch.tensor([[3, 99]], device=DEV), q, k, 64, table)
    flags = _native.device_status(torch.cuda.current_device(), clear=True)
    assert flags[0] == _native.STATUS_BAD_POSITION and flags[1] == 99


def test_rope_argument_errors():
    table = O.precompute_freqs_cis(32, 16, 1.5e6).to(DEV)
    k = torch.randn(1, 2, 2, 64, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        kernels.rotary_embedding(torch.zeros(1, 2, dtype=torch.long), k.cpu(), k.cpu(), 64, table.cpu())
    with pytest.raises(ValueError, match="one entry per token"):
        kernels.rope_reshape_and_cache(torch.zeros(3, dtype=torch.long, device=DEV), None, k, None, table)
    with pytest.raises(ValueError, match="rot_dim"):
        kernels.rope_reshape_and_cache(torch.zeros(2, dtype=torch.long, device=DEV), None,
                                       torch.zeros(1, 2, 2, 16, device=DEV, dtype=torch.bfloat16), None, table)


@pytest.mark.parametrize("P,n_new,bi_dtype", [(16, 1, torch.int64), (16, 4, torch.int32), (1, 1, torch.int64), (4, 3, torch.int64)])
def test_decode_step_metadata_matches_oracle(P, n_new, bi_dtype):
    g = torch.Generator().manual_seed(P * 10 + n_new)
    B, n_pages = 9, 200
    pt = PageTable(n_pages=n_pages, page_size=P, max_batch_size=B + 3, device=DEV)
    lens = torch.randint(n_new, 12 * P + 1, (B,), generator=g).tolist()
    rows = [pt.allocate() for _ in range(B)]
    for r, L in zip(rows, lens):
        pt.reserve(r, L)
    pt.commit_block_table()
    order = torch.randperm(B, generator=g).tolist()
    batch_idx = torch.tensor([rows[i] for i in order], dtype=bi_dtype, device=DEV)
    input_pos = torch.tensor([lens[i] - 1 for i in order], dtype=torch.int32, device=DEV)
    out_pt = torch.full((B, n_pages), -7, dtype=torch.int32, device=DEV)
    out_sk = torch.full((B,), -7, dtype=torch.int32, device=DEV)
    slots, positions = pt.populate_decode_step(batch_idx=batch_idx, input_pos=input_pos, out_page_table=out_pt,
                                               out_seqused_k=out_sk, n_new=n_new)
    ref_pt = torch.full((B, n_pages), -7, dtype=torch.int32)
    ref_sk = torch.full((B,), -7, dtype=torch.int32)
    ref_slots, ref_pos = O.build_decode_step_metadata(pt._page_table_cpu_tensor, batch_idx.cpu(), input_pos.cpu(),
                                                      ref_pt, ref_sk, P, n_new=n_new)
    assert torch.equal(out_pt.cpu(), ref_pt) and torch.equal(out_sk.cpu(), ref_sk)
    assert slots.dtype == torch.int64 and torch.equal(slots.cpu(), ref_slots)
    assert torch.equal(positions.cpu(), ref_pos)
    # the same as the two separate calls of the reference surface
    out_pt2 = torch.full_like(out_pt, -7)
    out_sk2 = torch.full_like(out_sk, -7)
    pt.populate_paged_kv_metadata(batch_idx=batch_idx, input_pos=input_pos, out_page_table=out_pt2, out_seqused_k=out_sk2)
    assert torch.equal(out_pt, out_pt2) and torch.equal(out_sk, out_sk2)
    assert torch.equal(slots, pt.build_slot_mapping(batch_idx, positions))
