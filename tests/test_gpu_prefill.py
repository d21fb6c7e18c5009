"""GPU parity of the paged prefill attention (many query rows per sequence, the tensor-memory
kernel) against the fp32 CPU oracle, through the same ``flash_attn_fwd`` surface and with the same
tolerance as the decode tests: ``|got - want| <= 2e-2 + 1e-2 * |want|`` per element and a relative
L2 error per output row of at most 1e-2."""

import pytest
import torch

from helpers import make_paged_problem
from kestrel_b200 import _native, kernels
from oracle import paged_kv_oracle as O
from test_gpu_attention import assert_close, run_case

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _clean_status():
    _native.device_status(torch.cuda.current_device(), clear=True)
    yield
    flags = _native.device_status(torch.cuda.current_device(), clear=True)
    assert flags[0] == 0, f"kernel diagnostics: {flags}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("head_dim", [128, 64])
def test_prefill_chunk_on_a_cached_prefix(dtype, head_dim):
    # a 128-token prompt chunk per sequence on top of contexts of assorted lengths (bottom-right causal)
    lengths = [128, 129, 200, 729 + 128, 1000, 143, 257, 2048]
    p = make_paged_problem(seed=11, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=32, n_kv_heads=8,
                           head_dim=head_dim, page_size=16, seqlen_q=128, dtype=dtype, lengths=lengths)
    out, want = run_case(p, dtype)
    assert_close(out, want, f"prefill chunk {dtype} D={head_dim}")


@pytest.mark.parametrize("seqlen_q,group,heads_kv,head_dim", [(16, 4, 8, 128), (37, 4, 2, 128), (64, 1, 4, 64),
                                                               (100, 8, 1, 128), (33, 2, 3, 64), (130, 1, 2, 128),
                                                               (21, 6, 2, 128)])
def test_prefill_shapes_and_gqa(seqlen_q, group, heads_kv, head_dim):
    _shapes_case(seqlen_q, group, heads_kv, head_dim)


# packed rows on either side of the switch between the split-KV kernels and the prefill kernel
# (33 rows, 65 on FP8 pools; 17, 33 on FP8 pools, with head_dim 128 once there is a CTA per SM)
@pytest.mark.parametrize("seqlen_q,group,heads_kv,head_dim", [(8, 4, 2, 128), (9, 4, 2, 128), (10, 4, 2, 128), (12, 4, 2, 128),
                                                               (32, 1, 3, 128), (33, 1, 3, 128), (39, 1, 3, 128), (40, 1, 3, 128),
                                                               (13, 4, 2, 64), (14, 4, 2, 64),
                                                               (55, 1, 4, 64), (56, 1, 4, 64), (63, 1, 4, 64)])
def test_rows_around_the_kernel_switch(seqlen_q, group, heads_kv, head_dim):
    _shapes_case(seqlen_q, group, heads_kv, head_dim)


@pytest.mark.parametrize("seqlen_q,group,heads_kv,head_dim", [(16, 4, 2, 128), (64, 1, 2, 128), (65, 1, 2, 128), (17, 4, 2, 64),
                                                               (33, 2, 1, 128)])
def test_rows_around_the_kernel_switch_fp8_pools(seqlen_q, group, heads_kv, head_dim):
    lengths = [seqlen_q, seqlen_q + 1, seqlen_q + 15, seqlen_q + 113, 3 * seqlen_q + 500, max(1, seqlen_q - 5), 7]
    p = make_paged_problem(seed=70 + seqlen_q, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=group * heads_kv,
                           n_kv_heads=heads_kv, head_dim=head_dim, page_size=16, seqlen_q=seqlen_q,
                           dtype=torch.bfloat16, lengths=lengths)
    out, want = run_case(p, torch.bfloat16, kv="fp8", scales=(0.02, 0.03))
    assert_close(out, want, f"fp8 Sq={seqlen_q} G={group} Hkv={heads_kv} D={head_dim}")


def _shapes_case(seqlen_q, group, heads_kv, head_dim):
    lengths = [seqlen_q, seqlen_q + 1, seqlen_q + 15, seqlen_q + 113, 3 * seqlen_q + 500, max(1, seqlen_q - 5), 7]
    p = make_paged_problem(seed=12 + seqlen_q, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=group * heads_kv,
                           n_kv_heads=heads_kv, head_dim=head_dim, page_size=16, seqlen_q=seqlen_q,
                           dtype=torch.bfloat16, lengths=lengths)
    out, want = run_case(p, torch.bfloat16)
    assert_close(out, want, f"Sq={seqlen_q} G={group} Hkv={heads_kv} D={head_dim}")


@pytest.mark.parametrize("page_size", [1, 2, 8, 16, 64, 256])
@pytest.mark.parametrize("head_dim,seqlen_q", [(128, 32), (64, 32), (128, 96), (64, 130)])
def test_prefill_page_sizes(page_size, head_dim, seqlen_q):
    """TMA boxes of one token (page size 1) up to a whole 128-key tile (page size 256); 32 query tokens at GQA 4 fill
    one Q tile (key split), 96 and 130 two and more."""
    lengths = [300, 64, 65, 1, 513, 1300]
    p = make_paged_problem(seed=13, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=8, n_kv_heads=2, head_dim=head_dim,
                           page_size=page_size, seqlen_q=seqlen_q, dtype=torch.bfloat16, lengths=lengths)
    out, want = run_case(p, torch.bfloat16)
    assert_close(out, want, f"page_size={page_size} D={head_dim} Sq={seqlen_q}")


@pytest.mark.parametrize("causal,window", [(False, None), (True, 63), (True, 200), (True, 0)])
def test_prefill_non_causal_and_sliding_window(causal, window):
    lengths = [64, 100, 400, 1500]
    p = make_paged_problem(seed=14, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=16, n_kv_heads=4, head_dim=128,
                           page_size=16, seqlen_q=48, dtype=torch.bfloat16, lengths=lengths)
    out, want = run_case(p, torch.bfloat16, causal=causal, window=window)
    assert_close(out, want, f"causal={causal} window={window}")


def test_prefill_seqused_q_lse_and_empty_sequences():
    lengths = [500, 0, 77, 1024, 300]
    p = make_paged_problem(seed=15, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=32, n_kv_heads=8, head_dim=64,
                           page_size=16, seqlen_q=40, dtype=torch.bfloat16, lengths=lengths)
    sq = torch.tensor([40, 40, 13, 0, 33], dtype=torch.int32)
    out, want, lse, want_lse = run_case(p, torch.bfloat16, seqused_q=sq, return_lse=True)
    for b, n in enumerate(sq.tolist()):  # rows past seqused_q are not written: compare the valid ones
        if n == 0:
            continue
        assert_close(out[b, :n], want[b, :n], f"seqused_q row {b}")
        got, ref = lse[b, :, :n].cpu(), want_lse[b, :, :n]
        fin = torch.isfinite(ref)
        assert torch.equal(torch.isfinite(got), fin)
        assert (got[fin] - ref[fin]).abs().max().item() <= 2e-2 if fin.any() else True


def test_prefill_packed_rows_with_cu_seqlens():
    lengths = [200, 64, 1000, 129]
    qlens = [64, 17, 128, 129]
    Sq = max(qlens)
    p = make_paged_problem(seed=16, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=8, n_kv_heads=2, head_dim=128,
                           page_size=16, seqlen_q=Sq, dtype=torch.bfloat16, lengths=lengths)
    want = O.paged_attention(p["q"].to(torch.bfloat16).float(), p["k_pool"], p["v_pool"], p["page_table"],
                             p["seqused_k"], seqused_q=torch.tensor(qlens))
    q_packed = torch.cat([p["q"][b, :n] for b, n in enumerate(qlens)]).to(torch.bfloat16).to(DEV)
    cu = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device=DEV)
    out, _ = kernels.flash_attn_fwd(
        q_packed, p["k_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3),
        p["v_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3), page_table=p["page_table"].to(DEV),
        seqused_k=p["seqused_k"].to(DEV), cu_seqlens_q=cu, max_seqlen_q=Sq, causal=True)
    start = 0
    for b, n in enumerate(qlens):
        assert_close(out[start:start + n], want[b, :n], f"packed sequence {b}")
        start += n


def test_prefill_ignores_garbage_past_the_sequence_end():
    # rows of the last page beyond seqused_k hold NaN patterns; they must not reach the output
    lengths = [77, 130, 5]
    p = make_paged_problem(seed=17, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=8, n_kv_heads=2, head_dim=128,
                           page_size=16, seqlen_q=64, dtype=torch.bfloat16, lengths=lengths)
    k = p["k_pool"].to(torch.bfloat16).to(DEV)
    v = p["v_pool"].to(torch.bfloat16).to(DEV)
    for b, L in enumerate(lengths):
        page = int(p["page_table"][b, (L - 1) // 16])
        off = L % 16
        if off:
            k[page, :, off:, :] = float("nan")
            v[page, :, off:, :] = float("nan")
    q = p["q"].to(torch.bfloat16).to(DEV)
    out, _ = kernels.flash_attn_fwd(q, k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3), page_table=p["page_table"].to(DEV),
                                    seqused_k=p["seqused_k"].to(DEV), causal=True)
    want = O.paged_attention(p["q"].to(torch.bfloat16).float(), p["k_pool"], p["v_pool"], p["page_table"], p["seqused_k"])
    assert_close(out, want, "garbage past the end")


# ---- key split: a CTA whose second Q tile has no rows (at most 128 packed rows per KV head) runs its two
# pipelines on the even and the odd key tiles of the same rows and combines them at the end

@pytest.mark.parametrize("seqlen_q,group,heads_kv,head_dim", [(40, 1, 2, 128), (128, 1, 2, 128), (16, 4, 2, 128), (10, 8, 1, 128),
                                                               (56, 1, 3, 64), (32, 4, 1, 64), (100, 1, 2, 64), (129, 1, 2, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_key_split_of_a_single_q_tile(seqlen_q, group, heads_kv, head_dim, dtype):
    # 2 to 40 key tiles, odd and even counts, a sequence that is all chunk, one just past a tile boundary
    lengths = [seqlen_q, seqlen_q + 129, 256, 257, 385, 1000, 2049, 5000, max(seqlen_q, 130)]
    p = make_paged_problem(seed=61 + seqlen_q, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=group * heads_kv,
                           n_kv_heads=heads_kv, head_dim=head_dim, page_size=16, seqlen_q=seqlen_q, dtype=dtype,
                           lengths=lengths)
    out, want, lse, want_lse = run_case(p, dtype, return_lse=True)
    assert_close(out, want, f"key split Sq={seqlen_q} G={group} D={head_dim} {dtype}")
    assert torch.allclose(lse.cpu(), want_lse, atol=2e-3, rtol=1e-3)


@pytest.mark.parametrize("seqlen_q,group,heads_kv,head_dim", [(65, 1, 2, 128), (128, 1, 2, 128), (17, 4, 2, 128), (10, 8, 1, 128),
                                                               (70, 1, 3, 64), (32, 4, 1, 64)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_key_split_on_fp8_pools(seqlen_q, group, heads_kv, head_dim, dtype):
    # e4m3 tiles are widened into a ring of four f16 tiles (three and the unused second Q tile)
    lengths = [seqlen_q, seqlen_q + 129, 256, 257, 385, 1000, 2049, 5000, max(seqlen_q, 130)]
    p = make_paged_problem(seed=64 + seqlen_q, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=group * heads_kv,
                           n_kv_heads=heads_kv, head_dim=head_dim, page_size=16, seqlen_q=seqlen_q, dtype=dtype,
                           lengths=lengths)
    out, want, lse, want_lse = run_case(p, dtype, kv="fp8", scales=(0.02, 0.03), return_lse=True)
    assert_close(out, want, f"fp8 key split Sq={seqlen_q} G={group} D={head_dim} {dtype}")
    assert torch.allclose(lse.cpu(), want_lse, atol=3e-3, rtol=1e-3)


def test_key_split_on_fp8_pools_from_33_rows_with_a_cta_per_sm():
    # 40 sequences x 4 KV heads reach the SM count: 40 and 64 packed rows of an e4m3 pool go to the key split
    rng = torch.Generator().manual_seed(65)
    for seqlen_q in (10, 16):
        lengths = torch.randint(seqlen_q, 900, (40,), generator=rng).tolist()
        p = make_paged_problem(seed=66 + seqlen_q, batch=40, len_lo=0, len_hi=0, n_q_heads=16, n_kv_heads=4, head_dim=128,
                               page_size=16, seqlen_q=seqlen_q, dtype=torch.bfloat16, lengths=lengths)
        out, want = run_case(p, torch.bfloat16, kv="fp8", scales=(0.02, 0.03))
        assert_close(out, want, f"fp8 key split, {4 * seqlen_q} rows, 160 CTAs")


@pytest.mark.parametrize("causal,window", [(False, None), (True, 63), (True, 200), (True, 1000), (True, 0)])
@pytest.mark.parametrize("head_dim", [128, 64])
def test_key_split_non_causal_and_sliding_window(causal, window, head_dim):
    lengths = [130, 400, 1500, 3000]
    p = make_paged_problem(seed=62, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=16, n_kv_heads=4, head_dim=head_dim,
                           page_size=16, seqlen_q=24, dtype=torch.bfloat16, lengths=lengths)
    out, want = run_case(p, torch.bfloat16, causal=causal, window=window)
    assert_close(out, want, f"key split causal={causal} window={window} D={head_dim}")


def test_key_split_seqused_q_and_garbage_past_the_sequence_end():
    lengths = [500, 333, 1031, 300]
    p = make_paged_problem(seed=63, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=8, n_kv_heads=8, head_dim=64,
                           page_size=16, seqlen_q=64, dtype=torch.bfloat16, lengths=lengths)
    k = p["k_pool"].to(torch.bfloat16).to(DEV)
    v = p["v_pool"].to(torch.bfloat16).to(DEV)
    for b, L in enumerate(lengths):   # NaN patterns behind the last key of every sequence
        page, off = int(p["page_table"][b, (L - 1) // 16]), L % 16
        if off:
            k[page, :, off:, :] = float("nan")
            v[page, :, off:, :] = float("nan")
    sq = torch.tensor([64, 57, 1, 60], dtype=torch.int32)
    out, _ = kernels.flash_attn_fwd(p["q"].to(torch.bfloat16).to(DEV), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3),
                                    page_table=p["page_table"].to(DEV), seqused_k=p["seqused_k"].to(DEV),
                                    seqused_q=sq.to(DEV), causal=True)
    want = O.paged_attention(p["q"].to(torch.bfloat16).float(), p["k_pool"], p["v_pool"], p["page_table"],
                             p["seqused_k"], seqused_q=sq)
    for b, n in enumerate(sq.tolist()):
        assert_close(out[b, :n], want[b, :n], f"key split, seqused_q row {b}")


def test_key_split_block_mask_on_a_short_chunk():
    # 100 query rows (one Q tile) on a cached prefix, an image block inside the chunk
    Sq, L = 100, 100 + 700
    ids = _image_prompt_ids(1, Sq, [[(10, 60, 0)]])
    p = make_paged_problem(seed=64, batch=1, len_lo=0, len_hi=0, n_q_heads=4, n_kv_heads=4, head_dim=128, page_size=16,
                           seqlen_q=Sq, dtype=torch.bfloat16, lengths=[L])
    rt = kernels.get_runtime()
    out, _ = rt.attention.flash_attn_fwd(
        p["q"].to(torch.bfloat16).to(DEV), p["k_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3),
        p["v_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3), page_table=p["page_table"].to(DEV),
        seqused_k=p["seqused_k"].to(DEV), paged_kv_non_tma=True, causal=False, pack_gqa=False,
        mask_mod=rt.attention.block_bidirectional_mask, aux_tensors=[ids.to(DEV)])
    want = O.paged_attention(p["q"].to(torch.bfloat16).float(), p["k_pool"], p["v_pool"], p["page_table"], p["seqused_k"],
                             block_ids=ids)
    assert_close(out, want, "key split with a block mask")


def _image_prompt_ids(B, Sq, layouts):
    """block ids per position: ``layouts[b]`` is a list of (start, length, id) image blocks."""
    ids = torch.full((B, Sq), -1, dtype=torch.int32)
    for b, blocks in enumerate(layouts):
        for start, n, bid in blocks:
            ids[b, start:start + n] = bid
    return ids


def test_block_visibility_rows():
    ids = torch.tensor([[0, 0, 0, -1, -1, 1, 1, -1], [-1, 3, 3, 3, 3, 3, 3, 3]], dtype=torch.int32, device=DEV)
    got = kernels.block_visibility(ids).cpu().tolist()
    assert got == [[2, 2, 2, 3, 4, 6, 6, 7], [0, 7, 7, 7, 7, 7, 7, 7]]
    assert kernels.block_visibility(ids, 4).cpu().tolist() == [[2, 2, 2, 3], [0, 3, 3, 3]]


@pytest.mark.parametrize("head_dim,group,heads_kv", [(64, 1, 8), (128, 4, 2)])
def test_prefill_block_bidirectional_mask(head_dim, group, heads_kv):
    # whole prompts (no cached prefix): BOS + a 729-position image + text; two images between text; text only;
    # a short padded row
    Sq = 900
    lengths = [900, 900, 300, 40]
    layouts = [[(0, 730, 0)], [(5, 200, 0), (400, 333, 1)], [], [(1, 30, 2)]]
    ids = _image_prompt_ids(len(lengths), Sq, layouts)
    p = make_paged_problem(seed=21, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=group * heads_kv,
                           n_kv_heads=heads_kv, head_dim=head_dim, page_size=16, seqlen_q=Sq, dtype=torch.bfloat16,
                           lengths=lengths)
    sq = torch.tensor(lengths, dtype=torch.int32)
    q = p["q"].to(torch.bfloat16).to(DEV)
    rt = kernels.get_runtime()
    out, _ = rt.attention.flash_attn_fwd(
        q, p["k_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3), p["v_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3),
        page_table=p["page_table"].to(DEV), seqused_q=sq.to(DEV), seqused_k=p["seqused_k"].to(DEV), paged_kv_non_tma=True,
        causal=False, pack_gqa=False, mask_mod=rt.attention.block_bidirectional_mask, aux_tensors=[ids.to(DEV)])
    want = O.paged_attention(p["q"].to(torch.bfloat16).float(), p["k_pool"], p["v_pool"], p["page_table"], p["seqused_k"],
                             seqused_q=sq, block_ids=ids)
    causal_only = O.paged_attention(p["q"].to(torch.bfloat16).float(), p["k_pool"], p["v_pool"], p["page_table"],
                                    p["seqused_k"], seqused_q=sq)
    assert (want[0, :700] - causal_only[0, :700]).abs().max() > 0.05   # the mask matters
    assert torch.equal(want[2, :300], causal_only[2, :300])            # and leaves text-only prompts alone
    for b, n in enumerate(lengths):
        assert_close(out[b, :n], want[b, :n], f"block mask, sequence {b}")


def test_prefill_block_mask_on_a_chunk_after_a_cached_prefix():
    # the ids index the query rows of this call; keys before the chunk are plain causal context
    Sq, L = 256, 256 + 333
    ids = _image_prompt_ids(1, Sq, [[(10, 200, 0)]])
    p = make_paged_problem(seed=22, batch=1, len_lo=0, len_hi=0, n_q_heads=8, n_kv_heads=2, head_dim=128, page_size=16,
                           seqlen_q=Sq, dtype=torch.bfloat16, lengths=[L])
    out, _ = kernels.flash_attn_fwd(
        p["q"].to(torch.bfloat16).to(DEV), p["k_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3),
        p["v_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3), page_table=p["page_table"].to(DEV),
        seqused_k=p["seqused_k"].to(DEV), mask_mod=kernels.block_bidirectional_mask, aux_tensors=[ids.to(DEV)])
    want = O.paged_attention(p["q"].to(torch.bfloat16).float(), p["k_pool"], p["v_pool"], p["page_table"], p["seqused_k"],
                             block_ids=ids)
    assert_close(out, want, "block mask on a chunk")


def test_block_mask_argument_errors():
    q = torch.zeros(1, 4, 2, 64, device=DEV, dtype=torch.bfloat16)
    pool = torch.zeros(4, 16, 2, 64, device=DEV, dtype=torch.bfloat16)
    kw = dict(page_table=torch.zeros(1, 2, dtype=torch.int32, device=DEV), seqused_k=torch.tensor([4], dtype=torch.int32, device=DEV))
    with pytest.raises(NotImplementedError, match="only mask_mod"):
        kernels.flash_attn_fwd(q, pool, pool, mask_mod=lambda *a: True, aux_tensors=[], **kw)
    with pytest.raises(ValueError, match="aux_tensors"):
        kernels.flash_attn_fwd(q, pool, pool, mask_mod=kernels.block_bidirectional_mask, **kw)
    with pytest.raises(NotImplementedError, match="packed rows"):
        kernels.flash_attn_fwd(q[0], pool, pool, mask_mod=kernels.block_bidirectional_mask,
                               aux_tensors=[torch.zeros(1, 4, dtype=torch.int32, device=DEV)],
                               cu_seqlens_q=torch.tensor([0, 4], dtype=torch.int32, device=DEV), **kw)


def test_prefill_calls_need_only_the_plan_arrays_as_scratch():
    import ctypes as C
    lib = _native.load()
    a = _native.AttnArgs()
    a.struct_bytes = C.sizeof(_native.AttnArgs)
    a.device = torch.cuda.current_device()
    a.batch, a.total_q, a.seqlen_q = 64, 64 * 1024, 1024
    a.n_q_heads, a.n_kv_heads, a.head_dim, a.page_size = 32, 8, 128, 16
    a.q_dtype = a.kv_dtype = _native.DTYPE_BF16
    bound = int(lib.kb200_attn_workspace_bytes(a.batch, a.total_q, 32, 8, 128, a.device))
    need = int(lib.kb200_attn_workspace_bytes_for(C.byref(a)))
    assert 0 < need < 64 * 1024 < bound            # a few plan arrays against gigabytes of split-KV partials
    a.kv_dtype = _native.DTYPE_E4M3                 # FP8 pools: the same kernel, tiles widened on the fly
    assert int(lib.kb200_attn_workspace_bytes_for(C.byref(a))) == need
    a.kv_dtype, a.seqlen_q, a.total_q = _native.DTYPE_BF16, 1, 64  # decode
    # (the bound also covers e4m3 pools with one-token pages, whose partials are wider)
    assert 64 * 1024 < int(lib.kb200_attn_workspace_bytes_for(C.byref(a))) <= int(lib.kb200_attn_workspace_bytes(64, 64, 32, 8, 128, a.device))


@pytest.mark.parametrize("head_dim", [128, 64])
@pytest.mark.parametrize("qdtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("per_head", [True, False])
def test_prefill_fp8_kv(head_dim, qdtype, per_head):
    lengths = [128, 129, 200, 729 + 128, 1000, 143, 2048]
    p = make_paged_problem(seed=31, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=32, n_kv_heads=8,
                           head_dim=head_dim, page_size=16, seqlen_q=128, dtype=qdtype, lengths=lengths, outlier_frac=0.01)
    if per_head:
        ks = p["k_pool"].abs().amax(dim=(0, 2, 3)) / 448
        vs = p["v_pool"].abs().amax(dim=(0, 2, 3)) / 448
    else:
        ks = float(p["k_pool"].abs().max() / 448)
        vs = float(p["v_pool"].abs().max() / 448)
    out, want = run_case(p, qdtype, kv="fp8", scales=(ks, vs))
    assert_close(out, want, f"fp8 prefill D={head_dim} {qdtype} per_head={per_head}")


@pytest.mark.parametrize("page_size,seqlen_q,group,heads_kv", [(16, 37, 4, 2), (64, 64, 1, 4), (256, 100, 8, 1), (4, 33, 2, 3),
                                                               (1, 40, 4, 2)])
def test_prefill_fp8_kv_shapes_and_pages(page_size, seqlen_q, group, heads_kv):
    lengths = [seqlen_q, seqlen_q + 17, 3 * seqlen_q + 500, max(1, seqlen_q - 5), 7, 0]
    p = make_paged_problem(seed=32 + seqlen_q, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=group * heads_kv,
                           n_kv_heads=heads_kv, head_dim=128, page_size=page_size, seqlen_q=seqlen_q,
                           dtype=torch.bfloat16, lengths=lengths)
    out, want = run_case(p, torch.bfloat16, kv="fp8", scales=(0.02, 0.03))
    assert_close(out, want, f"fp8 P={page_size} Sq={seqlen_q} G={group}")


def test_prefill_fp8_kv_windows_and_block_mask():
    lengths = [400, 1500]
    p = make_paged_problem(seed=33, batch=2, len_lo=0, len_hi=0, n_q_heads=16, n_kv_heads=4, head_dim=128, page_size=16,
                           seqlen_q=48, dtype=torch.bfloat16, lengths=lengths)
    out, want = run_case(p, torch.bfloat16, kv="fp8", scales=(0.02, 0.03), window=100)
    assert_close(out, want, "fp8 window")
    Sq = 300
    ids = _image_prompt_ids(1, Sq, [[(3, 250, 0)]])
    p = make_paged_problem(seed=34, batch=1, len_lo=0, len_hi=0, n_q_heads=8, n_kv_heads=2, head_dim=64, page_size=16,
                           seqlen_q=Sq, dtype=torch.bfloat16, lengths=[Sq])
    kq = O.fp8_quantise(p["k_pool"].permute(0, 2, 1, 3), 0.02).permute(0, 2, 1, 3).contiguous()
    vq = O.fp8_quantise(p["v_pool"].permute(0, 2, 1, 3), 0.03).permute(0, 2, 1, 3).contiguous()
    out, _ = kernels.flash_attn_fwd(
        p["q"].to(torch.bfloat16).to(DEV), kq.to(DEV).view(torch.float8_e4m3fn).permute(0, 2, 1, 3),
        vq.to(DEV).view(torch.float8_e4m3fn).permute(0, 2, 1, 3), page_table=p["page_table"].to(DEV),
        seqused_k=p["seqused_k"].to(DEV), mask_mod=kernels.block_bidirectional_mask, aux_tensors=[ids.to(DEV)],
        k_scale=0.02, v_scale=0.03)
    want = O.paged_attention(p["q"].to(torch.bfloat16).float(), kq, vq, p["page_table"], p["seqused_k"], block_ids=ids,
                             k_scale=0.02, v_scale=0.03)
    assert_close(out, want, "fp8 block mask")


def test_prefill_in_a_cuda_graph_with_changing_lengths():
    # lengths and page indices are read on the device: one captured graph serves calls with other lengths
    Sq = 64
    lengths = [700, 130, 64]
    p = make_paged_problem(seed=41, batch=3, len_lo=0, len_hi=0, n_q_heads=8, n_kv_heads=2, head_dim=128, page_size=16,
                           seqlen_q=Sq, dtype=torch.bfloat16, lengths=lengths)
    q = p["q"].to(torch.bfloat16).to(DEV)
    k = p["k_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3)
    v = p["v_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3)
    table, sk = p["page_table"].to(DEV), p["seqused_k"].to(DEV)
    out = torch.empty_like(q)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        kernels.flash_attn_fwd(q, k, v, page_table=table, seqused_k=sk, causal=True, out=out)   # sizes the scratch
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            kernels.flash_attn_fwd(q, k, v, page_table=table, seqused_k=sk, causal=True, out=out)
    torch.cuda.current_stream().wait_stream(stream)
    for new_lengths in ([700, 130, 64], [300, 100, 50], [64, 65, 33]):   # within the pages each sequence owns
        sk.copy_(torch.tensor(new_lengths, dtype=torch.int32))
        out.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        want = O.paged_attention(p["q"].to(torch.bfloat16).float(), p["k_pool"], p["v_pool"], p["page_table"],
                                 torch.tensor(new_lengths, dtype=torch.int32))
        assert_close(out, want, f"graph replay with lengths {new_lengths}")


def test_prefill_through_the_allocation_free_entry_point():
    import ctypes as C
    import math
    lib = _native.load()
    Sq = 256
    lengths = [1000, 300]
    p = make_paged_problem(seed=42, batch=2, len_lo=0, len_hi=0, n_q_heads=32, n_kv_heads=8, head_dim=64, page_size=16,
                           seqlen_q=Sq, dtype=torch.bfloat16, lengths=lengths)
    q = p["q"].to(torch.bfloat16).to(DEV)
    k = p["k_pool"].to(torch.bfloat16).to(DEV)
    v = p["v_pool"].to(torch.bfloat16).to(DEV)
    table, sk = p["page_table"].to(DEV), p["seqused_k"].to(DEV)
    out = torch.full_like(q, float("nan"))
    kv_view = k.permute(0, 2, 1, 3)
    a = _native.AttnArgs()
    a.struct_bytes = C.sizeof(_native.AttnArgs)
    a.device = q.device.index
    a.stream = torch.cuda.current_stream().cuda_stream
    a.q, a.out = q.data_ptr(), out.data_ptr()
    a.q_batch_stride, a.q_row_stride, a.q_head_stride = q.stride(0), q.stride(1), q.stride(2)
    a.o_batch_stride, a.o_row_stride, a.o_head_stride = out.stride(0), out.stride(1), out.stride(2)
    a.k_cache, a.v_cache = k.data_ptr(), v.data_ptr()
    a.kv_page_stride, a.kv_token_stride, a.kv_head_stride = kv_view.stride(0), kv_view.stride(1), kv_view.stride(2)
    a.n_pages = k.shape[0]
    a.page_table, a.pt_row_stride, a.seqused_k = table.data_ptr(), table.stride(0), sk.data_ptr()
    a.batch, a.total_q, a.seqlen_q = 2, 2 * Sq, Sq
    a.n_q_heads, a.n_kv_heads, a.head_dim, a.page_size = 32, 8, 64, 16
    a.q_dtype = a.kv_dtype = _native.DTYPE_BF16
    a.softmax_scale, a.causal, a.window_left = 1.0 / math.sqrt(64), 1, -1
    a.k_scale = a.v_scale = 1.0
    # the generic bound for these dimensions exceeds what a prefill-shaped call really needs
    assert int(lib.kb200_attn_workspace_bytes_for(C.byref(a))) < 4096
    _native.check(lib.kb200_paged_attention_static(C.byref(a)))
    torch.cuda.synchronize()
    want = O.paged_attention(p["q"].to(torch.bfloat16).float(), p["k_pool"], p["v_pool"], p["page_table"], p["seqused_k"])
    assert_close(out, want, "static entry point, prefill-shaped call")


def test_config4_full_size_prefill_chunk_sampled_and_repaged():
    """Configuration 4's prefill at full size: 512 requests, a shared 729-token prefix (45 full pages
    referenced by every page-table row, the partly filled 46th page private per request) and the first
    chunk of each request's suffix (U[32,256], at most 128 tokens) as one packed call.  Eight requests
    are checked against the oracle; moving every private page to another physical page must not
    change one output bit."""
    g = torch.Generator().manual_seed(4004)
    B, P, hq, hkv, D, prefix = 512, 16, 32, 8, 64, 729
    suffix = torch.randint(32, 257, (B,), generator=g)
    chunk = suffix.clamp(max=128)
    L = prefix + chunk
    shared = prefix // P
    own = (L + P - 1) // P - shared
    n_pages = 1 + shared + int(own.sum())
    table = torch.zeros(B, int((L.max() + P - 1) // P), dtype=torch.int32)
    table[:, :shared] = torch.arange(1, shared + 1, dtype=torch.int32)
    perm = (torch.randperm(n_pages - 1 - shared, generator=g) + 1 + shared).to(torch.int32)
    cur = 0
    for b in range(B):
        n = int(own[b])
        table[b, shared:shared + n] = perm[cur:cur + n]
        cur += n
    k_pool = torch.randn(n_pages, hkv, P, D, generator=g).to(torch.bfloat16)
    v_pool = torch.randn(n_pages, hkv, P, D, generator=g).to(torch.bfloat16)
    total = int(chunk.sum())
    q = torch.randn(total, hq, D, generator=g).to(torch.bfloat16)
    cu = torch.zeros(B + 1, dtype=torch.int32)
    cu[1:] = chunk.cumsum(0)

    def run(kp, vp, tb):
        out, _ = kernels.flash_attn_fwd(q.to(DEV), kp.to(DEV).permute(0, 2, 1, 3), vp.to(DEV).permute(0, 2, 1, 3),
                                        page_table=tb.to(DEV), seqused_k=L.to(torch.int32).to(DEV), cu_seqlens_q=cu.to(DEV),
                                        max_seqlen_q=128, causal=True)
        return out.cpu()

    out = run(k_pool, v_pool, table)
    for b in [0, 1, 7, 100, 255, 256, 400, 511]:
        n = int(chunk[b])
        qb = torch.zeros(1, 128, hq, D)
        qb[0, :n] = q[int(cu[b]):int(cu[b]) + n].float()
        want = O.paged_attention(qb, k_pool.float(), v_pool.float(), table[b:b + 1], L[b:b + 1].to(torch.int32),
                                 seqused_q=torch.tensor([n]))
        assert_close(out[int(cu[b]):int(cu[b]) + n], want[0, :n], f"request {b}")
    # physical re-paging of the private pages
    move = torch.arange(n_pages)
    priv = torch.arange(1 + shared, n_pages)
    move[priv] = priv[torch.randperm(priv.numel(), generator=g)]
    k2, v2 = torch.empty_like(k_pool), torch.empty_like(v_pool)
    k2[move] = k_pool
    v2[move] = v_pool
    table2 = move.to(torch.int32)[table.long()]
    out2 = run(k2, v2, table2)
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))
