"""GPU parity of the paged split-KV decode attention against the fp32 CPU oracle.

Tolerance (stated by the build target for bf16 attention outputs: 2e-2 absolute / 1e-2 relative),
applied the way ``torch.testing.assert_close(atol=2e-2, rtol=1e-2)`` does -- every element must
satisfy ``|got - want| <= 2e-2 + 1e-2 * |want|`` -- and, on top of that, the relative L2 error of
every output row (one query head, ``head_dim`` values) must stay below 1e-2.  An element-wise
relative bound alone is not meaningful here: outputs are sums with cancellation and are rounded
to bf16/fp16 (half an ulp is 0.2 % of the value, and 0.06 absolute once a value passes 16).

Wherever the expected outputs stay below 8 in magnitude -- every N(0,1) case: half a bf16 ulp is then at
most 0.016 -- the plain reading of the target, ``max |got - want| <= 2e-2`` with no relative term, is
asserted as well.
"""

import math

import pytest
import torch

from helpers import make_paged_problem
from kestrel_b200 import _native, kernels
from kestrel_b200.attention import paged_attention
from oracle import paged_kv_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
ABS_TOL, REL_TOL = 2e-2, 1e-2


@pytest.fixture(autouse=True)
def _clean_status():
    _native.device_status(torch.cuda.current_device(), clear=True)
    yield
    flags = _native.device_status(torch.cuda.current_device(), clear=True)
    assert flags[0] == 0, f"kernel diagnostics: {flags}"


def assert_close(got, want, what=""):
    got = got.float().cpu()
    assert torch.isfinite(got).all(), what
    diff = (got - want).abs()
    excess = (diff - (ABS_TOL + REL_TOL * want.abs())).max().item()
    assert excess <= 0, (what, "element", diff.max().item(), excess)
    if want.abs().max().item() < 8.0:
        assert diff.max().item() <= ABS_TOL, (what, "plain max-abs", diff.max().item())
    num = diff.pow(2).sum(dim=-1).sqrt()
    den = want.pow(2).sum(dim=-1).sqrt()
    live = den > 1e-3
    if live.any():
        rel = (num[live] / den[live]).max().item()
        assert rel <= REL_TOL, (what, "row L2", rel)
    if (~live).any():
        assert num[~live].max().item() <= 1e-3, (what, "rows that should be ~0")


def run_case(p, dtype, *, kv="same", causal=True, window=None, seqused_q=None, scales=None, softmax_scale=None,
             return_lse=False):
    q = p["q"].to(dtype).to(DEV)
    if kv == "fp8":
        ks, vs = scales
        kq = O.fp8_quantise(p["k_pool"].permute(0, 2, 1, 3), ks).permute(0, 2, 1, 3).contiguous()
        vq = O.fp8_quantise(p["v_pool"].permute(0, 2, 1, 3), vs).permute(0, 2, 1, 3).contiguous()
        k_dev = kq.to(DEV).view(torch.float8_e4m3fn)
        v_dev = vq.to(DEV).view(torch.float8_e4m3fn)
        k_ref, v_ref = kq, vq
        ks_arg = ks.to(DEV) if isinstance(ks, torch.Tensor) else ks
        vs_arg = vs.to(DEV) if isinstance(vs, torch.Tensor) else vs
    else:
        k_dev, v_dev = p["k_pool"].to(dtype).to(DEV), p["v_pool"].to(dtype).to(DEV)
        k_ref, v_ref = p["k_pool"], p["v_pool"]
        ks = vs = ks_arg = vs_arg = None
    out, lse = kernels.flash_attn_fwd(
        q, k_dev.permute(0, 2, 1, 3), v_dev.permute(0, 2, 1, 3), page_table=p["page_table"].to(DEV),
        seqused_k=p["seqused_k"].to(DEV), seqused_q=None if seqused_q is None else seqused_q.to(DEV),
        causal=causal, window_size_left=window, window_size_right=0 if window is not None else None,
        softmax_scale=softmax_scale, k_scale=ks_arg, v_scale=vs_arg, paged_kv_non_tma=True, return_lse=return_lse)
    want = O.paged_attention(p["q"].to(dtype).float(), k_ref, v_ref, p["page_table"], p["seqused_k"],
                             softmax_scale=softmax_scale, causal=causal, window_left=window, k_scale=ks, v_scale=vs,
                             seqused_q=seqused_q, return_lse=return_lse)
    assert out.shape == q.shape and out.dtype == dtype
    if return_lse:
        want, want_lse = want
        return out, want, lse, want_lse
    return out, want


EDGE_LENGTHS = [1, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 500, 1000]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("head_dim", [128, 64])
def test_decode_edge_lengths(dtype, head_dim):
    p = make_paged_problem(seed=1, batch=len(EDGE_LENGTHS), len_lo=0, len_hi=0, n_q_heads=32, n_kv_heads=8,
                           head_dim=head_dim, page_size=16, dtype=dtype, lengths=EDGE_LENGTHS)
    out, want = run_case(p, dtype)
    assert_close(out, want, f"{dtype} D={head_dim}")


@pytest.mark.parametrize("head_dim", [128, 64])
@pytest.mark.parametrize("per_head", [True, False])
@pytest.mark.parametrize("qdtype", [torch.bfloat16, torch.float16])
def test_decode_fp8_kv(head_dim, per_head, qdtype):
    p = make_paged_problem(seed=2, batch=len(EDGE_LENGTHS), len_lo=0, len_hi=0, n_q_heads=32, n_kv_heads=8,
                           head_dim=head_dim, page_size=16, dtype=qdtype, lengths=EDGE_LENGTHS, outlier_frac=0.01)
    if per_head:
        ks = p["k_pool"].abs().amax(dim=(0, 2, 3)) / 448
        vs = p["v_pool"].abs().amax(dim=(0, 2, 3)) / 448
    else:
        ks = float(p["k_pool"].abs().max() / 448)
        vs = float(p["v_pool"].abs().max() / 448)
    out, want = run_case(p, qdtype, kv="fp8", scales=(ks, vs))
    assert_close(out, want, f"fp8 D={head_dim} per_head={per_head}")


@pytest.mark.parametrize("seqlen_q,group,heads_kv", [(4, 4, 8), (2, 4, 2), (4, 8, 2), (1, 1, 8), (3, 16, 1), (1, 6, 2), (16, 1, 2),
                                                      (2, 2, 4), (4, 1, 8), (3, 1, 2), (1, 3, 4)])
@pytest.mark.parametrize("kv", ["same", "fp8"])
def test_multi_query_causal_and_gqa_shapes(seqlen_q, group, heads_kv, kv):
    lengths = [1, 3, 4, 5, 16, 17, 40, 64, 65, 333]
    p = make_paged_problem(seed=3 + seqlen_q, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=group * heads_kv,
                           n_kv_heads=heads_kv, head_dim=128, page_size=16, seqlen_q=seqlen_q, dtype=torch.bfloat16,
                           lengths=lengths)
    scales = (0.02, 0.03) if kv == "fp8" else None
    out, want = run_case(p, torch.bfloat16, kv=kv, scales=scales)
    assert_close(out, want, f"Sq={seqlen_q} G={group} kv={kv}")


def test_seqused_q_and_non_causal_and_lse():
    lengths = [7, 64, 65, 200, 0, 31]
    p = make_paged_problem(seed=9, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=8, n_kv_heads=2, head_dim=64,
                           page_size=16, seqlen_q=4, dtype=torch.bfloat16, lengths=lengths)
    sq = torch.tensor([4, 1, 3, 0, 2, 4], dtype=torch.int32)
    out, want, lse, want_lse = run_case(p, torch.bfloat16, seqused_q=sq, return_lse=True)
    for b, n in enumerate(sq.tolist()):  # rows past seqused_q are not written: compare the valid ones
        if n == 0:
            continue
        if lengths[b] == 0:
            assert (out[b, :n] == 0).all()
            continue
        assert_close(out[b, :n], want[b, :n], f"seqused_q row {b}")
        fin = torch.isfinite(want_lse[b, :, :n])
        assert torch.allclose(lse[b, :, :n].cpu()[fin], want_lse[b, :, :n][fin], atol=2e-3, rtol=1e-3)
        assert torch.equal(torch.isinf(lse[b, :, :n].cpu()), ~fin)
    out, want = run_case(p, torch.bfloat16, causal=False)
    assert_close(out, want, "non-causal")


@pytest.mark.parametrize("window", [0, 5, 31, 32, 100, 4000])
@pytest.mark.parametrize("kv,seqlen_q", [("same", 2), ("fp8", 2), ("fp8", 1)])
def test_sliding_window(window, kv, seqlen_q):
    lengths = [1, 30, 33, 64, 100, 101, 700]
    p = make_paged_problem(seed=11, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=8, n_kv_heads=2, head_dim=128,
                           page_size=16, seqlen_q=seqlen_q, dtype=torch.bfloat16, lengths=lengths)
    out, want = run_case(p, torch.bfloat16, kv=kv, window=window, causal=False,
                         scales=(0.02, 0.02) if kv == "fp8" else None)
    assert_close(out, want, f"window={window}")


@pytest.mark.parametrize("page_size", [1, 2, 4, 8, 32, 64, 128])
@pytest.mark.parametrize("kv,head_dim", [("same", 128), ("same", 64), ("fp8", 128), ("fp8", 64)])
def test_page_sizes(page_size, kv, head_dim):
    lengths = [1, 2, 9, 63, 64, 65, 130, 257]
    p = make_paged_problem(seed=13, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=8, n_kv_heads=2,
                           head_dim=head_dim, page_size=page_size, dtype=torch.bfloat16, lengths=lengths)
    out, want = run_case(p, torch.bfloat16, kv=kv, scales=(0.02, 0.02) if kv == "fp8" else None)
    assert_close(out, want, f"P={page_size}")


@pytest.mark.parametrize("heads_q,heads_kv,seqlen_q", [(32, 32, 1), (32, 8, 1), (32, 8, 4), (8, 8, 64), (32, 8, 3)])
def test_fp8_pool_with_one_token_pages_and_64_byte_rows(heads_q, heads_kv, seqlen_q):
    """The reference's own FP8 configuration (page size 1, head_dim 64, e4m3 with per-layer scalar scales,
    kestrel/models/moondream/runtime.py:645-663; Moondream is MHA 32/32): a token row of one head is 64 bytes,
    too short for a TMA box, so the warps gather their tiles with 16-byte asynchronous copies.  Decode
    (transposed kernel), multi-query verify (16-row kernel) and a prefill-shaped call, which stays on the
    split-KV kernels for such pools."""
    lengths = [1, 2, 31, 63, 64, 65, 127, 129, 700, 2100]
    p = make_paged_problem(seed=19, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=heads_q, n_kv_heads=heads_kv,
                           head_dim=64, page_size=1, seqlen_q=seqlen_q, dtype=torch.bfloat16,
                           lengths=[L + seqlen_q for L in lengths], outlier_frac=0.01)
    ks = float(p["k_pool"].abs().max() / 448)
    vs = float(p["v_pool"].abs().max() / 448)
    out, want = run_case(p, torch.bfloat16, kv="fp8", scales=(ks, vs))
    assert_close(out, want, f"P=1 D=64 e4m3, {heads_q}/{heads_kv} heads, Sq={seqlen_q}")


@pytest.mark.parametrize("heads_q,heads_kv,head_dim,seqlen_q,page_size", [
    (32, 32, 64, 1, 1),    # the reference's own FP8 geometry: four KV heads read as one wide head of 256
    (32, 32, 64, 2, 1),    # two query tokens: all 8 rows of the wide head's segment
    (16, 8, 64, 1, 1),     # GQA 2 x four heads
    (12, 12, 64, 1, 2),    # pages of two tokens, twelve heads = three packs
    (32, 8, 128, 1, 1),    # 128-byte rows: two KV heads per pack, GQA 4
    (8, 4, 128, 2, 2),
    (6, 6, 64, 1, 1),      # six heads are not a multiple of four: no packing
])
@pytest.mark.parametrize("qdtype", [torch.bfloat16, torch.float16])
def test_fp8_pools_with_tiny_pages_read_several_heads_as_one(heads_q, heads_kv, head_dim, seqlen_q, page_size, qdtype):
    """e4m3 pools with pages of one or two tokens and per-layer scalar scales: KV heads whose rows lie side by
    side are read as one head of 256 bytes.  Edge lengths, an empty sequence, one sequence long enough to be cut
    by many tile ranges (the merge on the wide head), log-sum-exp."""
    lengths = [1, 2, 15, 16, 17, 63, 64, 65, 129, 700, 0, 9000]
    p = make_paged_problem(seed=91, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=heads_q, n_kv_heads=heads_kv,
                           head_dim=head_dim, page_size=page_size, seqlen_q=seqlen_q, dtype=qdtype,
                           lengths=[L + seqlen_q if L else 0 for L in lengths], outlier_frac=0.01)
    ks = float(p["k_pool"].abs().max() / 448)
    vs = float(p["v_pool"].abs().max() / 448)
    out, want, lse, want_lse = run_case(p, qdtype, kv="fp8", scales=(ks, vs), return_lse=True)
    for b, L in enumerate(lengths):
        if L == 0:
            assert (out[b] == 0).all() and torch.isinf(lse[b]).all()
            continue
        assert_close(out[b], want[b], f"packed heads {heads_q}/{heads_kv} D={head_dim} P={page_size} sequence {b}")
        fin = torch.isfinite(want_lse[b])
        assert torch.allclose(lse[b].cpu()[fin], want_lse[b][fin], atol=3e-3, rtol=1e-3)


@pytest.mark.parametrize("heads_q,heads_kv,seqlen_q,page_size", [(32, 32, 1, 1), (32, 32, 4, 1), (16, 8, 1, 2), (6, 6, 2, 1), (5, 5, 1, 1)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_16_bit_pools_with_tiny_pages_read_two_heads_as_one(heads_q, heads_kv, seqlen_q, page_size, dtype):
    """The reference's default pools (page size 1, kestrel/config.py:164; MHA heads of 64): a (token, head) row has
    128 bytes, two heads side by side are read as one of 256.  Five heads cannot pair up and stay single."""
    lengths = [1, 2, 15, 16, 17, 63, 64, 65, 129, 700, 0, 9000]
    p = make_paged_problem(seed=93, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=heads_q, n_kv_heads=heads_kv,
                           head_dim=64, page_size=page_size, seqlen_q=seqlen_q, dtype=dtype,
                           lengths=[L + seqlen_q if L else 0 for L in lengths])
    out, want, lse, want_lse = run_case(p, dtype, return_lse=True)
    for b, L in enumerate(lengths):
        if L == 0:
            assert (out[b] == 0).all() and torch.isinf(lse[b]).all()
            continue
        assert_close(out[b], want[b], f"paired heads {heads_q}/{heads_kv} P={page_size} Sq={seqlen_q} sequence {b}")
        fin = torch.isfinite(want_lse[b])
        assert torch.allclose(lse[b].cpu()[fin], want_lse[b][fin], atol=3e-3, rtol=1e-3)


@pytest.mark.parametrize("window,causal", [(None, False), (0, True), (40, True), (1000, True)])
def test_fp8_packed_heads_masks_and_seqused_q(window, causal):
    lengths = [5, 64, 130, 700, 2500]
    p = make_paged_problem(seed=92, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=16, n_kv_heads=16, head_dim=64,
                           page_size=1, seqlen_q=2, dtype=torch.bfloat16, lengths=lengths)
    sq = torch.tensor([2, 1, 2, 0, 2], dtype=torch.int32)
    out, want = run_case(p, torch.bfloat16, kv="fp8", scales=(0.02, 0.03), causal=causal, window=window, seqused_q=sq)
    for b, n in enumerate(sq.tolist()):
        if n:
            assert_close(out[b, :n], want[b, :n], f"packed heads window={window} causal={causal} sequence {b}")


@pytest.mark.parametrize("kv", ["same", "fp8"])
def test_single_long_sequence_is_split_across_warps_and_merged(kv):
    """One sequence of 20k keys: every (head) segment is cut into many partials that the merge combines."""
    p = make_paged_problem(seed=17, batch=2, len_lo=0, len_hi=0, n_q_heads=8, n_kv_heads=2, head_dim=128, page_size=16,
                           dtype=torch.bfloat16, lengths=[20011, 3], seqlen_q=2)
    out, want, lse, want_lse = run_case(p, torch.bfloat16, kv=kv, scales=(0.02, 0.02) if kv == "fp8" else None,
                                        return_lse=True)
    assert_close(out, want, "long")
    assert torch.allclose(lse.cpu(), want_lse, atol=2e-3, rtol=1e-3)


def test_long_sequences_cut_by_dozens_of_ranges():
    """270k keys in three sequences: every (sequence, head) segment is spread over dozens of warps' tile ranges
    (more than one 32-lane ballot's worth for the longest), on the 16-bit and the FP8 kernels."""
    p = make_paged_problem(seed=77, batch=3, len_lo=0, len_hi=0, n_q_heads=32, n_kv_heads=8, head_dim=128,
                           page_size=16, dtype=torch.bfloat16, lengths=[150001, 70003, 49999])
    out, want, lse, want_lse = run_case(p, torch.bfloat16, return_lse=True)
    assert_close(out, want, "bf16")
    assert torch.allclose(lse.cpu(), want_lse, atol=2e-3, rtol=1e-3)
    out, want = run_case(p, torch.bfloat16, kv="fp8", scales=(0.03, 0.02))
    assert_close(out, want, "fp8")
    p["q"] = p["q"].repeat(1, 4, 1, 1)      # 4 query rows per sequence: the 16-row kernel on the FP8 pool
    out, want = run_case(p, torch.bfloat16, kv="fp8", scales=(0.03, 0.02))
    assert_close(out, want, "fp8 verify")


def test_peaked_softmax_and_custom_scale():
    """Scores with a large dynamic range: one key dominates; softmax_scale=1.0 as Gemma passes."""
    p = make_paged_problem(seed=19, batch=4, len_lo=200, len_hi=900, n_q_heads=8, n_kv_heads=2, head_dim=64,
                           page_size=16, dtype=torch.bfloat16)
    out, want = run_case(p, torch.bfloat16, softmax_scale=1.0)
    assert_close(out, want, "scale=1")


def test_op_surface_strided_query_and_layer_object():
    """paged_attention(query [B,H,S,D]) on a query sliced out of a fused QKV projection."""
    B, Hq, Hkv, D, P = 5, 32, 8, 128, 16
    p = make_paged_problem(seed=23, batch=B, len_lo=10, len_hi=400, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D,
                           page_size=P, dtype=torch.bfloat16)
    fused = torch.zeros(B, 1, (Hq + 2 * Hkv) * D, dtype=torch.bfloat16, device=DEV)
    fused[..., : Hq * D] = p["q"].to(torch.bfloat16).reshape(B, 1, Hq * D).to(DEV)
    q_bshd = fused[..., : Hq * D].view(B, 1, Hq, D)
    query = q_bshd.transpose(1, 2)  # what model code holds: [B, H, S, D]

    class Layer:
        k_cache = p["k_pool"].to(torch.bfloat16).to(DEV)
        v_cache = p["v_pool"].to(torch.bfloat16).to(DEV)
        k_scale = 1.0
        v_scale = 1.0

    out = paged_attention(query, paged_kv_layer=Layer, page_table=p["page_table"].to(DEV),
                          paged_kv_seqlens_k=p["seqused_k"].to(DEV), scaling=1.0 / math.sqrt(D))
    want = O.paged_attention(p["q"].to(torch.bfloat16).float(), p["k_pool"], p["v_pool"], p["page_table"], p["seqused_k"])
    assert out.shape == (B, 1, Hq, D)
    assert_close(out, want, "op surface")
    with pytest.raises(RuntimeError, match="requires fp16/bf16 query"):
        paged_attention(query.float(), paged_kv_layer=Layer, page_table=p["page_table"].to(DEV),
                        paged_kv_seqlens_k=p["seqused_k"].to(DEV), scaling=1.0)
    win = paged_attention(query, paged_kv_layer=Layer, page_table=p["page_table"].to(DEV),
                          paged_kv_seqlens_k=p["seqused_k"].to(DEV), scaling=1.0 / math.sqrt(D), sliding_window=8)
    want_w = O.paged_attention(p["q"].to(torch.bfloat16).float(), p["k_pool"], p["v_pool"], p["page_table"],
                               p["seqused_k"], window_left=7)
    assert_close(win, want_w, "sliding_window=8")


def test_packed_queries_with_cu_seqlens():
    lengths = [40, 7, 129, 64]
    qlens = [3, 1, 4, 2]
    p = make_paged_problem(seed=29, batch=4, len_lo=0, len_hi=0, n_q_heads=8, n_kv_heads=2, head_dim=128, page_size=16,
                           seqlen_q=4, dtype=torch.bfloat16, lengths=lengths)
    rows = [p["q"][b, :n] for b, n in enumerate(qlens)]
    packed = torch.cat(rows).to(torch.bfloat16).to(DEV)
    cu = torch.tensor([0, 3, 4, 8, 10], dtype=torch.int32, device=DEV)
    out, _ = kernels.flash_attn_fwd(packed, p["k_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3),
                                    p["v_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3),
                                    page_table=p["page_table"].to(DEV), cu_seqlens_q=cu,
                                    seqused_k=p["seqused_k"].to(DEV), causal=True)
    want = O.paged_attention(p["q"].to(torch.bfloat16).float(), p["k_pool"], p["v_pool"], p["page_table"],
                             p["seqused_k"], seqused_q=torch.tensor(qlens))
    want_packed = torch.cat([want[b, :n] for b, n in enumerate(qlens)])
    assert_close(out, want_packed, "packed")


def test_unsupported_modes_raise():
    q = torch.zeros(1, 1, 8, 128, dtype=torch.bfloat16, device=DEV)
    kv = torch.zeros(4, 16, 2, 128, dtype=torch.bfloat16, device=DEV)
    pt = torch.zeros(1, 4, dtype=torch.int32, device=DEV)
    sk = torch.ones(1, dtype=torch.int32, device=DEV)
    with pytest.raises(NotImplementedError):
        kernels.flash_attn_fwd(q, kv, kv)
    with pytest.raises(NotImplementedError):
        kernels.flash_attn_fwd(q, kv, kv, page_table=pt, seqused_k=sk, mask_mod=object())
    with pytest.raises(NotImplementedError):
        kernels.flash_attn_fwd(q, kv, kv, page_table=pt, seqused_k=sk, window_size_left=3, window_size_right=2)
    with pytest.raises(NotImplementedError, match="head_dim"):
        kernels.flash_attn_fwd(torch.zeros(1, 1, 8, 96, dtype=torch.bfloat16, device=DEV),
                               torch.zeros(4, 16, 2, 96, dtype=torch.bfloat16, device=DEV),
                               torch.zeros(4, 16, 2, 96, dtype=torch.bfloat16, device=DEV), page_table=pt, seqused_k=sk)
    with pytest.raises(NotImplementedError, match="page_size"):
        kv3 = torch.zeros(4, 3, 2, 128, dtype=torch.bfloat16, device=DEV)
        kernels.flash_attn_fwd(q, kv3, kv3, page_table=pt, seqused_k=sk)
    with pytest.raises(ValueError, match="must equal the query dtype"):
        kernels.flash_attn_fwd(q, kv.half(), kv.half(), page_table=pt, seqused_k=sk)


def test_bad_page_index_is_reported_not_faulted():
    p = make_paged_problem(seed=31, batch=2, len_lo=0, len_hi=0, n_q_heads=8, n_kv_heads=2, head_dim=128, page_size=16,
                           dtype=torch.bfloat16, lengths=[40, 40])
    table = p["page_table"].clone()
    table[1, 1] = p["n_pages"] + 1000  # outside the pool: the copy unit zero-fills, nothing is read
    out, _ = kernels.flash_attn_fwd(p["q"].to(torch.bfloat16).to(DEV), p["k_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3),
                                    p["v_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3), page_table=table.to(DEV),
                                    seqused_k=p["seqused_k"].to(DEV), causal=True)
    flags = _native.device_status(torch.cuda.current_device(), clear=True)
    assert flags[0] == _native.STATUS_BAD_PAGE and flags[1] == p["n_pages"] + 1000
    want = O.paged_attention(p["q"].to(torch.bfloat16).float(), p["k_pool"], p["v_pool"], p["page_table"], p["seqused_k"])
    assert_close(out[0], want[0], "untouched sequence")
    assert torch.isfinite(out.float()).all()


def test_baseline_config2_shape_full_batch():
    """bf16, batch 64, contexts U[1024, 8192], 32/8 heads, D=128, page 16, pool 1.25x, scattered pages."""
    p = make_paged_problem(seed=1002, batch=64, len_lo=1024, len_hi=8192, n_q_heads=32, n_kv_heads=8, head_dim=128,
                           page_size=16, dtype=torch.bfloat16)
    out, want = run_case(p, torch.bfloat16)
    assert_close(out, want, "config 2")


def test_graph_capture_and_replay_with_changing_lengths():
    """The op is allocation-free after workspace reservation and reads lengths/pages from device
    memory, so one captured graph serves steps with different lengths."""
    p = make_paged_problem(seed=37, batch=6, len_lo=50, len_hi=600, n_q_heads=32, n_kv_heads=8, head_dim=128,
                           page_size=16, dtype=torch.bfloat16)
    q = p["q"].to(torch.bfloat16).to(DEV)
    k = p["k_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3)
    v = p["v_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3)
    table = p["page_table"].to(DEV)
    seq = p["seqused_k"].to(DEV)
    out = torch.empty_like(q)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        kernels.reserve_attention_workspace(batch=6, total_q=6, n_q_heads=32, n_kv_heads=8, head_dim=128)
        kernels.flash_attn_fwd(q, k, v, page_table=table, seqused_k=seq, causal=True, out=out)  # warm-up
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            kernels.flash_attn_fwd(q, k, v, page_table=table, seqused_k=seq, causal=True, out=out)
    for shrink in (0, 7, 33):
        new_len = (p["seqused_k"] - shrink).clamp(min=1)
        seq.copy_(new_len.to(DEV))
        graph.replay()
        torch.cuda.synchronize()
        want = O.paged_attention(p["q"].to(torch.bfloat16).float(), p["k_pool"], p["v_pool"], p["page_table"], new_len)
        assert_close(out, want, f"replay shrink={shrink}")
