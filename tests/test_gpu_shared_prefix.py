"""GPU parity of attention over a shared cached prefix (``shared_prefix_pages``).

Requests attached to one radix-cache prefix map the same physical pages at the start of their page-table
rows.  With the hint the library reads those pages once for the whole batch (one pass of all query rows over
the prefix, one pass per sequence over the rest, combined by their log-sum-exps); the result must equal
the plain call's and the fp32 oracle's within the attention tolerance (2e-2 absolute / 1e-2 relative).
"""

import pytest
import torch

from helpers import make_paged_problem
from kestrel_b200 import _native, kernels
from oracle import paged_kv_oracle as O
from test_gpu_attention import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _clean_status():
    _native.device_status(torch.cuda.current_device(), clear=True)
    yield
    flags = _native.device_status(torch.cuda.current_device(), clear=True)
    assert flags[0] == 0, f"kernel diagnostics: {flags}"


def shared_problem(*, seed, batch, n_shared, extra_lo, extra_hi, head_dim, seqlen_q=1, n_kv_heads=8, page_size=16,
                   dtype=torch.bfloat16, extras=None):
    """Every sequence = the same n_shared full pages + its own extra tokens (>= seqlen_q)."""
    g = torch.Generator().manual_seed(seed)
    if extras is None:
        extras = torch.randint(extra_lo, extra_hi + 1, (batch,), generator=g).tolist()
    lengths = [n_shared * page_size + e for e in extras]
    p = make_paged_problem(seed=seed, batch=batch, len_lo=0, len_hi=0, n_q_heads=32, n_kv_heads=n_kv_heads,
                           head_dim=head_dim, page_size=page_size, seqlen_q=seqlen_q, dtype=dtype, lengths=lengths)
    p["page_table"][:, :n_shared] = p["page_table"][0, :n_shared].clone()
    return p


def run(p, dtype, n_shared, *, causal=True, fp8=False, return_lse=False, q_dev=None):
    q = p["q"].to(dtype).to(DEV) if q_dev is None else q_dev
    kw = {}
    if fp8:
        ks = torch.full((p["k_pool"].shape[1],), 0.02)
        vs = torch.full((p["k_pool"].shape[1],), 0.03)
        kq = O.fp8_quantise(p["k_pool"].permute(0, 2, 1, 3), ks).permute(0, 2, 1, 3).contiguous()
        vq = O.fp8_quantise(p["v_pool"].permute(0, 2, 1, 3), vs).permute(0, 2, 1, 3).contiguous()
        k_dev, v_dev = kq.to(DEV).view(torch.float8_e4m3fn), vq.to(DEV).view(torch.float8_e4m3fn)
        k_ref, v_ref = kq, vq
        kw = dict(k_scale=ks.to(DEV), v_scale=vs.to(DEV))
        okw = dict(k_scale=ks, v_scale=vs)
    else:
        k_dev, v_dev = p["k_pool"].to(dtype).to(DEV), p["v_pool"].to(dtype).to(DEV)
        k_ref, v_ref = p["k_pool"], p["v_pool"]
        okw = {}
    common = dict(page_table=p["page_table"].to(DEV), seqused_k=p["seqused_k"].to(DEV), causal=causal,
                  return_lse=return_lse, **kw)
    got = kernels.flash_attn_fwd(q, k_dev.permute(0, 2, 1, 3), v_dev.permute(0, 2, 1, 3),
                                 shared_prefix_pages=n_shared, **common)
    plain = kernels.flash_attn_fwd(q, k_dev.permute(0, 2, 1, 3), v_dev.permute(0, 2, 1, 3), **common)
    want = O.paged_attention(p["q"].to(dtype).float(), k_ref, v_ref, p["page_table"], p["seqused_k"], causal=causal,
                             return_lse=return_lse, **okw)
    return got, plain, want


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("head_dim", [64, 128])
def test_decode_on_shared_prefix(dtype, head_dim):
    # 45 shared pages = the full pages of a 729-token image prefix; suffix lengths ragged, some minimal
    p = shared_problem(seed=3, batch=40, n_shared=45, extra_lo=1, extra_hi=300, head_dim=head_dim, dtype=dtype,
                       extras=[1, 2, 15, 16, 17, 33] + [50 + 7 * i for i in range(34)])
    (out, _), (plain, _), want = run(p, dtype, 45)
    assert_close(out, want, f"shared {dtype} D={head_dim}")
    assert_close(plain, want, "plain")
    # the two paths differ only by the rounding of the partial outputs to the 16-bit type
    assert (out.float() - plain.float()).abs().max().item() < (2e-2 if dtype == torch.bfloat16 else 4e-3)


@pytest.mark.parametrize("seqlen_q", [2, 4])
def test_multi_query_rows_and_lse(seqlen_q):
    p = shared_problem(seed=5, batch=24, n_shared=20, extra_lo=seqlen_q, extra_hi=200, head_dim=128, seqlen_q=seqlen_q,
                       extras=[seqlen_q, seqlen_q + 1] + [30 + 9 * i for i in range(22)])
    (out, lse), (plain, lse_plain), (want, want_lse) = run(p, torch.bfloat16, 20, return_lse=True)
    assert_close(out, want, f"Sq={seqlen_q}")
    assert torch.allclose(lse.cpu(), want_lse, atol=2e-3, rtol=1e-3)
    assert torch.allclose(lse.cpu(), lse_plain.cpu(), atol=2e-3, rtol=1e-3)


@pytest.mark.parametrize("page_size,n_shared", [(16, 40), (64, 9), (128, 5)])
def test_long_prefix_is_cut_in_two_key_ranges(page_size, n_shared):
    # few CTAs and at least four tiles of prefix keys: the prefix pass runs as two sequences of keys over
    # the same query rows (three partial results per row to combine); log-sum-exp checked as well
    p = shared_problem(seed=23, batch=24, n_shared=n_shared, extra_lo=2, extra_hi=150, head_dim=128, seqlen_q=2,
                       page_size=page_size)
    (out, lse), (plain, lse_plain), (want, want_lse) = run(p, torch.bfloat16, n_shared, return_lse=True)
    assert_close(out, want, f"P={page_size}")
    assert torch.allclose(lse.cpu(), want_lse, atol=2e-3, rtol=1e-3)


def test_non_causal_and_suffix_empty():
    # without the causal mask a sequence may consist of the shared pages alone
    p = shared_problem(seed=7, batch=20, n_shared=8, extra_lo=0, extra_hi=0, head_dim=64,
                       extras=[0, 0, 1, 16, 40] + [3 * i for i in range(15)])
    (out, _), _, want = run(p, torch.bfloat16, 8, causal=False)
    assert_close(out, want, "non-causal")


@pytest.mark.parametrize("head_dim", [64, 128])
def test_fp8_pools(head_dim):
    p = shared_problem(seed=9, batch=32, n_shared=45, extra_lo=1, extra_hi=256, head_dim=head_dim)
    (out, _), _, want = run(p, torch.bfloat16, 45, fp8=True)
    assert_close(out, want, f"fp8 D={head_dim}")


def test_mha_heads_and_page_size_64():
    p = shared_problem(seed=11, batch=16, n_shared=6, extra_lo=1, extra_hi=200, head_dim=64, n_kv_heads=32,
                       page_size=64)
    (out, _), _, want = run(p, torch.bfloat16, 6)
    assert_close(out, want, "MHA, 64-token pages")


def test_strided_query_rows():
    # q as a slice of a fused qkv buffer (row stride larger than the row)
    p = shared_problem(seed=13, batch=32, n_shared=10, extra_lo=4, extra_hi=100, head_dim=128, seqlen_q=4)
    fused = torch.zeros(32, 4, 48, 128, dtype=torch.bfloat16, device=DEV)
    fused[:, :, :32] = p["q"].to(torch.bfloat16).to(DEV)
    (out, _), _, want = run(p, torch.bfloat16, 10, q_dev=fused[:, :, :32])
    assert_close(out, want, "strided q")


def test_hint_is_ignored_where_it_does_not_apply():
    # few query rows (below the tensor-memory kernel's threshold), a window, seqused_q: plain path, same bits
    p = shared_problem(seed=15, batch=2, n_shared=4, extra_lo=1, extra_hi=50, head_dim=128)
    (out, _), (plain, _), want = run(p, torch.bfloat16, 4)
    assert torch.equal(out, plain)
    p = shared_problem(seed=16, batch=32, n_shared=4, extra_lo=1, extra_hi=50, head_dim=128)
    q = p["q"].to(torch.bfloat16).to(DEV)
    kd, vd = p["k_pool"].to(torch.bfloat16).to(DEV), p["v_pool"].to(torch.bfloat16).to(DEV)
    args = dict(page_table=p["page_table"].to(DEV), seqused_k=p["seqused_k"].to(DEV), causal=True, window_size_left=31)
    a, _ = kernels.flash_attn_fwd(q, kd.permute(0, 2, 1, 3), vd.permute(0, 2, 1, 3), shared_prefix_pages=4, **args)
    b, _ = kernels.flash_attn_fwd(q, kd.permute(0, 2, 1, 3), vd.permute(0, 2, 1, 3), **args)
    assert torch.equal(a, b)
    with pytest.raises(ValueError):
        kernels.flash_attn_fwd(q, kd.permute(0, 2, 1, 3), vd.permute(0, 2, 1, 3), shared_prefix_pages=10 ** 6, **args)


def test_a_broken_promise_is_reported():
    # sequence 3 is shorter than the prefix it is said to share
    p = shared_problem(seed=17, batch=32, n_shared=4, extra_lo=1, extra_hi=50, head_dim=128)
    p["seqused_k"][3] = 40
    dev = torch.cuda.current_device()
    q = p["q"].to(torch.bfloat16).to(DEV)
    kd, vd = p["k_pool"].to(torch.bfloat16).to(DEV), p["v_pool"].to(torch.bfloat16).to(DEV)
    kernels.flash_attn_fwd(q, kd.permute(0, 2, 1, 3), vd.permute(0, 2, 1, 3), page_table=p["page_table"].to(DEV),
                           seqused_k=p["seqused_k"].to(DEV), causal=True, shared_prefix_pages=4)
    torch.cuda.synchronize()
    flags = _native.device_status(dev, clear=True)
    assert flags[0] == _native.STATUS_BAD_PREFIX and flags[1] == 3


def test_graph_replay():
    p = shared_problem(seed=19, batch=48, n_shared=12, extra_lo=1, extra_hi=120, head_dim=64)
    q = p["q"].to(torch.bfloat16).to(DEV)
    kd, vd = p["k_pool"].to(torch.bfloat16).to(DEV), p["v_pool"].to(torch.bfloat16).to(DEV)
    pt, sk = p["page_table"].to(DEV), p["seqused_k"].to(DEV)
    out = torch.empty_like(q)
    call = lambda: kernels.flash_attn_fwd(q, kd.permute(0, 2, 1, 3), vd.permute(0, 2, 1, 3), page_table=pt,
                                          seqused_k=sk, causal=True, out=out, shared_prefix_pages=12)
    call()
    torch.cuda.synchronize()
    first = out.clone()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        call()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            call()
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, first)
    want = O.paged_attention(p["q"].to(torch.bfloat16).float(), p["k_pool"], p["v_pool"], p["page_table"], p["seqused_k"],
                             causal=True)
    assert_close(out, want, "graph replay")


def test_through_the_allocation_free_entry_point():
    import ctypes as C
    import math
    lib = _native.load()
    p = shared_problem(seed=21, batch=32, n_shared=45, extra_lo=1, extra_hi=200, head_dim=64)
    q = p["q"].to(torch.bfloat16).to(DEV)
    k, v = p["k_pool"].to(torch.bfloat16).to(DEV), p["v_pool"].to(torch.bfloat16).to(DEV)
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
    a.batch, a.total_q, a.seqlen_q = 32, 32, 1
    a.n_q_heads, a.n_kv_heads, a.head_dim, a.page_size = 32, 8, 64, 16
    a.q_dtype = a.kv_dtype = _native.DTYPE_BF16
    a.softmax_scale, a.causal, a.window_left = 1.0 / math.sqrt(64), 1, -1
    a.k_scale = a.v_scale = 1.0
    plain_need = int(lib.kb200_attn_workspace_bytes_for(C.byref(a)))
    a.shared_prefix_pages = 45
    assert int(lib.kb200_attn_workspace_bytes_for(C.byref(a))) > plain_need   # both passes plus the first one's output
    _native.check(lib.kb200_paged_attention_static(C.byref(a)))
    torch.cuda.synchronize()
    want = O.paged_attention(p["q"].to(torch.bfloat16).float(), p["k_pool"], p["v_pool"], p["page_table"], p["seqused_k"])
    assert_close(out, want, "static entry point, shared prefix")
