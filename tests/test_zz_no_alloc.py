"""The allocation-free attention entry point, ``kb200_paged_attention_static``.

Some hosts cannot hand the library a scratch buffer: an engine that gave all of its HBM to the
KV pool at start-up, a C host without a device allocator, code running inside a stream capture.
For them the library carries a fixed 32 MiB scratch array in its device image.  This test drives
that entry point through the C ABI (a hand-filled ``kb200_attn_args``), twice in a row because all
calls share the one array, and checks the results against the ordinary entry point, which gets a
caller-allocated workspace, and against the CPU oracle.  It is collected last on purpose and needs no
state from other tests.
"""

import ctypes as C
import math

import pytest
import torch

from helpers import make_paged_problem
from kestrel_b200 import _native
from oracle import paged_kv_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
ABS_TOL, REL_TOL = 2e-2, 1e-2   # the tolerance of the other attention tests


def _args(q, out, k, v, table, seqused, *, kv_dtype, ks=None, vs=None, workspace=None):
    B, Sq, Hq, D = q.shape
    kv_view = k.permute(0, 2, 1, 3)  # [n_pages, P, H_kv, D] view of the pool
    a = _native.AttnArgs()
    a.struct_bytes = C.sizeof(_native.AttnArgs)
    a.device = q.device.index
    a.stream = torch.cuda.current_stream(q.device).cuda_stream
    a.q, a.out, a.lse = q.data_ptr(), out.data_ptr(), None
    a.q_batch_stride, a.q_row_stride, a.q_head_stride = q.stride(0), q.stride(1), q.stride(2)
    a.o_batch_stride, a.o_row_stride, a.o_head_stride = out.stride(0), out.stride(1), out.stride(2)
    a.k_cache, a.v_cache = k.data_ptr(), v.data_ptr()
    a.kv_page_stride, a.kv_token_stride, a.kv_head_stride = kv_view.stride(0), kv_view.stride(1), kv_view.stride(2)
    a.n_pages = k.shape[0]
    a.page_table, a.pt_row_stride = table.data_ptr(), table.stride(0)
    a.seqused_k, a.seqused_q, a.cu_seqlens_q = seqused.data_ptr(), None, None
    a.batch, a.total_q, a.seqlen_q = B, B * Sq, Sq
    a.n_q_heads, a.n_kv_heads, a.head_dim, a.page_size = Hq, k.shape[1], D, k.shape[2]
    a.q_dtype = _native.DTYPE_BF16
    a.kv_dtype = kv_dtype
    a.softmax_scale = 1.0 / math.sqrt(D)
    a.causal, a.window_left = 1, -1
    a.k_scale, a.v_scale = 1.0, 1.0
    a.k_scale_per_head = ks.data_ptr() if ks is not None else None
    a.v_scale_per_head = vs.data_ptr() if vs is not None else None
    if workspace is not None:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    else:
        a.workspace, a.workspace_bytes = None, 0
    return a


def _close(got, want):
    got, want = got.float(), want.float()
    assert torch.isfinite(got).all()
    assert ((got - want).abs() <= ABS_TOL + REL_TOL * want.abs()).all()


@pytest.mark.parametrize("kv", ["fp8", "bf16"])
def test_static_scratch_matches_caller_workspace_twice_in_a_row(kv):
    lib = _native.load()
    dev = torch.cuda.current_device()
    # two different problems, so the second call finds the first one's leftovers in the shared array;
    # the long sequence makes many warps leave partials there
    problems = [
        make_paged_problem(seed=41, batch=5, len_lo=0, len_hi=0, n_q_heads=32, n_kv_heads=8, head_dim=128,
                           page_size=16, dtype=torch.bfloat16, lengths=[9000, 17, 700, 1, 4096]),
        make_paged_problem(seed=42, batch=3, len_lo=0, len_hi=0, n_q_heads=32, n_kv_heads=8, head_dim=128,
                           page_size=16, dtype=torch.bfloat16, lengths=[33, 12000, 64]),
    ]
    for p in problems:
        q = p["q"].to(torch.bfloat16).to(DEV)
        table = p["page_table"].to(DEV)
        seqused = p["seqused_k"].to(DEV)
        if kv == "fp8":
            g = torch.Generator().manual_seed(1)
            k = torch.randint(0, 0x70, p["k_pool"].shape, generator=g, dtype=torch.uint8).to(DEV)
            v = torch.randint(0, 0x70, p["v_pool"].shape, generator=g, dtype=torch.uint8).to(DEV)
            ks = torch.full((8,), 0.05, device=DEV)
            vs = torch.full((8,), 0.03, device=DEV)
            kv_dtype = _native.DTYPE_E4M3
        else:
            k = p["k_pool"].to(torch.bfloat16).to(DEV)
            v = p["v_pool"].to(torch.bfloat16).to(DEV)
            ks = vs = None
            kv_dtype = _native.DTYPE_BF16
        B = q.shape[0]
        need = int(lib.kb200_attn_workspace_bytes(B, B, 32, 8, 128, dev))
        assert 0 < need <= _native.STATIC_SCRATCH_BYTES
        ws = torch.empty(need, dtype=torch.uint8, device=DEV)
        want = torch.empty_like(q)
        got = torch.full_like(q, float("nan"))
        _native.check(lib.kb200_paged_attention(C.byref(_args(q, want, k, v, table, seqused, kv_dtype=kv_dtype, ks=ks, vs=vs,
                                                              workspace=ws))))
        torch.cuda.synchronize()
        allocations = torch.cuda.memory_stats()["allocation.all.allocated"]   # count of allocation requests so far
        _native.check(lib.kb200_paged_attention_static(C.byref(_args(q, got, k, v, table, seqused, kv_dtype=kv_dtype,
                                                                     ks=ks, vs=vs))))
        torch.cuda.synchronize()
        # nothing went through torch's allocator either (frees by the garbage collector do not move this counter)
        assert torch.cuda.memory_stats()["allocation.all.allocated"] == allocations
        _close(got, want)
        # the same work, the same reduction order: the two entry points agree to the last bit
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        # and both are right: the fp32 oracle on the same pools
        ref = O.paged_attention(q.cpu().float(), k.cpu(), v.cpu(), p["page_table"], p["seqused_k"],
                                k_scale=None if ks is None else ks.cpu(), v_scale=None if vs is None else vs.cpu())
        _close(got.cpu(), ref)
        assert (got.float().cpu() - ref).abs().max().item() <= ABS_TOL
    flags = _native.device_status(dev, clear=True)
    assert flags[0] == 0, flags


def test_static_scratch_rejects_problems_that_do_not_fit():
    lib = _native.load()
    dev = torch.cuda.current_device()
    B = 4096
    assert int(lib.kb200_attn_workspace_bytes(B, B, 32, 8, 128, dev)) > _native.STATIC_SCRATCH_BYTES
    q = torch.zeros(B, 1, 32, 128, dtype=torch.bfloat16, device=DEV)
    k = torch.zeros(4, 8, 16, 128, dtype=torch.bfloat16, device=DEV)
    table = torch.zeros(B, 1, dtype=torch.int32, device=DEV)
    seqused = torch.ones(B, dtype=torch.int32, device=DEV)
    rc = lib.kb200_paged_attention_static(C.byref(_args(q, torch.empty_like(q), k, k, table, seqused,
                                                        kv_dtype=_native.DTYPE_BF16)))
    assert rc == -4
    msg = lib.kb200_last_error().decode()
    assert "built-in buffer" in msg and "kb200_paged_attention" in msg
    # largest decode batch (8 KV heads, head_dim 128) the built-in buffer serves
    # (sized as the entry point sizes it, for the call at hand; the bound over all calls of these dimensions is
    # larger: it also covers e4m3 pools with one-token pages, whose partials are twice as wide)
    a = _native.AttnArgs()
    a.struct_bytes = C.sizeof(_native.AttnArgs)
    a.device = dev
    a.seqlen_q, a.n_q_heads, a.n_kv_heads, a.head_dim, a.page_size = 1, 32, 8, 128, 16
    a.q_dtype = a.kv_dtype = _native.DTYPE_BF16

    def need(b):
        a.batch = a.total_q = b
        return int(lib.kb200_attn_workspace_bytes_for(C.byref(a)))

    fit = max(b for b in range(1, 400) if need(b) <= _native.STATIC_SCRATCH_BYTES)
    assert fit >= 128
    assert need(fit) <= int(lib.kb200_attn_workspace_bytes(fit, fit, 32, 8, 128, dev))
    print(f"static scratch serves decode batches up to {fit} (32 q / 8 kv heads, head_dim 128)")
