"""GPU parity of the 32-row split-KV kernel (17 to 39 packed query rows per KV head; up to 55 with head_dim 64)
against the fp32 CPU oracle: an 8-token verify at GQA 4, a 4-token verify at GQA 8, short prompt chunks.

Same tolerance as ``test_gpu_attention.py`` (2e-2 absolute / 1e-2 relative per element, 1e-2 relative L2 per row).
"""

import pytest
import torch

from helpers import make_paged_problem
from kestrel_b200 import kernels
from oracle import paged_kv_oracle as O
from test_gpu_attention import DEV, _clean_status, assert_close, run_case  # noqa: F401  (autouse fixture)

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seqlen_q,group,heads_kv", [(8, 4, 2), (4, 8, 2), (17, 1, 3), (5, 4, 4), (32, 1, 2), (3, 6, 2),
                                                      (33, 1, 2), (39, 1, 2), (9, 4, 1), (2, 16, 1)])
@pytest.mark.parametrize("kv", ["same", "fp8"])
@pytest.mark.parametrize("head_dim", [128, 64])
def test_shapes_with_17_to_39_rows(seqlen_q, group, heads_kv, kv, head_dim):
    lengths = [seqlen_q, seqlen_q + 1, seqlen_q + 15, 64, 65, seqlen_q + 113, 3 * seqlen_q + 500, max(1, seqlen_q - 5), 7]
    p = make_paged_problem(seed=40 + seqlen_q, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=group * heads_kv,
                           n_kv_heads=heads_kv, head_dim=head_dim, page_size=16, seqlen_q=seqlen_q,
                           dtype=torch.bfloat16, lengths=lengths)
    out, want = run_case(p, torch.bfloat16, kv=kv, scales=(0.02, 0.03) if kv == "fp8" else None)
    assert_close(out, want, f"Sq={seqlen_q} G={group} Hkv={heads_kv} D={head_dim} kv={kv}")


@pytest.mark.parametrize("kv,dtype", [("same", torch.bfloat16), ("same", torch.float16), ("fp8", torch.bfloat16),
                                      ("fp8", torch.float16)])
def test_long_sequences_are_cut_and_merged_with_two_slots_per_worker(kv, dtype):
    """20k and 9k keys against 32 rows: every segment is spread over many warps; log-sum-exp checked too."""
    p = make_paged_problem(seed=51, batch=3, len_lo=0, len_hi=0, n_q_heads=8, n_kv_heads=2, head_dim=128, page_size=16,
                           dtype=dtype, lengths=[20011, 9000, 40], seqlen_q=8)
    out, want, lse, want_lse = run_case(p, dtype, kv=kv, scales=(0.02, 0.02) if kv == "fp8" else None, return_lse=True)
    assert_close(out, want, "long")
    assert torch.allclose(lse.cpu(), want_lse, atol=2e-3, rtol=1e-3)


@pytest.mark.parametrize("page_size", [1, 2, 4, 8, 32, 64, 128])
@pytest.mark.parametrize("kv,head_dim", [("same", 128), ("same", 64), ("fp8", 128), ("fp8", 64)])
def test_page_sizes(page_size, kv, head_dim):
    lengths = [300, 64, 65, 1, 513, 2000]
    p = make_paged_problem(seed=52, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=8, n_kv_heads=2, head_dim=head_dim,
                           page_size=page_size, seqlen_q=6, dtype=torch.bfloat16, lengths=lengths)
    out, want = run_case(p, torch.bfloat16, kv=kv, scales=(0.02, 0.03) if kv == "fp8" else None)
    assert_close(out, want, f"page_size={page_size} kv={kv} D={head_dim}")


@pytest.mark.parametrize("window", [0, 5, 31, 100, 4000])
@pytest.mark.parametrize("kv", ["same", "fp8"])
def test_sliding_window_and_non_causal(window, kv):
    lengths = [6, 30, 33, 64, 100, 101, 700]
    p = make_paged_problem(seed=53, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=8, n_kv_heads=2, head_dim=128,
                           page_size=16, seqlen_q=6, dtype=torch.bfloat16, lengths=lengths)
    scales = (0.02, 0.02) if kv == "fp8" else None
    out, want = run_case(p, torch.bfloat16, kv=kv, window=window, scales=scales)
    assert_close(out, want, f"window={window}")
    out, want = run_case(p, torch.bfloat16, kv=kv, causal=False, scales=scales)
    assert_close(out, want, "non-causal")


def test_seqused_q_leaves_rows_past_the_end_untouched():
    lengths = [7, 64, 65, 200, 0, 31]
    p = make_paged_problem(seed=54, batch=len(lengths), len_lo=0, len_hi=0, n_q_heads=8, n_kv_heads=2, head_dim=64,
                           page_size=16, seqlen_q=7, dtype=torch.bfloat16, lengths=lengths)
    sq = torch.tensor([7, 1, 5, 0, 2, 4], dtype=torch.int32)
    out, want, lse, want_lse = run_case(p, torch.bfloat16, seqused_q=sq, return_lse=True)
    for b, n in enumerate(sq.tolist()):
        if n == 0:
            continue
        if lengths[b] == 0:
            assert (out[b, :n] == 0).all()
            continue
        assert_close(out[b, :n], want[b, :n], f"seqused_q row {b}")
        fin = torch.isfinite(want_lse[b, :, :n])
        assert torch.allclose(lse[b, :, :n].cpu()[fin], want_lse[b, :, :n][fin], atol=2e-3, rtol=1e-3)


def test_packed_rows_of_mixed_lengths():
    """Packed queries, 1 to 9 tokens per sequence at GQA 4 (mean 20 rows): sequences of 16 rows or fewer leave
    the second block of their segment empty."""
    lengths = [400, 70, 1290, 64, 3000]
    qlens = [9, 1, 8, 2, 5]
    p = make_paged_problem(seed=55, batch=5, len_lo=0, len_hi=0, n_q_heads=8, n_kv_heads=2, head_dim=128, page_size=16,
                           seqlen_q=9, dtype=torch.bfloat16, lengths=lengths)
    packed = torch.cat([p["q"][b, :n] for b, n in enumerate(qlens)]).to(torch.bfloat16).to(DEV)
    cu = torch.tensor([0, 9, 10, 18, 20, 25], dtype=torch.int32, device=DEV)
    out, _ = kernels.flash_attn_fwd(packed, p["k_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3),
                                    p["v_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3),
                                    page_table=p["page_table"].to(DEV), cu_seqlens_q=cu,
                                    seqused_k=p["seqused_k"].to(DEV), causal=True)
    want = O.paged_attention(p["q"].to(torch.bfloat16).float(), p["k_pool"], p["v_pool"], p["page_table"],
                             p["seqused_k"], seqused_q=torch.tensor(qlens))
    assert_close(out, torch.cat([want[b, :n] for b, n in enumerate(qlens)]), "packed")


@pytest.mark.parametrize("batch", [16, 64])
def test_verify_batch_at_full_size(batch):
    """Contexts U[2048, 16384], 8-token verify at GQA 4 (the 4-token verify configuration's shape with twice the
    tokens per step).  16 sequences x 8 KV heads stay on the 32-row kernel; 64 x 8 reach the SM count and go to the
    tensor-memory kernel with its key split."""
    p = make_paged_problem(seed=56, batch=batch, len_lo=2048, len_hi=16384, n_q_heads=32, n_kv_heads=8, head_dim=128,
                           page_size=16, seqlen_q=8, dtype=torch.bfloat16, pool_factor=1.02)
    out, want = run_case(p, torch.bfloat16)
    assert_close(out, want, "verify batch")


@pytest.mark.parametrize("bound", [None, 8])
def test_packed_rows_with_and_without_a_row_bound_at_a_batch_that_fills_the_sms(bound):
    """40 sequences x 4 KV heads (a CTA per SM), 5 to 8 packed query tokens at GQA 4.  With ``max_seqlen_q`` the call
    may take the tensor-memory kernel's key split; without it (the reference's packed call passes none,
    kestrel/ops/attention.py:69-86) nothing bounds a sequence's rows and the 32-row kernel keeps the call."""
    import random
    rng = random.Random(5)
    batch = 40
    lengths = [rng.randint(40, 900) for _ in range(batch)]
    qlens = [rng.randint(5, 8) for _ in range(batch)]
    p = make_paged_problem(seed=57, batch=batch, len_lo=0, len_hi=0, n_q_heads=16, n_kv_heads=4, head_dim=128, page_size=16,
                           seqlen_q=8, dtype=torch.bfloat16, lengths=lengths)
    packed = torch.cat([p["q"][b, :n] for b, n in enumerate(qlens)]).to(torch.bfloat16).to(DEV)
    cu = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device=DEV)
    kw = {} if bound is None else {"max_seqlen_q": bound}
    out, _ = kernels.flash_attn_fwd(packed, p["k_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3),
                                    p["v_pool"].to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3),
                                    page_table=p["page_table"].to(DEV), cu_seqlens_q=cu,
                                    seqused_k=p["seqused_k"].to(DEV), causal=True, **kw)
    want = O.paged_attention(p["q"].to(torch.bfloat16).float(), p["k_pool"], p["v_pool"], p["page_table"],
                             p["seqused_k"], seqused_q=torch.tensor(qlens))
    assert_close(out, torch.cat([want[b, :n] for b, n in enumerate(qlens)]), f"packed, bound={bound}")
