"""Seeded synthetic inputs shared by the CPU and GPU tests."""

from __future__ import annotations

import numpy as np
import torch


def from_np(a: np.ndarray, dtype: str) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype == "bfloat16":
        return t.view(torch.bfloat16)
    return t


def make_paged_problem(*, seed: int, batch: int, len_lo: int, len_hi: int, n_q_heads: int, n_kv_heads: int,
                       head_dim: int, page_size: int, seqlen_q: int = 1, pool_factor: float = 1.25,
                       dtype: torch.dtype = torch.float32, outlier_frac: float = 0.0, lengths=None):
    """A pool filled through a seeded random page permutation, plus queries.

    Returns a dict with fp32 master copies: ``k_pool, v_pool [n_pages,H,P,D]`` (already rounded
    to ``dtype``), ``q [B,Sq,Hq,D]``, ``page_table int32 [B, max_pages]`` (unused entries -1),
    ``seqused_k int32 [B]``.  Page 0 is never handed out (the reference reserves it).
    """
    g = torch.Generator().manual_seed(seed)
    if lengths is None:
        lengths = torch.randint(len_lo, len_hi + 1, (batch,), generator=g).tolist()
    pages_per = [-(-L // page_size) for L in lengths]
    total_pages = sum(pages_per)
    n_pages = max(int(total_pages * pool_factor) + 2, total_pages + 2)
    perm = (torch.randperm(n_pages - 1, generator=g) + 1).tolist()
    max_pages = max(pages_per + [1])
    page_table = torch.full((batch, max_pages), -1, dtype=torch.int32)
    cur = 0
    for b, n in enumerate(pages_per):
        page_table[b, :n] = torch.tensor(perm[cur:cur + n], dtype=torch.int32)
        cur += n

    def draw(shape):
        x = torch.randn(shape, generator=g)
        if outlier_frac > 0:
            mask = torch.rand(shape, generator=g) < outlier_frac
            x = torch.where(mask, x * 20.0, x)
        return x

    k_pool = draw((n_pages, n_kv_heads, page_size, head_dim)).to(dtype).float()
    v_pool = draw((n_pages, n_kv_heads, page_size, head_dim)).to(dtype).float()
    q = draw((batch, seqlen_q, n_q_heads, head_dim)).to(dtype).float()
    return {
        "k_pool": k_pool, "v_pool": v_pool, "q": q, "page_table": page_table,
        "seqused_k": torch.tensor(lengths, dtype=torch.int32), "lengths": lengths, "n_pages": n_pages,
    }
