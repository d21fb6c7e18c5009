"""Paged attention op with the call surface of ``paged_attention`` in ``kestrel/ops/attention.py:49-89``,
plus the ``shared_prefix_pages`` hint.

A Kestrel installation keeps its own ``kestrel/ops/attention.py`` and reaches this library through
``install_as_kestrel_kernels()``; this module serves callers that use the library without Kestrel (the
benchmark, the tests) and the one extension the reference's function has no argument for.
"""

from __future__ import annotations

from typing import Any, Optional

import torch

from .kernels import flash_attn_fwd

_QUERY_DTYPES = (torch.float16, torch.bfloat16)


def paged_attention(query: torch.Tensor, *, paged_kv_layer: Any, page_table: torch.Tensor,
                    paged_kv_seqlens_k: torch.Tensor, scaling: float,
                    paged_kv_seqlens_q: Optional[torch.Tensor] = None,
                    cu_seqlens_q: Optional[torch.Tensor] = None,
                    sliding_window: Optional[int] = None,
                    shared_prefix_pages: int = 0) -> torch.Tensor:
    """``query [B, H_q, S, D]`` against one paged K/V layer; returns ``[B, S, H_q, D]`` in the query dtype.

    ``paged_kv_layer``: ``k_cache`` / ``v_cache`` ``[n_pages, H_kv, P, D]`` and, for FP8 pools, ``k_scale`` /
    ``v_scale``.  ``paged_kv_seqlens_k`` counts each sequence's keys including the tokens just appended.
    Mask: causal, bottom-right aligned; with ``sliding_window = W`` each query sees the last ``W`` keys up to
    its own position.  ``paged_kv_seqlens_q`` limits the valid query rows per sequence (padded layout);
    with ``cu_seqlens_q`` the ``B * S`` rows are handed over packed instead.

    ``shared_prefix_pages`` (not in the reference): leading page-table entries that every row of the batch
    maps to the same full pages; they are read once for the whole batch (see ``flash_attn_fwd``).
    """
    n_seq, n_heads, n_rows, head_dim = query.shape
    if query.dtype not in _QUERY_DTYPES:
        raise RuntimeError(f"paged attention requires fp16/bf16 query, got {query.dtype}")
    rows = query.permute(0, 2, 1, 3)                       # [B, S, H_q, D], a view
    packed = cu_seqlens_q is not None
    mask = (dict(causal=True, window_size_left=None, window_size_right=None) if sliding_window is None
            else dict(causal=False, window_size_left=sliding_window - 1, window_size_right=0))
    pools = [getattr(paged_kv_layer, name).permute(0, 2, 1, 3) for name in ("k_cache", "v_cache")]
    out, _lse = flash_attn_fwd(
        rows.reshape(n_seq * n_rows, n_heads, head_dim) if packed else rows, *pools,
        page_table=page_table, seqused_k=paged_kv_seqlens_k,
        seqused_q=None if packed else paged_kv_seqlens_q,
        cu_seqlens_q=cu_seqlens_q, max_seqlen_q=n_rows if packed else None,
        paged_kv_non_tma=True, softmax_scale=scaling,
        k_scale=getattr(paged_kv_layer, "k_scale", None), v_scale=getattr(paged_kv_layer, "v_scale", None),
        shared_prefix_pages=shared_prefix_pages, **mask)
    return out.view(n_seq, n_rows, n_heads, head_dim) if packed else out


__all__ = ["paged_attention"]
