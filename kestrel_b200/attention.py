"""Model-independent paged attention op (mirror of ``kestrel/ops/attention.py:49-89``)."""

from __future__ import annotations

from typing import Any

import torch

from .kernels import flash_attn_fwd


def paged_attention(
    query: torch.Tensor,
    *,
    paged_kv_layer: Any,
    page_table: torch.Tensor,
    paged_kv_seqlens_k: torch.Tensor,
    scaling: float,
    paged_kv_seqlens_q: torch.Tensor | None = None,
    cu_seqlens_q: torch.Tensor | None = None,
    sliding_window: int | None = None,
    shared_prefix_pages: int = 0,
) -> torch.Tensor:
    """Attend ``query [B, H_q, S, D]`` (batched) or packed rows against one paged K/V layer.

    ``paged_kv_layer`` exposes ``k_cache`` / ``v_cache`` ``[n_pages, H_kv, P, D]`` and,
    for FP8 pools, ``k_scale`` / ``v_scale``.  ``paged_kv_seqlens_k`` counts the keys of
    each sequence including the tokens just appended.  Without ``sliding_window`` the
    mask is causal (bottom-right aligned); with it, each query sees the last
    ``sliding_window`` keys up to its own position.  With ``cu_seqlens_q`` the rows of
    all sequences are packed along the first axis and the result is reshaped back to
    ``[B, S, H_q, D]``.  Returns ``[B, S, H_q, D]`` in the query dtype.

    ``shared_prefix_pages`` (not in the reference): leading page-table entries that every row of the
    batch maps to the same full pages; they are then read once for the whole batch (see ``flash_attn_fwd``).
    """
    q = query.transpose(1, 2)
    seqused_q = paged_kv_seqlens_q
    if cu_seqlens_q is not None:
        q = q.flatten(0, 1)
        seqused_q = None
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError(f"paged attention requires fp16/bf16 query, got {q.dtype}")
    windowed = sliding_window is not None
    out, _ = flash_attn_fwd(
        q,
        paged_kv_layer.k_cache.permute(0, 2, 1, 3),
        paged_kv_layer.v_cache.permute(0, 2, 1, 3),
        page_table=page_table,
        cu_seqlens_q=cu_seqlens_q,
        seqused_q=seqused_q,
        seqused_k=paged_kv_seqlens_k,
        paged_kv_non_tma=True,
        causal=not windowed,
        window_size_left=sliding_window - 1 if windowed else None,
        window_size_right=0 if windowed else None,
        softmax_scale=scaling,
        k_scale=getattr(paged_kv_layer, "k_scale", None),
        v_scale=getattr(paged_kv_layer, "v_scale", None),
        max_seqlen_q=query.shape[2] if cu_seqlens_q is not None else None,
        shared_prefix_pages=shared_prefix_pages,
    )
    if cu_seqlens_q is not None:
        out = out.reshape(query.shape[0], query.shape[2], *out.shape[-2:])
    return out


__all__ = ["paged_attention"]
