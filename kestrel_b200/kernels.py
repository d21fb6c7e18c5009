"""``kestrel_kernels``-compatible runtime object for the paged-KV path.

The reference binds its kernels at import time with
``from kestrel_kernels import get_runtime`` and then calls
``get_runtime().cache.reshape_and_cache_flash``,
``get_runtime().cache.build_paged_kv_metadata`` (``kestrel/kv_cache.py:10-17``) and
``get_runtime().attention.flash_attn_fwd`` (``kestrel/ops/attention.py:69``,
``kestrel/models/moondream/text.py:30-31``).  :func:`get_runtime` returns an
object with exactly those attributes, backed by the sm_100a library through its
C ABI; :func:`install_as_kestrel_kernels` registers this module under the name
``kestrel_kernels`` so the reference's own ``kv_cache.py`` / ``ops/attention.py``
run on it unmodified.

Every function here takes CUDA tensors and enqueues on the current stream of
the tensors' device.  There is no CPU path: CPU tensors raise.
"""

from __future__ import annotations

import ctypes as C
import math
import sys
from typing import Any, Optional, Sequence

import torch

from . import _native

_TORCH_TO_DTYPE = {
    torch.float32: _native.DTYPE_F32,
    torch.float16: _native.DTYPE_F16,
    torch.bfloat16: _native.DTYPE_BF16,
    torch.float8_e4m3fn: _native.DTYPE_E4M3,
    torch.uint8: _native.DTYPE_E4M3,  # the reference passes FP8 pools viewed as uint8
}


def _require_cuda(name: str, t: torch.Tensor) -> int:
    if not isinstance(t, torch.Tensor) or t.device.type != "cuda":
        dev = getattr(t, "device", type(t).__name__)
        raise RuntimeError(
            f"{name} must be a CUDA tensor (got {dev}); the kestrel_b200 kernels have no CPU fallback"
        )
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def _stream(device_index: int) -> int:
    return torch.cuda.current_stream(device_index).cuda_stream


def _cache_view_geometry(name: str, cache: torch.Tensor) -> tuple[int, int, int, int, int, int, int]:
    """(n_pages, page_size, n_heads, head_dim, page_stride, token_stride, head_stride) of a
    ``[n_pages, page_size, n_heads, head_dim]`` cache view."""
    if cache.ndim != 4:
        raise ValueError(f"{name} must have shape [n_pages, page_size, n_heads, head_dim]")
    if cache.stride(3) != 1:
        raise ValueError(f"{name} must be contiguous in head_dim")
    n_pages, page_size, n_heads, head_dim = cache.shape
    return (n_pages, page_size, n_heads, head_dim, cache.stride(0), cache.stride(1), cache.stride(2))


# ---------------------------------------------------------------------------
# cache ops
# ---------------------------------------------------------------------------

def reshape_and_cache_flash(key: torch.Tensor, value: torch.Tensor, key_cache: torch.Tensor,
                            value_cache: torch.Tensor, slot_mapping: torch.Tensor,
                            kv_cache_dtype: str, k_scale: torch.Tensor, v_scale: torch.Tensor) -> None:
    """Append token rows to the paged pools (call shape of ``kestrel/kv_cache.py:222-231``).

    ``key, value [T, H_kv, D]`` (token stride free, heads and D compact);
    ``key_cache, value_cache`` the ``[n_pages, P, H_kv, D]`` views (uint8 or
    float8_e4m3fn when ``kv_cache_dtype`` starts with ``"fp8"``);
    ``slot_mapping int64 [T]``; ``k_scale, v_scale`` fp32 device tensors with 1 or
    ``H_kv`` elements (used only for FP8).  Rows with a negative slot are skipped.
    """
    dev = _require_cuda("key", key)
    for nm, t in (("value", value), ("key_cache", key_cache), ("value_cache", value_cache),
                  ("slot_mapping", slot_mapping)):
        if _require_cuda(nm, t) != dev:
            raise ValueError(f"{nm} lives on a different device than key")
    if key.ndim != 3 or value.ndim != 3 or key.shape != value.shape:
        raise ValueError("key and value must both have shape [num_tokens, n_kv_heads, head_dim]")
    T, H, D = key.shape
    for nm, t in (("key", key), ("value", value)):
        if t.stride(2) != 1 or t.stride(1) != D:
            raise ValueError(f"{nm} must be compact across heads/head_dim; got stride={t.stride()}")
    n_pages, P, Hc, Dc, ps, ts, hs = _cache_view_geometry("key_cache", key_cache)
    if _cache_view_geometry("value_cache", value_cache) != (n_pages, P, Hc, Dc, ps, ts, hs):
        raise ValueError("key_cache and value_cache must have the same shape and strides")
    if (Hc, Dc) != (H, D):
        raise ValueError(f"cache heads/head_dim {(Hc, Dc)} do not match the rows {(H, D)}")
    if slot_mapping.dtype != torch.int64 or slot_mapping.ndim != 1 or not slot_mapping.is_contiguous():
        raise ValueError("slot_mapping must be a contiguous 1-D int64 tensor")
    if slot_mapping.numel() != T:
        raise RuntimeError("slot_mapping size does not match the number of token rows")
    if T == 0:
        return
    quant = str(kv_cache_dtype).startswith("fp8")
    if quant:
        if key_cache.dtype not in (torch.uint8, torch.float8_e4m3fn):
            raise ValueError("fp8 kv_cache_dtype needs uint8 or float8_e4m3fn caches")
        cache_dt = _native.DTYPE_E4M3
        for nm, s in (("k_scale", k_scale), ("v_scale", v_scale)):
            if s is None or s.dtype != torch.float32 or _require_cuda(nm, s) != dev:
                raise ValueError(f"{nm} must be an fp32 tensor on the cache device")
            if s.numel() not in (1, H) or not s.is_contiguous():
                raise ValueError(f"{nm} must hold 1 or n_kv_heads contiguous values")
        if k_scale.numel() != v_scale.numel():
            raise ValueError("k_scale and v_scale must have the same number of elements")
        n_scales = k_scale.numel()
        ks_ptr, vs_ptr = k_scale.data_ptr(), v_scale.data_ptr()
    else:
        if key_cache.dtype != key.dtype:
            raise ValueError(f"cache dtype {key_cache.dtype} does not match row dtype {key.dtype}")
        cache_dt = _TORCH_TO_DTYPE.get(key_cache.dtype)
        if cache_dt is None or key_cache.dtype in (torch.uint8, torch.float8_e4m3fn):
            raise ValueError(f"unsupported cache dtype {key_cache.dtype}")
        n_scales, ks_ptr, vs_ptr = 1, None, None
    in_dt = _TORCH_TO_DTYPE.get(key.dtype)
    if in_dt is None or key.dtype in (torch.uint8, torch.float8_e4m3fn) or value.dtype != key.dtype:
        raise ValueError(f"unsupported row dtype {key.dtype}/{value.dtype}")
    lib = _native.load()
    _native.check(lib.kb200_reshape_and_cache_flash(
        key.data_ptr(), value.data_ptr(), key.stride(0), value.stride(0),
        key_cache.data_ptr(), value_cache.data_ptr(), ps, ts, hs,
        slot_mapping.data_ptr(), T, n_pages, P, H, D, in_dt, cache_dt,
        ks_ptr, vs_ptr, n_scales, dev, _stream(dev)))


def build_slot_mapping(page_table: torch.Tensor, batch_idx: torch.Tensor, positions: torch.Tensor,
                       page_size: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``slots = page_table[batch, pos // P] * P + pos % P`` as int64, shaped like ``positions``
    (one launch for ``kestrel/kv_cache.py:524-551``)."""
    dev = _require_cuda("page_table", page_table)
    if _require_cuda("batch_idx", batch_idx) != dev or _require_cuda("positions", positions) != dev:
        raise ValueError("page_table, batch_idx and positions must live on one device")
    if page_table.dtype != torch.int32 or page_table.ndim != 2 or page_table.stride(1) != 1:
        raise ValueError("page_table must be int32 [rows, pages] contiguous in the last dimension")
    if batch_idx.ndim == 1:
        if positions.ndim != 2 or positions.shape[0] != batch_idx.shape[0]:
            raise ValueError("1-D batch_idx needs positions of shape [batch, seq]")
        per_row, row_len = 1, positions.shape[1]
    else:
        if batch_idx.shape != positions.shape:
            raise ValueError("batch_idx and positions shape mismatch")
        per_row, row_len = 0, 1
    for nm, t in (("batch_idx", batch_idx), ("positions", positions)):
        if t.dtype not in (torch.int32, torch.int64):
            raise ValueError(f"{nm} must be int32 or int64")
    batch_idx = batch_idx.contiguous()
    positions_c = positions.contiguous()
    if out is None:
        out = torch.empty(positions.shape, dtype=torch.int64, device=positions.device)
    elif out.dtype != torch.int64 or out.shape != positions.shape or not out.is_contiguous():
        raise ValueError("out must be a contiguous int64 tensor shaped like positions")
    n = positions_c.numel()
    if n == 0:
        return out
    if per_row and row_len == 0:
        return out
    lib = _native.load()
    _native.check(lib.kb200_build_slot_mapping(
        page_table.data_ptr(), page_table.stride(0), page_table.shape[0], page_table.shape[1],
        batch_idx.data_ptr(), int(batch_idx.dtype == torch.int64), per_row, row_len,
        positions_c.data_ptr(), int(positions_c.dtype == torch.int64), out.data_ptr(), n,
        int(page_size), dev, _stream(dev)))
    return out


def build_paged_kv_metadata(page_table: torch.Tensor, batch_idx: torch.Tensor, input_pos: torch.Tensor,
                            out_page_table: torch.Tensor, out_seqused_k: torch.Tensor,
                            page_size: int) -> None:
    """Decode metadata (call shape of ``kestrel/kv_cache.py:515-522``): ``out_seqused_k = input_pos + 1``
    and the live prefix of each active page-table row copied into ``out_page_table``."""
    dev = _require_cuda("page_table", page_table)
    for nm, t in (("batch_idx", batch_idx), ("input_pos", input_pos), ("out_page_table", out_page_table),
                  ("out_seqused_k", out_seqused_k)):
        if _require_cuda(nm, t) != dev:
            raise ValueError(f"{nm} must live on the page table's device")
    if page_table.dtype != torch.int32 or out_page_table.dtype != torch.int32:
        raise ValueError("page tables must be int32")
    if input_pos.dtype != torch.int32 or out_seqused_k.dtype != torch.int32:
        raise ValueError("input_pos and out_seqused_k must be int32")
    if batch_idx.dtype not in (torch.int32, torch.int64):
        raise ValueError("batch_idx must be int32 or int64")
    if page_table.ndim != 2 or out_page_table.ndim != 2 or page_table.stride(1) != 1 or out_page_table.stride(1) != 1:
        raise ValueError("page tables must be 2-D and contiguous in the last dimension")
    B = batch_idx.shape[0]
    if input_pos.shape[0] != B or out_page_table.shape[0] < B or out_seqused_k.shape[0] < B:
        raise ValueError("metadata buffers are smaller than the batch")
    if B == 0:
        return
    batch_idx = batch_idx.contiguous()
    input_pos = input_pos.contiguous()
    if not out_seqused_k.is_contiguous():
        raise ValueError("out_seqused_k must be contiguous")
    lib = _native.load()
    _native.check(lib.kb200_build_paged_kv_metadata(
        page_table.data_ptr(), page_table.stride(0), page_table.shape[0], page_table.shape[1],
        batch_idx.data_ptr(), int(batch_idx.dtype == torch.int64), input_pos.data_ptr(),
        out_page_table.data_ptr(), out_page_table.stride(0), out_page_table.shape[1],
        out_seqused_k.data_ptr(), B, int(page_size), dev, _stream(dev)))


def build_decode_step_metadata(page_table: torch.Tensor, batch_idx: torch.Tensor, input_pos: torch.Tensor,
                               out_page_table: torch.Tensor, out_seqused_k: torch.Tensor, page_size: int, *,
                               n_new: int = 1, out_slot_mapping: Optional[torch.Tensor] = None,
                               out_positions: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """One launch for the head of a decode step (``kestrel/models/moondream/runtime.py:2554-2564``):
    :func:`build_paged_kv_metadata`, the int64 ``position_ids`` and the slot mapping of the ``n_new``
    tokens per row that end at ``input_pos``.  Returns ``(slot_mapping, position_ids)``, both int64
    ``[B, n_new]`` (written into ``out_slot_mapping`` / ``out_positions`` when given)."""
    dev = _require_cuda("page_table", page_table)
    for nm, t in (("batch_idx", batch_idx), ("input_pos", input_pos), ("out_page_table", out_page_table),
                  ("out_seqused_k", out_seqused_k)):
        if _require_cuda(nm, t) != dev:
            raise ValueError(f"{nm} must live on the page table's device")
    if page_table.dtype != torch.int32 or out_page_table.dtype != torch.int32:
        raise ValueError("page tables must be int32")
    if input_pos.dtype != torch.int32 or out_seqused_k.dtype != torch.int32:
        raise ValueError("input_pos and out_seqused_k must be int32")
    if batch_idx.dtype not in (torch.int32, torch.int64) or batch_idx.ndim != 1 or input_pos.ndim != 1:
        raise ValueError("batch_idx must be 1-D int32/int64 and input_pos 1-D")
    if page_table.ndim != 2 or out_page_table.ndim != 2 or page_table.stride(1) != 1 or out_page_table.stride(1) != 1:
        raise ValueError("page tables must be 2-D and contiguous in the last dimension")
    B = batch_idx.shape[0]
    n_new = int(n_new)
    if n_new < 1:
        raise ValueError("n_new must be at least 1")
    if input_pos.shape[0] != B or out_page_table.shape[0] < B or out_seqused_k.shape[0] < B:
        raise ValueError("metadata buffers are smaller than the batch")
    if not out_seqused_k.is_contiguous():
        raise ValueError("out_seqused_k must be contiguous")
    outs = []
    for nm, t in (("out_slot_mapping", out_slot_mapping), ("out_positions", out_positions)):
        if t is None:
            t = torch.empty((B, n_new), dtype=torch.int64, device=page_table.device)
        elif (t.dtype != torch.int64 or t.shape != (B, n_new) or not t.is_contiguous()
              or _require_cuda(nm, t) != dev):
            raise ValueError(f"{nm} must be a contiguous int64 [batch, n_new] tensor on the page table's device")
        outs.append(t)
    slots, positions = outs
    if B == 0:
        return slots, positions
    batch_idx = batch_idx.contiguous()
    input_pos = input_pos.contiguous()
    lib = _native.load()
    _native.check(lib.kb200_build_decode_step_metadata(
        page_table.data_ptr(), page_table.stride(0), page_table.shape[0], page_table.shape[1],
        batch_idx.data_ptr(), int(batch_idx.dtype == torch.int64), input_pos.data_ptr(),
        out_page_table.data_ptr(), out_page_table.stride(0), out_page_table.shape[1],
        out_seqused_k.data_ptr(), slots.data_ptr(), positions.data_ptr(), B, n_new, int(page_size),
        dev, _stream(dev)))
    return slots, positions


def _token_rows(name: str, t: torch.Tensor) -> tuple[torch.Tensor, int, int, int]:
    """``[T, H, D]`` view of ``t`` (``[T, H, D]`` or ``[B, S, H, D]``) without copying; heads and
    head_dim must be compact, the token stride is free (slices of a fused projection)."""
    if t.ndim == 4:
        B, S, H, D = t.shape
        sb, ss, sh, sd = t.stride()
        if sd != 1 or sh != D:
            raise ValueError(f"{name} must be compact across heads/head_dim; got stride={t.stride()}")
        if B == 1:
            t = t[0]
        elif S == 1:
            t = t[:, 0]
        elif sb == S * ss:
            t = t.as_strided((B * S, H, D), (ss, sh, sd), t.storage_offset())
        else:
            raise ValueError(f"{name} cannot be viewed as token rows; got shape={tuple(t.shape)} stride={t.stride()}")
    if t.ndim != 3:
        raise ValueError(f"{name} must have shape [tokens, heads, head_dim] or [batch, seq, heads, head_dim]")
    T, H, D = t.shape
    if t.stride(2) != 1 or t.stride(1) != D:
        raise ValueError(f"{name} must be compact across heads/head_dim; got stride={t.stride()}")
    return t, T, H, D


def rope_reshape_and_cache(positions: torch.Tensor, q: Optional[torch.Tensor], k: torch.Tensor,
                           v: Optional[torch.Tensor], cos_sin_cache: torch.Tensor,
                           key_cache: Optional[torch.Tensor] = None, value_cache: Optional[torch.Tensor] = None,
                           slot_mapping: Optional[torch.Tensor] = None, kv_cache_dtype: str = "auto",
                           k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None, *,
                           write_k: bool = True) -> None:
    """Rotary embedding of ``q`` and ``k`` in place and, when the pools are given, the append of
    rotated ``k`` plus ``v`` in the same launch -- ``rotary_embedding`` followed by
    ``PagedKVCache.update`` (``kestrel/models/moondream/text.py:125`` and ``:132``).

    ``positions`` int32/int64 with one entry per token row; ``q``/``k``/``v`` ``[T, H, D]`` or
    ``[B, S, H, D]`` views (``q`` may be ``None``); ``cos_sin_cache`` fp32 ``[max_pos, rot_dim]`` in the
    layout of ``kestrel/models/moondream/rope.py:6-32``.  Pool arguments as
    :func:`reshape_and_cache_flash`; with ``write_k=False`` the rotated K only goes to the pool.
    The pool contents are bit-identical to the two separate calls.
    """
    dev = _require_cuda("k", k)
    k_rows, T, Hkv, D = _token_rows("k", k)
    Hq = 0
    q_rows = None
    if q is not None:
        if _require_cuda("q", q) != dev or q.dtype != k.dtype:
            raise ValueError("q must live on k's device and share its dtype")
        q_rows, Tq, Hq, Dq = _token_rows("q", q)
        if (Tq, Dq) != (T, D):
            raise ValueError("q and k disagree on token count or head_dim")
    in_dt = _TORCH_TO_DTYPE.get(k.dtype)
    if in_dt is None or k.dtype in (torch.uint8, torch.float8_e4m3fn):
        raise ValueError(f"unsupported row dtype {k.dtype}")
    if _require_cuda("positions", positions) != dev or positions.dtype not in (torch.int32, torch.int64):
        raise ValueError("positions must be an int32/int64 tensor on k's device")
    if positions.numel() != T:
        raise ValueError("positions must hold one entry per token row")
    positions = positions.contiguous()
    if (_require_cuda("cos_sin_cache", cos_sin_cache) != dev or cos_sin_cache.dtype != torch.float32
            or cos_sin_cache.ndim != 2 or cos_sin_cache.stride(1) != 1):
        raise ValueError("cos_sin_cache must be an fp32 [max_pos, rot_dim] tensor on k's device")
    max_pos, rot = cos_sin_cache.shape
    if rot % 2 or rot > D or rot <= 0:
        raise ValueError(f"rot_dim {rot} must be even and at most head_dim {D}")
    append = key_cache is not None
    ptrs = dict(kc=None, vc=None, slots=None, ks=None, vs=None)
    ps = ts = hs = 0
    n_pages, P, n_scales = 0, 1, 1
    cache_dt = in_dt
    v_rows = None
    if append:
        if v is None or value_cache is None or slot_mapping is None:
            raise ValueError("the fused append needs v, value_cache and slot_mapping")
        if _require_cuda("v", v) != dev or v.dtype != k.dtype:
            raise ValueError("v must live on k's device and share its dtype")
        v_rows, Tv, Hv, Dv = _token_rows("v", v)
        if (Tv, Hv, Dv) != (T, Hkv, D):
            raise ValueError("k and v must have the same shape")
        n_pages, P, Hc, Dc, ps, ts, hs = _cache_view_geometry("key_cache", key_cache)
        if _cache_view_geometry("value_cache", value_cache) != (n_pages, P, Hc, Dc, ps, ts, hs):
            raise ValueError("key_cache and value_cache must have the same shape and strides")
        if (Hc, Dc) != (Hkv, D):
            raise ValueError(f"cache heads/head_dim {(Hc, Dc)} do not match the rows {(Hkv, D)}")
        for nm, t in (("key_cache", key_cache), ("value_cache", value_cache), ("slot_mapping", slot_mapping)):
            if _require_cuda(nm, t) != dev:
                raise ValueError(f"{nm} lives on a different device than k")
        if slot_mapping.dtype != torch.int64 or not slot_mapping.is_contiguous() or slot_mapping.numel() != T:
            raise ValueError("slot_mapping must be a contiguous int64 tensor with one entry per token row")
        if str(kv_cache_dtype).startswith("fp8"):
            if key_cache.dtype not in (torch.uint8, torch.float8_e4m3fn):
                raise ValueError("fp8 kv_cache_dtype needs uint8 or float8_e4m3fn caches")
            cache_dt = _native.DTYPE_E4M3
            for nm, s in (("k_scale", k_scale), ("v_scale", v_scale)):
                if s is None or s.dtype != torch.float32 or _require_cuda(nm, s) != dev:
                    raise ValueError(f"{nm} must be an fp32 tensor on the cache device")
                if s.numel() not in (1, Hkv) or not s.is_contiguous():
                    raise ValueError(f"{nm} must hold 1 or n_kv_heads contiguous values")
            if k_scale.numel() != v_scale.numel():
                raise ValueError("k_scale and v_scale must have the same number of elements")
            n_scales = k_scale.numel()
            ptrs["ks"], ptrs["vs"] = k_scale.data_ptr(), v_scale.data_ptr()
        elif key_cache.dtype != k.dtype:
            raise ValueError(f"cache dtype {key_cache.dtype} does not match row dtype {k.dtype}")
        ptrs["kc"], ptrs["vc"], ptrs["slots"] = key_cache.data_ptr(), value_cache.data_ptr(), slot_mapping.data_ptr()
    if T == 0:
        return
    lib = _native.load()
    _native.check(lib.kb200_rope_append(
        q_rows.data_ptr() if q_rows is not None else None, k_rows.data_ptr(),
        v_rows.data_ptr() if v_rows is not None else None,
        q_rows.stride(0) if q_rows is not None else 0, k_rows.stride(0),
        v_rows.stride(0) if v_rows is not None else 0, T, Hq, Hkv, D, rot,
        positions.data_ptr(), int(positions.dtype == torch.int64),
        cos_sin_cache.data_ptr(), max_pos, cos_sin_cache.stride(0),
        ptrs["kc"], ptrs["vc"], ps, ts, hs, ptrs["slots"], n_pages, P, in_dt, cache_dt,
        ptrs["ks"], ptrs["vs"], n_scales, 1 if write_k else 0, dev, _stream(dev)))


def rotary_embedding(position_ids: torch.Tensor, q: torch.Tensor, k: torch.Tensor, head_dim: int,
                     cos_sin_cache: torch.Tensor) -> None:
    """In-place rotary embedding of ``q`` and ``k`` (``[B, S, H, D]``) with the call shape of
    ``kestrel_kernels``' ``rotary.rotary_embedding`` (``kestrel/models/moondream/text.py:34,125``)."""
    if q.shape[-1] != head_dim or k.shape[-1] != head_dim:
        raise ValueError("head_dim does not match q/k")
    rope_reshape_and_cache(position_ids, q, k, None, cos_sin_cache)


def copy_pages(caches: Sequence[torch.Tensor], src_pages, dst_pages) -> None:
    """Copy-on-write: copy physical page ``src_pages[i]`` onto ``dst_pages[i]`` in every pool of
    ``caches`` (each ``[n_pages, ...]`` with contiguous pages; all the same geometry) in one launch.

    ``src_pages`` / ``dst_pages`` are int sequences or int32 device tensors; destinations
    must be distinct and disjoint from the sources.  The reference has no such op.
    """
    if len(caches) == 0:
        return
    first = caches[0]
    dev = _require_cuda("caches[0]", first)
    page_elems = math.prod(first.shape[1:])
    page_bytes = page_elems * first.element_size()
    stride_bytes = first.stride(0) * first.element_size()
    ptrs = (C.c_void_p * len(caches))()
    for i, c in enumerate(caches):
        if _require_cuda(f"caches[{i}]", c) != dev:
            raise ValueError("all pools must live on one device")
        if c.shape != first.shape or c.stride() != first.stride() or c.dtype != first.dtype:
            raise ValueError("all pools must share shape, strides and dtype")
        if not c[0].is_contiguous():
            raise ValueError("pages of a pool must be contiguous")
        ptrs[i] = c.data_ptr()

    def as_dev(x, nm):
        if isinstance(x, torch.Tensor):
            if x.dtype != torch.int32 or x.ndim != 1 or not x.is_contiguous() or _require_cuda(nm, x) != dev:
                raise ValueError(f"{nm} must be a contiguous 1-D int32 tensor on the pools' device")
            return x
        return torch.tensor(list(x), dtype=torch.int32, device=first.device)

    if not isinstance(src_pages, torch.Tensor) and not isinstance(dst_pages, torch.Tensor):
        s_l, d_l = [int(v) for v in src_pages], [int(v) for v in dst_pages]
        if len(s_l) != len(d_l):
            raise ValueError("src_pages and dst_pages differ in length")
        if len(set(d_l)) != len(d_l) or set(d_l) & set(s_l):
            raise ValueError("destination pages must be distinct and disjoint from the sources")
        n_pages = first.shape[0]
        if any(p < 0 or p >= n_pages for p in s_l + d_l):
            raise ValueError("page index out of range")
        src_pages, dst_pages = s_l, d_l
    src_t, dst_t = as_dev(src_pages, "src_pages"), as_dev(dst_pages, "dst_pages")
    if src_t.numel() != dst_t.numel():
        raise ValueError("src_pages and dst_pages differ in length")
    if src_t.numel() == 0:
        return
    lib = _native.load()
    _native.check(lib.kb200_copy_pages(ptrs, len(caches), page_bytes, stride_bytes, first.shape[0],
                                       src_t.data_ptr(), dst_t.data_ptr(), src_t.numel(), dev, _stream(dev)))


# ---------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------

class _BlockBidirectionalMask:
    """Stand-in for the ``mask_mod`` callable the reference takes from
    ``get_runtime().attention.block_bidirectional_mask`` (``kestrel/models/moondream/text.py:32``) and passes
    to ``flash_attn_fwd`` together with ``aux_tensors=[block_sequence_ids]`` for prompts with images: inside an
    image block (a run of equal ids >= 0) attention is bidirectional, everything else is causal.  It is only
    ever compared by identity; the mask itself is evaluated inside the prefill kernel."""

    def __repr__(self) -> str:
        return "kestrel_b200.kernels.block_bidirectional_mask"


block_bidirectional_mask = _BlockBidirectionalMask()


def block_visibility(block_ids: torch.Tensor, seqlen: Optional[int] = None,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[b, j]`` = last position of the run of equal, non-negative ``block_ids`` containing ``j``
    (``j`` itself where the id is negative): how far past itself query ``j`` sees under the
    block-bidirectional mask.  ``block_ids`` int32 ``[B, >= seqlen]`` on the GPU."""
    dev = _require_cuda("block_ids", block_ids)
    if block_ids.dtype != torch.int32 or block_ids.ndim != 2 or block_ids.stride(1) != 1:
        raise ValueError("block_ids must be int32 [batch, seqlen], contiguous in the last dimension")
    B = block_ids.shape[0]
    S = block_ids.shape[1] if seqlen is None else int(seqlen)
    if S > block_ids.shape[1]:
        raise ValueError("block_ids is shorter than the query rows")
    if out is None:
        out = torch.empty((B, S), dtype=torch.int32, device=block_ids.device)
    elif out.dtype != torch.int32 or out.shape != (B, S) or out.stride(1) != 1 or _require_cuda("out", out) != dev:
        raise ValueError("out must be an int32 [batch, seqlen] tensor on block_ids' device")
    if B and S:
        _native.check(_native.load().kb200_block_visibility(block_ids.data_ptr(), block_ids.stride(0), B, S,
                                                            out.data_ptr(), out.stride(0), dev, _stream(dev)))
    return out


_workspaces: dict[tuple[int, int], torch.Tensor] = {}
_retired_workspaces: list[torch.Tensor] = []   # outgrown buffers: a captured graph may still point at them
_ws_bytes_cache: dict[tuple, int] = {}
_WS_BYTES_CACHE_MAX = 1024


def _workspace(dev: int, stream: int, nbytes: int) -> torch.Tensor:
    """Scratch buffer of one (device, stream).  It only ever grows, and a buffer that was handed out
    is never given back to the allocator: a CUDA graph captured earlier keeps its address."""
    key = (dev, stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        # grow geometrically so steady-state decode never reallocates
        size = max(nbytes, 2 * ws.numel() if ws is not None else 0, 1 << 20)
        if ws is not None:
            _retired_workspaces.append(ws)
        ws = torch.empty(size, dtype=torch.uint8, device=torch.device("cuda", dev))
        _workspaces[key] = ws
    return ws


def reserve_attention_workspace(*, batch: int, total_q: int, n_q_heads: int, n_kv_heads: int,
                                head_dim: int, device: torch.device | int | None = None,
                                stream: "torch.cuda.Stream | None" = None, extra_bytes: int = 0) -> int:
    """Pre-size the scratch buffer of ``stream`` (default: the current stream of ``device``) for the
    largest problem that will run there, so that no allocation happens inside the op.  Call it on
    the stream the CUDA graph is captured on, before the capture.  ``extra_bytes`` adds room for
    calls that need more than the split-KV bound (a shared-prefix call's first-pass output, a
    block-mask call's visibility rows).  Returns the byte count reserved."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index if not isinstance(device, int) else device
    if dev is None:
        dev = torch.cuda.current_device()
    n = int(_native.load().kb200_attn_workspace_bytes(batch, total_q, n_q_heads, n_kv_heads, head_dim, dev))
    n += int(extra_bytes)
    _workspace(dev, stream.cuda_stream if stream is not None else _stream(dev), n)
    return n


def flash_attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *,
                   page_table: Optional[torch.Tensor] = None,
                   cu_seqlens_q: Optional[torch.Tensor] = None,
                   cu_seqlens_k: Optional[torch.Tensor] = None,
                   seqused_q: Optional[torch.Tensor] = None,
                   seqused_k: Optional[torch.Tensor] = None,
                   paged_kv_non_tma: bool = False,
                   causal: bool = False,
                   window_size_left: Optional[int] = None,
                   window_size_right: Optional[int] = None,
                   softmax_scale: Optional[float] = None,
                   k_scale: Any = None, v_scale: Any = None,
                   pack_gqa: Optional[bool] = None,
                   mask_mod: Any = None, aux_tensors: Any = None,
                   out: Optional[torch.Tensor] = None,
                   return_lse: bool = False,
                   max_seqlen_q: Optional[int] = None,
                   shared_prefix_pages: int = 0):
    """Paged attention with the call surface the reference uses for ``flash_attn_fwd``
    (``kestrel/ops/attention.py:69-86``, ``kestrel/models/moondream/text.py:158-185``).

    ``q [B, Sq, H_q, D]`` (or ``[total_q, H_q, D]`` with ``cu_seqlens_q``), fp16/bf16;
    ``k, v`` the ``[n_pages, P, H_kv, D]`` pool views (q's dtype, or FP8 e4m3 as
    float8_e4m3fn / uint8); ``page_table int32 [B, >= ceil(L/P)]``; ``seqused_k int32 [B]``.
    ``k_scale`` / ``v_scale``: python floats (as the reference passes) or fp32 device
    tensors with ``H_kv`` entries.  ``paged_kv_non_tma`` and ``pack_gqa`` are accepted and
    ignored (hints to the reference's kernel).  Returns ``(out, lse_or_None)``.

    ``mask_mod=block_bidirectional_mask`` with ``aux_tensors=[block_sequence_ids]`` (int32 ``[B, >= Sq]``, image
    block id or -1 per query position, ``kestrel/models/moondream/text.py:139-172``) adds bidirectional attention
    inside each image block to the causal mask (padded layout).

    ``shared_prefix_pages=n`` (extension): the caller promises that the first ``n`` page-table entries of every
    row are the same full pages (requests attached to one cached prefix, see ``PageTable.common_prefix_pages``)
    and that every query row sees all of their keys; the prefix is then read once for the whole batch.

    Not implemented (raise ``NotImplementedError``): dense K/V (``page_table=None``),
    ``cu_seqlens_k``, any other ``mask_mod``, a non-zero right window.
    """
    if page_table is None:
        raise NotImplementedError("dense (non-paged) attention is outside the paged-KV path")
    if cu_seqlens_k is not None:
        raise NotImplementedError("cu_seqlens_k is not supported; pass seqused_k")
    block_ids = None
    if mask_mod is not None or aux_tensors is not None:
        if mask_mod is not block_bidirectional_mask:
            raise NotImplementedError("the only mask_mod supported is attention.block_bidirectional_mask")
        if not aux_tensors or len(aux_tensors) != 1 or not isinstance(aux_tensors[0], torch.Tensor):
            raise ValueError("block_bidirectional_mask needs aux_tensors=[block_sequence_ids]")
        if cu_seqlens_q is not None:
            raise NotImplementedError("block_bidirectional_mask with packed rows (cu_seqlens_q) is not supported")
        if window_size_left is not None and window_size_left >= 0:
            raise NotImplementedError("block_bidirectional_mask cannot be combined with a sliding window")
        block_ids = aux_tensors[0]
    if seqused_k is None:
        raise ValueError("paged attention requires seqused_k")
    if window_size_right not in (None, 0, -1):
        raise NotImplementedError("only window_size_right in (None, 0) is supported")
    if window_size_left is not None and window_size_left >= 0 and not causal and window_size_right != 0:
        # FlashAttention reads (left >= 0, right < 0, causal=False) as "unbounded to the right"
        raise NotImplementedError("a left window needs window_size_right=0 (as the reference passes) or causal=True")
    dev = _require_cuda("q", q)
    for nm, t in (("k", k), ("v", v), ("page_table", page_table), ("seqused_k", seqused_k)):
        if _require_cuda(nm, t) != dev:
            raise ValueError(f"{nm} must live on q's device")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError(f"paged attention requires fp16/bf16 query, got {q.dtype}")
    packed = cu_seqlens_q is not None
    if packed:
        if q.ndim != 3:
            raise ValueError("with cu_seqlens_q, q must have shape [total_q, n_heads, head_dim]")
        total_q, Hq, D = q.shape
        B = cu_seqlens_q.shape[0] - 1
        if cu_seqlens_q.dtype != torch.int32 or not cu_seqlens_q.is_contiguous() or _require_cuda("cu_seqlens_q", cu_seqlens_q) != dev:
            raise ValueError("cu_seqlens_q must be a contiguous int32 tensor on q's device")
        Sq = int(max_seqlen_q) if max_seqlen_q is not None else total_q
        q_strides = (0, q.stride(0), q.stride(1))
    else:
        if q.ndim != 4:
            raise ValueError("q must have shape [batch, seqlen_q, n_heads, head_dim]")
        B, Sq, Hq, D = q.shape
        total_q = B * Sq
        q_strides = (q.stride(0), q.stride(1), q.stride(2))
    if q.stride(-1) != 1:
        raise ValueError("q must be contiguous in head_dim")
    n_pages, P, Hkv, Dk, ps, ts, hs = _cache_view_geometry("k", k)
    if _cache_view_geometry("v", v) != (n_pages, P, Hkv, Dk, ps, ts, hs):
        raise ValueError("k and v must have the same shape and strides")
    if Dk != D:
        raise ValueError(f"head_dim mismatch: q has {D}, K/V have {Dk}")
    if k.dtype != v.dtype:
        raise ValueError("k and v must share a dtype")
    fp8 = k.dtype in (torch.float8_e4m3fn, torch.uint8)
    if not fp8 and k.dtype != q.dtype:
        raise ValueError(f"K/V dtype {k.dtype} must equal the query dtype {q.dtype} or be FP8 e4m3")
    if page_table.dtype != torch.int32 or page_table.ndim != 2 or page_table.stride(1) != 1:
        raise ValueError("page_table must be int32 [batch, pages], contiguous in the last dimension")
    if page_table.shape[0] < B:
        raise ValueError("page_table has fewer rows than the batch")
    if seqused_k.dtype != torch.int32 or seqused_k.ndim != 1 or seqused_k.shape[0] < B or not seqused_k.is_contiguous():
        raise ValueError("seqused_k must be a contiguous int32 tensor with one entry per sequence")
    if seqused_q is not None:
        if packed:
            raise ValueError("seqused_q cannot be combined with cu_seqlens_q")
        if seqused_q.dtype != torch.int32 or seqused_q.shape[0] < B or not seqused_q.is_contiguous() or _require_cuda("seqused_q", seqused_q) != dev:
            raise ValueError("seqused_q must be a contiguous int32 tensor on q's device")
    if out is None:
        out = torch.empty_like(q)
    elif out.shape != q.shape or out.dtype != q.dtype or out.stride(-1) != 1 or _require_cuda("out", out) != dev:
        raise ValueError("out must match q in shape, dtype and device")
    lse = None
    if return_lse:
        lse = torch.empty((Hq, total_q) if packed else (B, Hq, Sq), dtype=torch.float32, device=q.device)
    if B == 0 or total_q == 0:
        return out, lse
    o_strides = (0, out.stride(0), out.stride(1)) if packed else (out.stride(0), out.stride(1), out.stride(2))

    ks_f = vs_f = 1.0
    ks_ptr = vs_ptr = None
    if fp8:
        def scale_arg(s, nm):
            if s is None:
                return 1.0, None
            if isinstance(s, torch.Tensor):
                if s.numel() == 1 and s.device.type != "cuda":
                    return float(s), None
                if s.dtype != torch.float32 or not s.is_contiguous() or _require_cuda(nm, s) != dev or s.numel() != Hkv:
                    raise ValueError(f"{nm} tensor must be contiguous fp32 with n_kv_heads entries on q's device")
                return 1.0, s.data_ptr()
            return float(s), None
        ks_f, ks_ptr = scale_arg(k_scale, "k_scale")
        vs_f, vs_ptr = scale_arg(v_scale, "v_scale")

    stream = _stream(dev)
    lib = _native.load()

    a = _native.AttnArgs()
    a.struct_bytes = C.sizeof(_native.AttnArgs)
    a.device = dev
    a.stream = stream
    a.q = q.data_ptr()
    a.out = out.data_ptr()
    a.lse = lse.data_ptr() if lse is not None else None
    a.q_batch_stride, a.q_row_stride, a.q_head_stride = q_strides
    a.o_batch_stride, a.o_row_stride, a.o_head_stride = o_strides
    a.k_cache = k.data_ptr()
    a.v_cache = v.data_ptr()
    a.kv_page_stride, a.kv_token_stride, a.kv_head_stride = ps, ts, hs
    a.n_pages = n_pages
    a.page_table = page_table.data_ptr()
    a.pt_row_stride = page_table.stride(0)
    a.seqused_k = seqused_k.data_ptr()
    a.seqused_q = seqused_q.data_ptr() if seqused_q is not None else None
    a.cu_seqlens_q = cu_seqlens_q.data_ptr() if packed else None
    a.batch = B
    a.total_q = total_q
    a.seqlen_q = Sq
    a.n_q_heads, a.n_kv_heads, a.head_dim, a.page_size = Hq, Hkv, D, P
    a.q_dtype = _TORCH_TO_DTYPE[q.dtype]
    a.kv_dtype = _native.DTYPE_E4M3 if fp8 else _TORCH_TO_DTYPE[k.dtype]
    a.softmax_scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    a.causal = 1 if causal else 0
    a.window_left = int(window_size_left) if window_size_left is not None and window_size_left >= 0 else -1
    a.k_scale, a.v_scale = ks_f, vs_f
    a.k_scale_per_head, a.v_scale_per_head = ks_ptr, vs_ptr
    if block_ids is not None:
        if _require_cuda("block_sequence_ids", block_ids) != dev or block_ids.ndim != 2 or block_ids.shape[0] < B:
            raise ValueError("block_sequence_ids must be an int32 [batch, >= seqlen_q] tensor on q's device")
        a.causal = 1   # the block mask extends the causal one (the reference passes causal=False next to mask_mod)
    if shared_prefix_pages:
        if shared_prefix_pages < 0 or shared_prefix_pages > page_table.shape[1]:
            raise ValueError("shared_prefix_pages must lie in [0, page_table.shape[1]]")
        a.shared_prefix_pages = int(shared_prefix_pages)
    # scratch: sized for this very call (prefill-shaped calls need only the plan arrays)
    wkey = (B, total_q, Sq, Hq, Hkv, D, a.kv_dtype, block_ids is not None, dev, int(shared_prefix_pages),
            q_strides, seqused_q is None, a.window_left)
    nbytes = _ws_bytes_cache.get(wkey)
    if nbytes is None:
        if block_ids is not None:
            a.q_visible_until = q.data_ptr()   # any non-null value: it selects the kernel the size depends on
        nbytes = int(lib.kb200_attn_workspace_bytes_for(C.byref(a)))
        if len(_ws_bytes_cache) >= _WS_BYTES_CACHE_MAX:
            _ws_bytes_cache.clear()
        _ws_bytes_cache[wkey] = nbytes = (nbytes + 255) & ~255
    vis_bytes = ((B * Sq * 4 + 255) & ~255) if block_ids is not None else 0
    ws = _workspace(dev, stream, nbytes + vis_bytes)
    if block_ids is not None:
        # the visibility rows live behind the kernel scratch in the same per-stream buffer
        vis = ws[nbytes:nbytes + B * Sq * 4].view(torch.int32).view(B, Sq)
        block_visibility(block_ids[:B], Sq, out=vis)
        a.q_visible_until = vis.data_ptr()
        a.q_visible_batch_stride = vis.stride(0)
    a.workspace = ws.data_ptr()
    a.workspace_bytes = nbytes
    _native.check(lib.kb200_paged_attention(C.byref(a)))
    return out, lse


# ---------------------------------------------------------------------------
# sampling hand-off
# ---------------------------------------------------------------------------

def sample_step_from_logits(logits: torch.Tensor, temperatures: torch.Tensor, top_ps: torch.Tensor, *,
                            out: Optional[torch.Tensor] = None, generator: Optional[torch.Generator] = None,
                            logprobs_out: Optional[torch.Tensor] = None,
                            uniforms: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of ``logits [B, V]`` (fp32/fp16/bf16): temperature, top-p nucleus, one draw -- the call
    the scheduler makes after the decoder stack (``kestrel/scheduler/scheduler.py:2986-2991``,
    ``kestrel/scheduler/spatial.py:105-123``).

    ``temperatures`` / ``top_ps`` fp32 ``[B]``; a temperature <= 1e-6 is greedy (arg-max, log-probability 0).
    The row's random number comes from ``generator`` (one ``torch.rand`` of ``B`` values on the logits' device)
    unless ``uniforms`` (fp32 ``[B]`` in [0, 1)) is given, which makes the call deterministic and allocation-free.
    Returns ``out`` (int64 ``[B]``, allocated when absent); ``logprobs_out`` (fp32 ``[B]``) receives
    ``logits[id] / T - logsumexp(logits / T)``.
    """
    dev = _require_cuda("logits", logits)
    if logits.ndim != 2 or logits.stride(1) != 1:
        raise ValueError("logits must have shape [batch, vocab], contiguous in the vocabulary")
    dt = _TORCH_TO_DTYPE.get(logits.dtype)
    if dt is None or logits.dtype in (torch.uint8, torch.float8_e4m3fn):
        raise ValueError(f"unsupported logits dtype {logits.dtype}")
    B, V = logits.shape
    for nm, t in (("temperatures", temperatures), ("top_ps", top_ps)):
        if _require_cuda(nm, t) != dev or t.dtype != torch.float32 or t.ndim != 1 or t.shape[0] < B or not t.is_contiguous():
            raise ValueError(f"{nm} must be a contiguous fp32 [batch] tensor on the logits' device")
    if out is None:
        out = torch.empty(B, dtype=torch.int64, device=logits.device)
    elif _require_cuda("out", out) != dev or out.dtype != torch.int64 or out.ndim != 1 or out.shape[0] < B or not out.is_contiguous():
        raise ValueError("out must be a contiguous int64 [batch] tensor on the logits' device")
    if logprobs_out is not None and (_require_cuda("logprobs_out", logprobs_out) != dev or logprobs_out.dtype != torch.float32
                                     or logprobs_out.ndim != 1 or logprobs_out.shape[0] < B or not logprobs_out.is_contiguous()):
        raise ValueError("logprobs_out must be a contiguous fp32 [batch] tensor on the logits' device")
    if uniforms is None:
        uniforms = torch.rand(B, generator=generator, device=logits.device, dtype=torch.float32)
    elif _require_cuda("uniforms", uniforms) != dev or uniforms.dtype != torch.float32 or uniforms.shape[0] < B or not uniforms.is_contiguous():
        raise ValueError("uniforms must be a contiguous fp32 [batch] tensor on the logits' device")
    if B == 0:
        return out
    _native.check(_native.load().kb200_sample_step_from_logits(
        logits.data_ptr(), dt, B, V, logits.stride(0), temperatures.data_ptr(), top_ps.data_ptr(), uniforms.data_ptr(),
        out.data_ptr(), logprobs_out.data_ptr() if logprobs_out is not None else None, dev, _stream(dev)))
    return out


# ---------------------------------------------------------------------------
# runtime object
# ---------------------------------------------------------------------------

class _Unavailable:
    """Namespace whose every attribute raises: kernels outside the paged-KV path."""

    def __init__(self, name: str) -> None:
        self._name = name

    def __getattr__(self, item: str):
        raise NotImplementedError(
            f"kestrel_kernels.{self._name}.{item} is outside the paged-KV path this library implements"
        )


class _CacheOps:
    reshape_and_cache_flash = staticmethod(reshape_and_cache_flash)
    build_paged_kv_metadata = staticmethod(build_paged_kv_metadata)
    build_slot_mapping = staticmethod(build_slot_mapping)
    build_decode_step_metadata = staticmethod(build_decode_step_metadata)
    rope_reshape_and_cache = staticmethod(rope_reshape_and_cache)
    copy_pages = staticmethod(copy_pages)


class _RotaryOps:
    rotary_embedding = staticmethod(rotary_embedding)

    def __getattr__(self, item: str):
        raise NotImplementedError(f"kestrel_kernels.rotary.{item} is outside the paged-KV path")


class _AttentionOps:
    flash_attn_fwd = staticmethod(flash_attn_fwd)
    block_bidirectional_mask = block_bidirectional_mask

    def __getattr__(self, item: str):
        raise NotImplementedError(f"kestrel_kernels.attention.{item} is outside the paged-KV path")


class _SamplingOps:
    sample_step_from_logits = staticmethod(sample_step_from_logits)

    def __getattr__(self, item: str):
        raise NotImplementedError(f"kestrel_kernels.sampling.{item} is outside the paged-KV path")


class Runtime:
    """What ``kestrel_kernels.get_runtime()`` returns, restricted to the paged-KV path."""

    def __init__(self) -> None:
        self.cache = _CacheOps()
        self.attention = _AttentionOps()
        self.rotary = _RotaryOps()
        self.sampling = _SamplingOps()
        for name in ("linear", "vision", "dense", "tau", "moe", "gated_delta",
                     "megakernel", "generated_decode", "linear_ops"):
            setattr(self, name, _Unavailable(name))


_RUNTIME: Optional[Runtime] = None


def get_runtime() -> Runtime:
    """Load the native library (raising if it is missing) and return the runtime object."""
    global _RUNTIME
    if _RUNTIME is None:
        _native.load()
        _RUNTIME = Runtime()
    return _RUNTIME


def install_as_kestrel_kernels() -> None:
    """Register this module as ``kestrel_kernels`` so Kestrel's own modules bind to it, and
    ``kestrel_kernels.sampling`` for the scheduler's ``from kestrel_kernels.sampling import
    sample_step_from_logits`` (``kestrel/scheduler/scheduler.py:47``)."""
    import types

    me = sys.modules[__name__]
    sys.modules["kestrel_kernels"] = me
    sampling = types.ModuleType("kestrel_kernels.sampling")
    sampling.sample_step_from_logits = sample_step_from_logits
    sys.modules["kestrel_kernels.sampling"] = sampling
    me.sampling = sampling
