"""CPU restatement of Kestrel's paged-KV hot path.  TEST INFRASTRUCTURE ONLY.

This module is the checker for the CUDA library, never a product code path:
only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import it.  Nothing under ``kestrel_b200/`` imports it.

What it restates (paths are relative to the m87-labs/kestrel v0.5.0 tree):

* slot mapping            -- ``kestrel/kv_cache.py:524-551`` (``PageTable.build_slot_mapping``)
* append                  -- ``kestrel/kv_cache.py:182-233`` (``PagedKVCache.update``; torch
                             fallback at ``:216-220``; negative slots are skipped as in
                             ``tests/test_kv_pool.py:119-121``)
* metadata builder        -- ``kestrel/kv_cache.py:454-522`` + ``kestrel/models/qwen35/runtime.py:1161-1166``
                             (tail of each output row stays untouched,
                             ``tests/test_page_table.py:48-79``)
* decode attention        -- call contract of ``kestrel/ops/attention.py:49-89`` and
                             ``kestrel/models/moondream/text.py:132-185``
* FP8 e4m3 quantise       -- ``reshape_and_cache_flash(..., "fp8_e4m3", k_scale, v_scale)`` as called
                             at ``kestrel/kv_cache.py:222-231``
* rotary embedding        -- ``rotary_embedding(position_ids, q, k, head_dim, cos_sin_cache)`` as called at
                             ``kestrel/models/moondream/text.py:125`` on the table of
                             ``kestrel/models/moondream/rope.py:6-32``; rotate-half formula of
                             ``kestrel/ops/rotary.py:58-72``
* per-step metadata       -- ``kestrel/models/moondream/runtime.py:2554-2564`` (metadata builder, then
                             ``input_pos.to(long).view(-1, 1)`` and the slot mapping of those positions)
* copy-on-write page copy -- no counterpart in the reference (it forbids prefix caching
                             with page_size > 1, ``kestrel/kv_cache.py:331-335``)

Pinning status.  Slot mapping, append, page-table bookkeeping and the metadata
builder are pinned against the reference's own torch path and its test vectors
(fixtures under ``tests/golden/`` made by ``tests/golden/make_golden.py``).
The arithmetic of attention and of FP8 quantisation lives in the binary wheel
``kestrel-kernels==0.4.9`` whose source is not part of the reference tree, so
for those two this oracle *defines* the semantics from the call sites
(FlashAttention conventions: GQA head ``h`` reads KV head ``h // group``,
bottom-right aligned causal mask, fp32 softmax; FP8 code =
round-to-nearest-even, saturate-to-finite of ``x / scale``): **parity
unpinned** for attention outputs and FP8 codes; the FP8 encoder is
cross-checked against ``torch.float8_e4m3fn``.  The rotary kernel is in the same
wheel: its cos/sin table and the rotate-half formula are pinned (fixtures made
from ``rope.py`` and ``ops/rotary.py``), the rounding of 16-bit rows is defined
here as "fp32 arithmetic with separately rounded products, one rounding to the
row dtype" -- **parity unpinned** for that rounding.
"""

from __future__ import annotations

import math
from typing import Optional, Sequence

import numpy as np
import torch

E4M3_MAX = 448.0


# ----------------------------------------------------------------------------
# FP8 e4m3fn codec (bit level, numpy)
# ----------------------------------------------------------------------------

def fp8_e4m3_encode(x: np.ndarray) -> np.ndarray:
    """fp32 -> e4m3fn code (uint8): round-to-nearest-even, saturate to +-448.

    Equals ``x.clamp(-448, 448).to(torch.float8_e4m3fn).view(uint8)`` for every
    finite input (checked in the tests); NaN maps to 0x7f / 0xff.
    Bit-level algorithm: e4m3fn has 4 exponent bits (bias 7), 3 mantissa bits,
    subnormals with step 2**-9 and no infinities.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32)
    sign = ((bits >> 31) & 1).astype(np.uint8) << 7
    a = np.abs(x).astype(np.float32)
    nan = np.isnan(a)
    a = np.where(nan, np.float32(0), a)
    a = np.minimum(a, np.float32(E4M3_MAX))
    out = np.zeros(a.shape, dtype=np.uint8)

    # Subnormal range of e4m3: |x| < 2**-6, quantum 2**-9.  np.rint rounds half to even.
    sub = a < np.float32(2.0 ** -6)
    q_sub = np.rint(a.astype(np.float64) * 512.0).astype(np.int64)  # 0..8 (8 == smallest normal)
    out = np.where(sub, q_sub.astype(np.uint8), out)

    # Normal range: round the fp32 mantissa (23 bits) to 3 bits, ties to even.
    ab = a.view(np.uint32).astype(np.int64)
    exp = (ab >> 23) - 127  # unbiased
    man = ab & 0x7FFFFF
    keep = man >> 20
    rem = man & 0xFFFFF
    half = 0x80000
    round_up = (rem > half) | ((rem == half) & ((keep & 1) == 1))
    keep = keep + round_up.astype(np.int64)
    carry = keep >> 3
    keep = keep & 7
    exp = exp + carry
    code = ((exp + 7) << 3) | keep
    code = np.minimum(code, 0x7E)  # 0x7e == 448; anything above saturates
    out = np.where(~sub, code.astype(np.uint8), out)
    out = np.where(nan, np.uint8(0x7F), out)
    return (out | sign).astype(np.uint8)


def fp8_e4m3_decode(code: np.ndarray) -> np.ndarray:
    """e4m3fn code (uint8) -> fp32 (exact)."""
    c = np.asarray(code, dtype=np.uint8).astype(np.int32)
    sign = np.where((c & 0x80) != 0, -1.0, 1.0)
    e = (c >> 3) & 0xF
    m = c & 7
    normal = np.ldexp(1.0 + m / 8.0, e - 7)
    subn = np.ldexp(m / 8.0, -6)
    val = np.where(e == 0, subn, normal)
    val = np.where((c & 0x7F) == 0x7F, np.nan, val)
    return (sign * val).astype(np.float32)


def fp8_quantise(x: torch.Tensor, scale) -> torch.Tensor:
    """``x / scale`` (true fp32 division) -> e4m3fn codes as a uint8 tensor.

    ``scale`` is a python float, a 0-dim tensor (the reference's per-layer
    ``k_scale_tensor`` / ``v_scale_tensor``, ``kestrel/kv_cache.py:174-181``) or a
    ``[H_kv]`` vector broadcast over ``x[..., H_kv, D]``.
    """
    xf = x.detach().to(torch.float32).cpu()
    s = torch.as_tensor(scale, dtype=torch.float32).cpu()
    if s.ndim == 1:
        s = s.view(*([1] * (xf.ndim - 2)), -1, 1)
    y = (xf / s).numpy()
    return torch.from_numpy(fp8_e4m3_encode(y))


# ----------------------------------------------------------------------------
# Integer / copy paths
# ----------------------------------------------------------------------------

def build_slot_mapping(page_table: torch.Tensor, batch_idx: torch.Tensor,
                       positions: torch.Tensor, page_size: int) -> torch.Tensor:
    """slot[b, s] = page_table[batch[b, s], pos // P] * P + pos % P  (int64)."""
    pt = page_table.cpu().to(torch.int64)
    pos = positions.cpu().to(torch.int64)
    bi = batch_idx.cpu().to(torch.int64)
    if bi.ndim == 1:
        bi = bi.view(-1, 1).expand_as(pos)
    elif bi.shape != pos.shape:
        raise ValueError("batch_idx and positions shape mismatch")
    phys = pt[bi.reshape(-1), (pos // page_size).reshape(-1)]
    slots = phys * page_size + (pos % page_size).reshape(-1)
    return slots.view_as(pos)


def append(k_cache: torch.Tensor, v_cache: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
           slot_mapping: torch.Tensor, *, k_scale=None, v_scale=None) -> None:
    """Scatter token rows ``k, v [T, H_kv, D]`` into ``[n_pages, H_kv, P, D]`` pools, in place.

    Row ``t`` lands at page ``slot // P``, offset ``slot % P``; rows whose slot
    is negative are skipped.  When the pools are uint8 (FP8 codes) the rows are
    quantised with :func:`fp8_quantise` first.
    """
    page_size = k_cache.shape[2]
    slots = slot_mapping.cpu().to(torch.int64).reshape(-1)
    if slots.numel() != k.shape[0]:
        raise RuntimeError("slot size mismatch")
    quant = k_cache.dtype == torch.uint8
    if quant:
        k_rows = fp8_quantise(k, k_scale)
        v_rows = fp8_quantise(v, v_scale)
    else:
        k_rows = k.detach().cpu().to(k_cache.dtype)
        v_rows = v.detach().cpu().to(v_cache.dtype)
    for t, slot in enumerate(slots.tolist()):
        if slot < 0:
            continue
        page, off = divmod(slot, page_size)
        k_cache[page, :, off, :] = k_rows[t]
        v_cache[page, :, off, :] = v_rows[t]


def build_paged_kv_metadata(page_table: torch.Tensor, batch_idx: torch.Tensor,
                            input_pos: torch.Tensor, out_page_table: torch.Tensor,
                            out_seqused_k: torch.Tensor, page_size: int) -> None:
    """seqused_k[r] = input_pos[r] + 1; copy the live page-table prefix of row batch_idx[r].

    Only ``ceil(seqused_k / P)`` leading entries of each output row are written.
    """
    for r, (b, pos) in enumerate(zip(batch_idx.tolist(), input_pos.tolist())):
        used = int(pos) + 1
        out_seqused_k[r] = used
        n = max(0, -(-used // page_size))
        out_page_table[r, :n] = page_table[int(b), :n]


def copy_pages(caches: Sequence[torch.Tensor], src_pages: Sequence[int],
               dst_pages: Sequence[int]) -> None:
    """Copy-on-write: for every pool ``c`` in ``caches``, ``c[dst] = c[src]`` pair by pair, in order."""
    for c in caches:
        for s, d in zip(src_pages, dst_pages):
            c[int(d)] = c[int(s)].clone()


# ----------------------------------------------------------------------------
# Page gather + attention
# ----------------------------------------------------------------------------

def _as_float(cache: torch.Tensor) -> torch.Tensor:
    if cache.dtype == torch.uint8:
        return torch.from_numpy(fp8_e4m3_decode(cache.cpu().numpy()))
    if cache.dtype == torch.float8_e4m3fn:
        return cache.cpu().to(torch.float32)
    return cache.cpu().to(torch.float32)


def gather_kv(cache: torch.Tensor, pages: torch.Tensor, length: int) -> torch.Tensor:
    """Gather ``length`` tokens of one sequence: ``[n_pages,H,P,D]`` -> ``[length, H, D]``."""
    n_pages_used = -(-length // cache.shape[2])
    sel = cache[pages[:n_pages_used].to(torch.int64)]          # [n, H, P, D]
    tok = sel.permute(0, 2, 1, 3).reshape(-1, cache.shape[1], cache.shape[3])
    return tok[:length]


def _scale_vec(scale, n_heads: int) -> torch.Tensor:
    if scale is None:
        return torch.ones(n_heads, dtype=torch.float32)
    s = torch.as_tensor(scale, dtype=torch.float32).cpu().reshape(-1)
    if s.numel() == 1:
        s = s.expand(n_heads)
    return s.contiguous()


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    page_table: torch.Tensor, seqused_k: torch.Tensor, *,
                    softmax_scale: Optional[float] = None, causal: bool = True,
                    window_left: Optional[int] = None,
                    k_scale=None, v_scale=None,
                    seqused_q: Optional[torch.Tensor] = None,
                    return_lse: bool = False,
                    block_ids: Optional[torch.Tensor] = None):
    """fp32 paged attention.

    ``q [B, Sq, H_q, D]``; pools ``[n_pages, H_kv, P, D]`` (float, or FP8 codes as
    uint8 / float8_e4m3fn, dequantised as ``code * scale``); ``page_table
    [B, >= ceil(L/P)] int32``; ``seqused_k [B]`` counts the keys *including*
    tokens appended this step.  Query row ``j`` of ``Sq_b`` valid rows sees keys
    ``<= L - Sq_b + j`` (bottom-right causal) and, with ``window_left = W``,
    keys ``>= L - Sq_b + j - W``.  Rows ``j >= seqused_q[b]`` and sequences with
    ``L == 0`` give zeros.  Returns fp32 ``[B, Sq, H_q, D]`` (and the natural-log
    LSE ``[B, H_q, Sq]`` when asked).

    ``block_ids [B, >= Sq]`` (int, image-block id >= 0 or -1 per query row) adds the
    block-bidirectional mask of ``kestrel/models/moondream/text.py:139-172``: inside a run of
    equal non-negative ids every row also sees the keys of the run's later rows (the mask
    callable itself lives in the absent wheel; this is its description at the call site and
    in ``kestrel/models/moondream/runtime.py:1671-1679`` -- parity unpinned).
    """
    B, Sq, Hq, D = q.shape
    Hkv = k_cache.shape[1]
    group = Hq // Hkv
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    ks = _scale_vec(k_scale, Hkv)
    vs = _scale_vec(v_scale, Hkv)
    kf = _as_float(k_cache)
    vf = _as_float(v_cache)
    qf = q.detach().cpu().to(torch.float32)
    pt = page_table.cpu()
    out = torch.zeros(B, Sq, Hq, D, dtype=torch.float32)
    lse = torch.full((B, Hq, Sq), float("-inf"), dtype=torch.float32)
    lens = seqused_k.cpu().tolist()
    qlens = seqused_q.cpu().tolist() if seqused_q is not None else [Sq] * B
    for b in range(B):
        L = int(lens[b])
        sq = min(int(qlens[b]), Sq)
        if L <= 0 or sq <= 0:
            continue
        K = gather_kv(kf, pt[b], L) * ks.view(1, -1, 1)       # [L, Hkv, D]
        V = gather_kv(vf, pt[b], L) * vs.view(1, -1, 1)
        K = K.repeat_interleave(group, dim=1)                 # [L, Hq, D]
        V = V.repeat_interleave(group, dim=1)
        s = torch.einsum("shd,lhd->hsl", qf[b, :sq], K) * scale   # [Hq, sq, L]
        key = torch.arange(L).view(1, 1, L)
        row = torch.arange(sq).view(1, sq, 1)
        limit = L - sq + row
        if block_ids is not None:
            ids = block_ids[b, :sq].tolist()
            run_end = list(range(sq))
            for jj in range(sq - 2, -1, -1):
                if ids[jj] >= 0 and ids[jj + 1] == ids[jj]:
                    run_end[jj] = run_end[jj + 1]
            limit = L - sq + torch.tensor(run_end).view(1, sq, 1)
        mask = torch.zeros(1, sq, L, dtype=torch.bool)
        if causal or window_left is not None or block_ids is not None:
            mask |= key > limit
        if window_left is not None:
            mask |= key < (limit - int(window_left))
        s = s.masked_fill(mask, float("-inf"))
        m = s.amax(dim=-1, keepdim=True)
        dead = torch.isinf(m) & (m < 0)
        m = torch.where(dead, torch.zeros_like(m), m)
        p = torch.exp(s - m)
        l = p.sum(dim=-1, keepdim=True)
        o = torch.einsum("hsl,lhd->shd", p / torch.where(l == 0, torch.ones_like(l), l), V)
        out[b, :sq] = o
        lse[b, :, :sq] = torch.where(l == 0, torch.full_like(l, float("-inf")),
                                     m + torch.log(l)).squeeze(-1)
    if return_lse:
        return out, lse
    return out


def decode_step(q, k_new, v_new, k_cache, v_cache, page_table_rows, batch_idx, input_pos,
                *, softmax_scale=None, k_scale=None, v_scale=None):
    """One hot-path step as the reference runs it (``models/moondream/text.py:132-185``):
    slot mapping -> append -> metadata -> attention.  ``input_pos [B, Sq]`` holds the
    positions of the new tokens; returns (out fp32 ``[B,Sq,Hq,D]``, seqused_k)."""
    P = k_cache.shape[2]
    B, Sq = input_pos.shape
    slots = build_slot_mapping(page_table_rows, batch_idx, input_pos, P)
    append(k_cache, v_cache, k_new.reshape(B * Sq, *k_new.shape[-2:]),
           v_new.reshape(B * Sq, *v_new.shape[-2:]), slots, k_scale=k_scale, v_scale=v_scale)
    width = page_table_rows.shape[1]
    compact = torch.full((B, width), -1, dtype=torch.int32)
    seqused = torch.zeros(B, dtype=torch.int32)
    build_paged_kv_metadata(page_table_rows, batch_idx, input_pos[:, -1].to(torch.int32),
                            compact, seqused, P)
    out = paged_attention(q, k_cache, v_cache, compact, seqused, softmax_scale=softmax_scale,
                          k_scale=k_scale, v_scale=v_scale)
    return out, seqused


# ----------------------------------------------------------------------------
# Rotary embedding (NeoX pairing, partial rotary) and the per-step metadata
# ----------------------------------------------------------------------------

def precompute_freqs_cis(dim: int, end: int, theta: float) -> torch.Tensor:
    """fp32 ``[end, dim]`` table: cos of ``dim/2`` frequencies then their sin
    (``kestrel/models/moondream/rope.py:6-32``); ``dim`` is the rotated width."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / float(dim)))
    freqs = torch.arange(end, dtype=torch.float32).unsqueeze(1) * inv_freq.unsqueeze(0)
    return torch.cat([torch.cos(freqs), torch.sin(freqs)], dim=-1)


def rotary_embedding(positions: torch.Tensor, x: torch.Tensor, cos_sin_cache: torch.Tensor) -> torch.Tensor:
    """Rotated copy of ``x [T, H, D]`` (any float dtype) for ``positions [T]``.

    Elements ``i`` and ``i + rot/2`` (``rot = cos_sin_cache.shape[1]``) form a pair,
    ``y1 = x1*cos - x2*sin``, ``y2 = x2*cos + x1*sin`` in fp32 (two rounded products,
    one rounded sum: what ``tensor*cos + rotate_half(tensor)*sin`` of
    ``kestrel/ops/rotary.py:58-72`` evaluates to in fp32), result rounded to ``x.dtype``;
    elements past ``rot`` are unchanged (call site ``kestrel/models/moondream/text.py:125``)."""
    rot = cos_sin_cache.shape[1]
    half = rot // 2
    cs = cos_sin_cache[positions.reshape(-1).long()].float()
    cos, sin = cs[:, None, :half], cs[:, None, half:]
    xf = x.float()
    x1, x2 = xf[..., :half], xf[..., half:rot]
    y1 = x1 * cos - x2 * sin
    y2 = x2 * cos + x1 * sin
    out = xf.clone()
    out[..., :half] = y1
    out[..., half:rot] = y2
    return out.to(x.dtype)


def build_decode_step_metadata(page_table: torch.Tensor, batch_idx: torch.Tensor, input_pos: torch.Tensor,
                               out_page_table: torch.Tensor, out_seqused_k: torch.Tensor, page_size: int,
                               n_new: int = 1) -> tuple[torch.Tensor, torch.Tensor]:
    """The metadata builder followed by the slot mapping of the ``n_new`` positions that end at
    ``input_pos`` (``kestrel/models/moondream/runtime.py:2554-2564``); returns ``(slots, positions)``,
    both int64 ``[B, n_new]``."""
    build_paged_kv_metadata(page_table, batch_idx, input_pos, out_page_table, out_seqused_k, page_size)
    positions = input_pos.to(torch.int64).view(-1, 1) - (n_new - 1) + torch.arange(n_new, dtype=torch.int64).view(1, -1)
    slots = build_slot_mapping(page_table, batch_idx.view(-1), positions, page_size)
    return slots, positions
