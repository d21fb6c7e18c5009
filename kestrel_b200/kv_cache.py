"""KV pool, per-layer paged cache and page table: the host side of the paged-KV path.

Mirrors the public surface of the reference's ``kestrel/kv_cache.py`` -- same class
and method names, argument meaning, return values, page/row numbering and error
behaviour -- so the scheduler, runtimes and prefix cache drive it unchanged:

* :class:`KVMemoryPool`   -- ``kestrel/kv_cache.py:52-136``
* :class:`PagedKVCache`   -- ``kestrel/kv_cache.py:139-233``
* :class:`PagedKVLayerSpec`, :func:`allocate_paged_kv_layers` -- ``:236-268``
* :class:`PageTable`      -- ``kestrel/kv_cache.py:271-771``

Differences, all additive:

* device work goes to the sm_100a kernels (no torch index fallback; CPU tensors
  raise in :meth:`PagedKVCache.update`);
* ``build_slot_mapping`` is one kernel launch on CUDA;
* FP8 scales may be per KV head (a sequence of ``n_heads`` floats) as well as per layer;
* copy-on-write of shared pages (:meth:`PageTable.cow_page`, :func:`copy_kv_pages`),
  which the reference lacks because it only allows prefix caching with ``page_size == 1``.
"""

from __future__ import annotations

import contextlib
import threading
import weakref
from dataclasses import dataclass
from typing import Iterable, Optional, Sequence

import numpy as np
import torch

from . import kernels as _k
from .buffers import CpuGpuBuffer


def resolve_device(device: torch.device | str) -> torch.device:
    """``"cuda"`` -> ``cuda:<current>``; everything else as given (``kestrel/device.py:21-36``)."""
    dev = torch.device(device)
    if dev.type == "cuda" and dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    return dev


def _on_stream(stream):
    return contextlib.nullcontext() if stream is None else torch.cuda.stream(stream)


def _flatten_bshd_tokens(name: str, tensor: torch.Tensor) -> torch.Tensor:
    """Zero-copy ``[B, S, H, D] -> [B*S, H, D]`` view; the token stride may exceed ``H*D``
    (K and V are slices of a fused projection).  Same checks and messages as
    ``kestrel/kv_cache.py:24-48``."""
    if tensor.ndim != 4:
        raise ValueError(f"{name} must have shape [batch, seq, heads, head_dim]")
    B, S, H, D = tensor.shape
    sb, ss, sh, sd = tensor.stride()
    if sd != 1 or sh != D:
        raise ValueError(
            f"{name} must be compact across heads/head_dim; "
            f"got shape={tuple(tensor.shape)} stride={tensor.stride()}"
        )
    tok = sb if S == 1 else ss
    if B > 1 and S > 1 and sb != S * tok:
        raise ValueError(
            f"{name} batch/sequence dimensions cannot be flattened without a copy; "
            f"got shape={tuple(tensor.shape)} stride={tensor.stride()}"
        )
    return tensor.as_strided((B * S, H, D), (tok, sh, sd), storage_offset=tensor.storage_offset())


class KVMemoryPool:
    """Accounts for (and optionally caps) the bytes handed out as per-layer K/V buffers.

    ``allocate_layer_kv`` returns zero-filled ``[n_pages, n_heads, page_size, head_dim]``
    K and V tensors and raises :class:`MemoryError` ("budget exceeded") when the cap
    would be passed; bytes return to the pool when the tensors are collected.
    Thread-safe.
    """

    def __init__(self, *, device: torch.device | str, budget_bytes: int | None = None):
        if budget_bytes is not None and budget_bytes < 0:
            raise ValueError(f"budget_bytes must be non-negative, got {budget_bytes}")
        self.device = resolve_device(device)
        self.budget_bytes = budget_bytes
        self.allocated_bytes = 0
        self._lock = threading.Lock()

    def _release_bytes(self, n: int) -> None:
        with self._lock:
            self.allocated_bytes = max(0, self.allocated_bytes - n)

    def allocate_layer_kv(self, *, n_pages: int, n_heads: int, page_size: int, head_dim: int,
                          dtype: torch.dtype) -> tuple[torch.Tensor, torch.Tensor]:
        shape = (n_pages, n_heads, page_size, head_dim)
        one = n_pages * n_heads * page_size * head_dim * torch.empty((), dtype=dtype).element_size()
        both = 2 * one
        with self._lock:
            if self.budget_bytes is not None and self.allocated_bytes + both > self.budget_bytes:
                raise MemoryError(
                    f"KVMemoryPool budget exceeded: requested {both} bytes, already used "
                    f"{self.allocated_bytes} of {self.budget_bytes}"
                )
            self.allocated_bytes += both
        try:
            k = torch.zeros(shape, dtype=dtype, device=self.device)
            v = torch.zeros(shape, dtype=dtype, device=self.device)
        except Exception:
            self._release_bytes(both)
            raise
        weakref.finalize(k, self._release_bytes, one)
        weakref.finalize(v, self._release_bytes, one)
        return k, v


class PagedKVCache(torch.nn.Module):
    """One layer's paged K/V pools plus the append op.

    Buffers ``k_cache``, ``v_cache`` ``[n_pages, n_heads, page_size, head_dim]``;
    ``quantized`` is true for ``torch.float8_e4m3fn`` pools, which need ``k_scale`` /
    ``v_scale`` (``ValueError`` otherwise).  ``k_scale`` / ``v_scale`` stay python floats
    when given as floats (what the reference's attention call reads) and become fp32
    device tensors ``k_scale_tensor`` / ``v_scale_tensor`` for the kernels; a sequence
    of ``n_heads`` floats selects per-head scales, in which case ``k_scale`` /
    ``v_scale`` are the device vectors themselves.
    """

    def __init__(self, page_table, n_heads, head_dim, dtype, pool: KVMemoryPool, *,
                 k_scale=None, v_scale=None):
        super().__init__()
        k_cache, v_cache = pool.allocate_layer_kv(
            n_pages=page_table.n_pages, n_heads=n_heads, page_size=page_table.page_size,
            head_dim=head_dim, dtype=dtype)
        self.register_buffer("k_cache", k_cache)
        self.register_buffer("v_cache", v_cache)
        self.page_table = page_table
        self.quantized = dtype == torch.float8_e4m3fn
        self._kv_cache_dtype = "fp8_e4m3" if self.quantized else "auto"
        per_head = False
        if self.quantized:
            if k_scale is None or v_scale is None:
                raise ValueError("FP8 KV cache requires per-layer k/v scales")
            per_head = not isinstance(k_scale, (int, float)) or not isinstance(v_scale, (int, float))
        else:
            k_scale = v_scale = 1.0
        if per_head:
            ks = torch.as_tensor(k_scale, dtype=torch.float32).reshape(-1)
            vs = torch.as_tensor(v_scale, dtype=torch.float32).reshape(-1)
            if ks.numel() != n_heads or vs.numel() != n_heads:
                raise ValueError("per-head FP8 scales need one value per KV head")
            self.register_buffer("k_scale_tensor", ks.to(pool.device).contiguous())
            self.register_buffer("v_scale_tensor", vs.to(pool.device).contiguous())
            self.k_scale = self.k_scale_tensor
            self.v_scale = self.v_scale_tensor
        else:
            self.k_scale = float(k_scale)
            self.v_scale = float(v_scale)
            self.register_buffer("k_scale_tensor", torch.tensor(self.k_scale, dtype=torch.float32, device=pool.device))
            self.register_buffer("v_scale_tensor", torch.tensor(self.v_scale, dtype=torch.float32, device=pool.device))

    def update(self, input_pos, k_val, v_val, *, slot_mapping: torch.Tensor):
        """Append ``k_val, v_val [B, S, H, D]`` at ``slot_mapping`` (shape of ``input_pos``);
        returns the inputs unchanged, like ``kestrel/kv_cache.py:182-233``."""
        k_rows = _flatten_bshd_tokens("k_val", k_val)
        v_rows = _flatten_bshd_tokens("v_val", v_val)
        if slot_mapping.shape != input_pos.shape:
            raise ValueError("slot_mapping must match input_pos shape")
        slots = slot_mapping.to(device=k_rows.device, dtype=torch.int64)
        if slots.numel() == 0:
            return k_val, v_val
        if slots.numel() != k_rows.shape[0]:
            raise RuntimeError("PagedKVCache.update slot size mismatch")
        slots = slots.contiguous().view(-1)
        _k.reshape_and_cache_flash(
            k_rows, v_rows,
            self.k_cache.permute(0, 2, 1, 3), self.v_cache.permute(0, 2, 1, 3),
            slots, self._kv_cache_dtype, self.k_scale_tensor.view(-1), self.v_scale_tensor.view(-1))
        return k_val, v_val

    def rope_update(self, input_pos, q, k_val, v_val, cos_sin_cache: torch.Tensor, *,
                    slot_mapping: torch.Tensor, write_k: bool = True):
        """Rotary embedding of ``q`` and ``k_val`` at ``input_pos`` followed by :meth:`update`, as
        one kernel launch (``kestrel/models/moondream/text.py:125`` then ``:132``).  ``q`` and
        ``k_val`` are rotated in place; the pools end up bit-identical to the two separate calls.
        Not in the reference."""
        if slot_mapping.shape != input_pos.shape:
            raise ValueError("slot_mapping must match input_pos shape")
        slots = slot_mapping.to(device=k_val.device, dtype=torch.int64).contiguous().view(-1)
        _k.rope_reshape_and_cache(
            input_pos.reshape(-1), q, k_val, v_val, cos_sin_cache,
            self.k_cache.permute(0, 2, 1, 3), self.v_cache.permute(0, 2, 1, 3),
            slots, self._kv_cache_dtype, self.k_scale_tensor.view(-1), self.v_scale_tensor.view(-1),
            write_k=write_k)
        return k_val, v_val


class LayerPagedCache(torch.nn.Module):
    """Adapter that wires a :class:`PagedKVCache` into a text block: the shape checks of
    ``_LayerPagedCache`` (``kestrel/models/moondream/runtime.py:426-481``) in front of ``update``.

    ``pos_ids`` is ``[S]`` or ``[1, S]`` (shared by the batch) or ``[B, S]``; ``k_val`` / ``v_val`` are
    ``[B, S, H_kv, D]``.  ``rope_update`` is the same adapter in front of the fused rotary + append.
    """

    def __init__(self, page_table: "PageTable", n_kv_heads: int, head_dim: int, dtype: torch.dtype,
                 pool: KVMemoryPool, *, k_scale=None, v_scale=None) -> None:
        super().__init__()
        self.cache = PagedKVCache(page_table, n_heads=n_kv_heads, head_dim=head_dim, dtype=dtype, pool=pool,
                                  k_scale=k_scale, v_scale=v_scale)

    @staticmethod
    def _positions(pos_ids: torch.Tensor, k_val: torch.Tensor, v_val: torch.Tensor) -> torch.Tensor:
        if k_val.shape != v_val.shape:
            raise ValueError("k_val and v_val must match shape")
        input_pos = torch.atleast_2d(pos_ids)
        if input_pos.device != k_val.device:
            input_pos = input_pos.to(device=k_val.device)
        if input_pos.shape[0] != 1 and input_pos.shape[0] != k_val.shape[0]:
            raise ValueError(f"Unsupported position shape {pos_ids.shape} for batch size {k_val.shape[0]}")
        if k_val.shape[1] != input_pos.shape[1]:
            raise ValueError(f"KV sequence length {k_val.shape[1]} does not match position tensor {input_pos.shape}")
        return input_pos

    def update(self, pos_ids: torch.Tensor, k_val: torch.Tensor, v_val: torch.Tensor, *, slot_mapping: torch.Tensor):
        input_pos = self._positions(pos_ids, k_val, v_val)
        return self.cache.update(input_pos=input_pos, k_val=k_val, v_val=v_val, slot_mapping=slot_mapping)

    def rope_update(self, pos_ids: torch.Tensor, q: torch.Tensor, k_val: torch.Tensor, v_val: torch.Tensor,
                    cos_sin_cache: torch.Tensor, *, slot_mapping: torch.Tensor, **kwargs):
        input_pos = self._positions(pos_ids, k_val, v_val)
        return self.cache.rope_update(input_pos, q, k_val, v_val, cos_sin_cache, slot_mapping=slot_mapping, **kwargs)


@dataclass(frozen=True, slots=True)
class PagedKVLayerSpec:
    """Physical storage shape for one paged-attention producer layer."""

    n_heads: int
    head_dim: int
    k_scale: float | None = None
    v_scale: float | None = None


def allocate_paged_kv_layers(*, layer_specs: Sequence[PagedKVLayerSpec | None], page_table: "PageTable",
                             pool: KVMemoryPool, dtype: torch.dtype) -> tuple[PagedKVCache | None, ...]:
    """One :class:`PagedKVCache` per non-``None`` spec (layers that share another layer's KV stay ``None``)."""
    layers = []
    for spec in layer_specs:
        if spec is None:
            layers.append(None)
            continue
        layers.append(PagedKVCache(page_table, n_heads=int(spec.n_heads), head_dim=int(spec.head_dim),
                                   dtype=dtype, pool=pool, k_scale=spec.k_scale, v_scale=spec.v_scale))
    return tuple(layers)


def copy_kv_pages(layers: Iterable[PagedKVCache | None], src_pages, dst_pages) -> None:
    """Run the pending copy-on-write copies on the K and V pools of every layer in one launch."""
    pools = []
    for layer in layers:
        if layer is not None:
            pools.append(layer.k_cache)
            pools.append(layer.v_cache)
    _k.copy_pages(pools, src_pages, dst_pages)


class PageTable:
    """Block table ``[max_batch_size, n_pages] int32`` with a pinned host copy, free lists
    and deferred host-to-device commits.

    Row 0 and physical page 0 are reserved (padding rows of a decode bucket write
    there).  Pages are handed out lowest-index first and reused LIFO.  Host-side
    edits mark rows dirty; :meth:`commit_block_table` uploads rows ``[0, max dirty]`` in
    one copy on ``h2d_stream``.  ``prefix_cache`` (optional) is asked to evict when
    the free list runs short and returns pages through :meth:`free_pages_to_pool`.
    """

    def __init__(self, n_pages: int, page_size: int, max_batch_size: int, device: str = "cuda",
                 prefix_cache=None, *, h2d_stream: torch.cuda.Stream | None = None):
        self.n_pages = n_pages
        self.page_size = page_size
        self.max_batch_size = max_batch_size
        self.device = device
        self._h2d_stream = h2d_stream

        self._page_table_buffer = CpuGpuBuffer(
            max_batch_size, n_pages, dtype=torch.int32, device=torch.device(device), pin_memory=True)
        self.page_table = self._page_table_buffer.gpu
        self._page_table_cpu_tensor = self._page_table_buffer.cpu
        self._page_table_cpu_np = self._page_table_buffer.np
        self._page_table_cpu_np[:] = -1
        self._page_table_cpu_np[0, :] = 0
        with _on_stream(self._h2d_stream):
            self._page_table_buffer.copy_to_gpu()

        self.page_table_cpu: list[list[int]] = [[] for _ in range(max_batch_size)]
        self.capacity = [0] * max_batch_size
        self.free_pages = list(range(n_pages - 1, 0, -1))
        self.free_batch_idx = list(range(max_batch_size - 1, 0, -1))
        self.num_blocks_per_row = np.zeros(max_batch_size, dtype=np.int32)
        self._dirty_rows: set[int] = set()
        self._pending_cow: list[tuple[int, int]] = []

        self.prefix_cache = None
        if prefix_cache is not None:
            page_granular = bool(getattr(prefix_cache, "page_granular", False))
            assert page_size == 1 or page_granular, (
                f"Prefix caching requires page_size=1, got {page_size}. "
                "With page_size>1, partial page reuse would cause leaks or corruption."
            )
            cache_page_size = getattr(prefix_cache, "page_size", page_size) if page_granular else page_size
            assert cache_page_size == page_size, (
                f"Prefix caching requires page_size={cache_page_size} (the page size of the cache), got {page_size}. "
                "A match would map pages that cover other positions than the tree recorded."
            )
            prefix_cache._free_pages_sink = self.free_pages_to_pool
            self.prefix_cache = prefix_cache

    # ------------------------------------------------------------------ queries
    @property
    def pages_available(self) -> int:
        return len(self.free_pages)

    def _pages_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    def can_reserve(self, size: int, batch_idx_int: int | None = None) -> bool:
        if batch_idx_int is None:
            return self.pages_available * self.page_size >= size and len(self.free_batch_idx) > 0
        return self.reserve(batch_idx_int, size, dry_run=True)

    def _reclaimable_enough(self, pages_needed: int) -> bool:
        have = self.pages_available
        if have >= pages_needed:
            return True
        cache = self.prefix_cache
        if cache is None:
            return False
        if have + cache.evictable_page_count() >= pages_needed:
            return True
        return have + cache.reclaimable_page_count() >= pages_needed

    def can_reserve_with_eviction(self, size: int, batch_idx_int: int | None = None) -> bool:
        if batch_idx_int is None:
            if not self.free_batch_idx:
                return False
            needed = self._pages_for(size)
        else:
            have = self.capacity[batch_idx_int]
            if size <= have:
                return True
            needed = self._pages_for(size - have)
        return self._reclaimable_enough(needed)

    def can_reserve_pages(self, size: int) -> bool:
        return self._reclaimable_enough(self._pages_for(size))

    def get_pages(self, batch_idx: int, start: int, end: int) -> list[int]:
        return self._page_table_cpu_tensor[batch_idx, start:end].tolist()

    def common_prefix_pages(self, batch_indices: Sequence[int], min_tokens: int | None = None) -> int:
        """Number of leading pages that all the given rows map to the same physical pages (host table).

        These are the pages of a cached prefix the rows were attached to with ``map_pages``
        (``kestrel/models/moondream/runtime.py:1572-1623``).  ``min_tokens`` caps the answer at the pages
        that lie entirely below that token count: pass the smallest ``seqused_k - seqlen_q`` of the
        step so that every query row sees every key of the prefix.  The result is what
        ``flash_attn_fwd(shared_prefix_pages=...)`` expects; it only changes when rows are mapped or
        released, so a scheduler computes it once per batch composition, not per step.
        """
        rows = list(batch_indices)
        if len(rows) < 2:
            return 0
        n = min(len(self.page_table_cpu[r]) for r in rows)
        if min_tokens is not None:
            n = min(n, max(0, int(min_tokens)) // self.page_size)
        if n <= 0:
            return 0
        tab = self._page_table_cpu_np[rows, :n]
        same = (tab == tab[0]).all(axis=0)
        return int(n if same.all() else same.argmin())

    # ------------------------------------------------------------------ rows and pages
    def allocate(self) -> int:
        row = self.free_batch_idx.pop()
        self.capacity[row] = 0
        self.num_blocks_per_row[row] = 0
        return row

    def _take_pages(self, count: int) -> list[int]:
        if count <= 0:   # free_pages[-0:] would be the whole list
            return []
        taken = self.free_pages[-count:]
        del self.free_pages[-count:]
        return taken

    def reserve(self, batch_idx: int, seq_len: int, dry_run: bool = False) -> bool:
        """Grow row ``batch_idx`` until it can hold ``seq_len`` tokens (evicting cached
        prefixes if needed); ``RuntimeError`` when the pool cannot supply the pages."""
        have = self.capacity[batch_idx]
        if seq_len <= have:
            return True
        need = self._pages_for(seq_len - have)
        enough = need <= self.pages_available
        if dry_run:
            return enough
        if not enough and self.prefix_cache is not None:
            self.prefix_cache.evict(need - self.pages_available)
            enough = need <= self.pages_available
        if not enough:
            msg = (
                f"Cannot reserve {need} pages for a sequence of length {seq_len} "
                f"in batch {batch_idx}. Only {self.pages_available} pages available. "
                f"Current capacity is {have} tokens."
            )
            if self.prefix_cache is not None:
                msg += " All cached prefixes are locked by active sequences."
            raise RuntimeError(msg)
        first = have // self.page_size
        pages = self._take_pages(need)
        self._page_table_cpu_np[batch_idx, first:first + need] = pages
        self.page_table_cpu[batch_idx] += pages
        self.capacity[batch_idx] = have + need * self.page_size
        self.num_blocks_per_row[batch_idx] = first + need
        self._dirty_rows.add(batch_idx)
        return True

    def allocate_pages(self, count: int) -> list[int]:
        """Unbound physical pages (to be placed with :meth:`map_pages`), evicting if short."""
        if len(self.free_pages) < count and self.prefix_cache is not None:
            self.prefix_cache.evict(count - len(self.free_pages))
        have = len(self.free_pages)
        if have < count:
            msg = f"Cannot allocate {count} pages: {have} available"
            if self.prefix_cache is not None:
                msg += ", all cached prefixes are locked by active sequences"
            raise RuntimeError(msg)
        return self._take_pages(count)

    def map_pages(self, batch_idx: int, logical_start: int, physical_pages: list[int]) -> None:
        """Bind ``physical_pages`` to consecutive logical pages of a row, starting exactly
        at the row's current page count."""
        held = len(self.page_table_cpu[batch_idx])
        assert logical_start == held, (
            f"map_pages must be called sequentially: expected logical_start={held}, got {logical_start}"
        )
        if not physical_pages:
            return
        stop = logical_start + len(physical_pages)
        self._page_table_cpu_np[batch_idx, logical_start:stop] = physical_pages
        self.capacity[batch_idx] = max(self.capacity[batch_idx], stop * self.page_size)
        self.page_table_cpu[batch_idx].extend(physical_pages)
        self.num_blocks_per_row[batch_idx] = max(int(self.num_blocks_per_row[batch_idx]), stop)
        self._dirty_rows.add(batch_idx)

    def unmap_pages(self, batch_idx: int, keep: int) -> None:
        """Drop the row's entries from logical page ``keep`` on WITHOUT freeing them: the inverse of
        :meth:`map_pages` for pages that stay with their owner (a prefix-cache attach that failed)."""
        row = self.page_table_cpu[batch_idx]
        if keep >= len(row):
            return
        self._page_table_cpu_np[batch_idx, keep:len(row)] = -1
        del row[keep:]
        self.capacity[batch_idx] = keep * self.page_size
        self.num_blocks_per_row[batch_idx] = keep
        self._dirty_rows.add(batch_idx)

    def free_pages_to_pool(self, pages: tuple[int, ...] | list[int]) -> None:
        self.free_pages.extend(pages)

    def erase(self, batch_idx: int, cached_page_count: int = 0) -> None:
        """Release a row.  Its first ``cached_page_count`` pages belong to the prefix cache
        and stay allocated; the rest return to the free list."""
        self.free_batch_idx.append(batch_idx)
        private = self.page_table_cpu[batch_idx][cached_page_count:]
        self.free_pages.extend(reversed(private))
        self.page_table_cpu[batch_idx] = []
        self.capacity[batch_idx] = 0
        self.num_blocks_per_row[batch_idx] = 0
        self._dirty_rows.discard(batch_idx)

    # ------------------------------------------------------------------ copy-on-write
    def cow_page(self, batch_idx: int, logical_page: int) -> tuple[int, int]:
        """Give row ``batch_idx`` a private copy of its ``logical_page``-th page.

        Takes a fresh physical page (evicting if needed), rewrites the row entry,
        marks the row dirty and queues the ``(src, dst)`` device copy; returns that
        pair.  The old page stays with its owner (the prefix cache / other rows).
        The queued copies run with :func:`copy_kv_pages` on the pairs from
        :meth:`take_pending_page_copies`, before the row's next append.
        """
        row_pages = self.page_table_cpu[batch_idx]
        if not 0 <= logical_page < len(row_pages):
            raise IndexError(f"row {batch_idx} has no logical page {logical_page}")
        src = row_pages[logical_page]
        (dst,) = self.allocate_pages(1)
        row_pages[logical_page] = dst
        self._page_table_cpu_np[batch_idx, logical_page] = dst
        self._dirty_rows.add(batch_idx)
        self._pending_cow.append((src, dst))
        return src, dst

    def take_pending_page_copies(self) -> tuple[list[int], list[int]]:
        """Pop the queued copy-on-write pairs as ``(src_pages, dst_pages)``."""
        pairs, self._pending_cow = self._pending_cow, []
        return [s for s, _ in pairs], [d for _, d in pairs]

    # ------------------------------------------------------------------ device side
    def _sync_page_table_row(self, batch_idx: int, start: int = 0, end: Optional[int] = None) -> None:
        end = self.n_pages if end is None else end
        if start >= end:
            return
        with _on_stream(self._h2d_stream):
            self.page_table[batch_idx, start:end].copy_(
                self._page_table_cpu_tensor[batch_idx, start:end], non_blocking=True)

    def _sync_full_page_table(self) -> None:
        with _on_stream(self._h2d_stream):
            self._page_table_buffer.copy_to_gpu()

    def commit_block_table(self, batch_indices: list[int] | None = None) -> None:
        """Upload dirty rows (all, or those among ``batch_indices``) as one copy of rows
        ``[0, max dirty row]``; clean rows cost nothing."""
        dirty = set(self._dirty_rows) if batch_indices is None else self._dirty_rows.intersection(batch_indices)
        if not dirty:
            return
        with _on_stream(self._h2d_stream):
            self._page_table_buffer.copy_to_gpu(max(dirty) + 1)
        self._dirty_rows -= dirty

    def build_slot_mapping(self, batch_idx: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """``slots[b, s] = page_table[batch, pos // P] * P + pos % P`` (int64, shape of ``positions``)."""
        if batch_idx.ndim != 1 and batch_idx.shape != positions.shape:
            raise ValueError("batch_idx and positions shape mismatch")
        if self.page_table.device.type != "cuda":
            raise RuntimeError("build_slot_mapping runs on the GPU; this PageTable lives on "
                               f"{self.page_table.device} (no CPU fallback)")
        if batch_idx.ndim == 1 and positions.ndim == 1:
            return _k.build_slot_mapping(self.page_table, batch_idx, positions.view(-1, 1), self.page_size).view(-1)
        return _k.build_slot_mapping(self.page_table, batch_idx, positions, self.page_size)

    def populate_paged_kv_metadata(self, *, batch_idx: torch.Tensor, input_pos: torch.Tensor,
                                   out_page_table: torch.Tensor, out_seqused_k: torch.Tensor) -> None:
        """Fill the compact decode metadata for the active rows (checks and messages of
        ``kestrel/kv_cache.py:454-522``)."""
        if batch_idx.ndim != 1:
            raise ValueError("batch_idx must be 1D for paged-KV metadata")
        if input_pos.ndim != 1:
            raise ValueError("input_pos must be 1D for paged-KV metadata")
        if batch_idx.shape[0] != input_pos.shape[0]:
            raise ValueError("batch_idx and input_pos must have the same length")
        if out_page_table.ndim != 2:
            raise ValueError("out_page_table must be 2D")
        if out_seqused_k.ndim != 1:
            raise ValueError("out_seqused_k must be 1D")
        n = batch_idx.shape[0]
        if out_page_table.shape[0] < n:
            raise ValueError("out_page_table has insufficient batch capacity")
        if out_page_table.shape[1] < self.n_pages:
            raise ValueError("out_page_table has insufficient page capacity")
        if out_seqused_k.shape[0] < n:
            raise ValueError("out_seqused_k has insufficient batch capacity")
        for nm, t in (("out_page_table", out_page_table), ("out_seqused_k", out_seqused_k),
                      ("input_pos", input_pos), ("page_table", self.page_table)):
            if t.dtype != torch.int32:
                raise ValueError(f"{nm} must be int32")
        if out_page_table.stride(-1) != 1:
            raise ValueError("out_page_table must be contiguous in the last dimension")
        dev = self.page_table.device
        if batch_idx.device != dev or input_pos.device != dev:
            raise ValueError(f"batch_idx/input_pos must live on {dev}, got {batch_idx.device}/{input_pos.device}")
        if out_page_table.device != dev or out_seqused_k.device != dev:
            raise ValueError(f"out_page_table/out_seqused_k must live on {dev}")
        if n == 0:
            return
        _k.build_paged_kv_metadata(self.page_table, batch_idx, input_pos, out_page_table, out_seqused_k,
                                   self.page_size)

    def populate_decode_step(self, *, batch_idx: torch.Tensor, input_pos: torch.Tensor,
                             out_page_table: torch.Tensor, out_seqused_k: torch.Tensor, n_new: int = 1,
                             out_slot_mapping: Optional[torch.Tensor] = None,
                             out_positions: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
        """:meth:`populate_paged_kv_metadata`, ``position_ids`` and :meth:`build_slot_mapping` for
        the ``n_new`` tokens per row ending at ``input_pos`` in one launch (the three steps at
        ``kestrel/models/moondream/runtime.py:2554-2564``).  Returns ``(slot_mapping, position_ids)``,
        int64 ``[B, n_new]``.  Not in the reference."""
        if out_page_table.ndim != 2 or out_page_table.shape[1] < self.n_pages:
            raise ValueError("out_page_table has insufficient page capacity")
        return _k.build_decode_step_metadata(self.page_table, batch_idx, input_pos, out_page_table, out_seqused_k,
                                             self.page_size, n_new=n_new, out_slot_mapping=out_slot_mapping,
                                             out_positions=out_positions)
