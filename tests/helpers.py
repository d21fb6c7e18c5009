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


def import_staged_reference():
    """The reference's own ``kestrel.kv_cache`` / ``kestrel.ops.attention`` / ``kestrel.prefix_cache`` modules
    (byte copies staged by ``oracle/stage_reference.py``) imported UNMODIFIED on top of this library:
    ``kestrel_b200.install_as_kestrel_kernels()`` registers the shim under the name they bind at import
    time (``kestrel/kv_cache.py:10-17``).  ``kestrel/__init__.py`` is not staged (it imports every model),
    so the package objects are made here.  Returns ``(kv_cache, ops.attention, prefix_cache)`` or ``None``
    when nothing is staged."""
    import importlib
    import sys
    import types
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "kestrel"
    if not (root / "kv_cache.py").exists():
        return None
    import kestrel_b200

    kestrel_b200.install_as_kestrel_kernels()
    if getattr(sys.modules.get("kestrel"), "__path__", None) != [str(root)]:
        for name in [m for m in sys.modules if m == "kestrel" or m.startswith("kestrel.")]:
            del sys.modules[name]
        pkg = types.ModuleType("kestrel")
        pkg.__path__ = [str(root)]
        sys.modules["kestrel"] = pkg
        rt = types.ModuleType("kestrel.runtime")          # kestrel/runtime/__init__.py pulls the model runtimes
        rt.__path__ = [str(root / "runtime")]
        sys.modules["kestrel.runtime"] = rt
    return (importlib.import_module("kestrel.kv_cache"), importlib.import_module("kestrel.ops.attention"),
            importlib.import_module("kestrel.prefix_cache"))
