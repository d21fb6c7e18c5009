"""B200-native (sm_100a) implementation of Kestrel's paged-KV hot path.

Public surface: the host-side classes of ``kestrel/kv_cache.py`` (:mod:`.kv_cache`), the
paged attention op of ``kestrel/ops/attention.py`` (:mod:`.attention`) and a
``kestrel_kernels``-compatible runtime object (:mod:`.kernels`).  The kernels live in
``libkestrel_b200.so`` (C ABI: ``include/kestrel_b200.h``); importing this package
does not load it, the first kernel call or :func:`kernels.get_runtime` does, and
fails loudly if it is missing.
"""

from .attention import paged_attention
from .kernels import get_runtime, install_as_kestrel_kernels
from .kv_cache import (KVMemoryPool, LayerPagedCache, PagedKVCache, PagedKVLayerSpec, PageTable,
                       allocate_paged_kv_layers, copy_kv_pages)
from .prefix_cache import (CacheNamespace, ImageToken, PagedRadixCache, SequenceCacheState, attach_cached_prefix,
                           finalize_cached_prompt, release_cached_sequence, retain_generated_prefix)

__all__ = [
    "KVMemoryPool", "LayerPagedCache", "PagedKVCache", "PagedKVLayerSpec", "PageTable", "allocate_paged_kv_layers",
    "copy_kv_pages", "paged_attention", "get_runtime", "install_as_kestrel_kernels",
    "PagedRadixCache", "CacheNamespace", "ImageToken", "attach_cached_prefix", "SequenceCacheState",
    "finalize_cached_prompt", "retain_generated_prefix", "release_cached_sequence",
]
__version__ = "0.1.0"
