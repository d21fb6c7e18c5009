"""pytest plugin that makes ``import kestrel...`` resolve to this repository's host mirror.

Loaded with ``-p tests.reference_alias`` by ``tests/test_reference_suites.py`` in a child pytest
process that collects the reference's OWN test files (staged by ``oracle/stage_reference.py``):
``kestrel.kv_cache`` is ``kestrel_b200.kv_cache`` and ``kestrel.prefix_cache`` is
``kestrel_b200.prefix_cache`` with ``RadixPrefixCache`` naming the page-granular cache (page size 1,
its default, is the reference's only mode); ``kestrel.runtime.tokens`` is the reference's own staged
file.  ``kestrel.models.moondream.runtime`` -- imported at the
top of the reference's ``tests/test_page_table.py`` for five tests of the Moondream runtime's cache
policy -- is an empty stand-in: those tests fail on their first use of it and are listed as expected
failures by the caller.
"""

from __future__ import annotations

import importlib.util
import sys
import types
from pathlib import Path

import kestrel_b200.kv_cache as _kv
import kestrel_b200.prefix_cache as _pc


def _package(name: str) -> types.ModuleType:
    mod = types.ModuleType(name)
    mod.__path__ = []  # a package without files: only the aliases below exist under it
    sys.modules[name] = mod
    return mod


def install() -> None:
    root = _package("kestrel")
    sys.modules["kestrel.kv_cache"] = root.kv_cache = _kv

    pc = types.ModuleType("kestrel.prefix_cache")
    for name in ("CacheNamespace", "CacheToken", "ImageToken", "InsertResult", "MatchResult", "TreeNode"):
        setattr(pc, name, getattr(_pc, name))
    pc.RadixPrefixCache = _pc.PagedRadixCache
    sys.modules["kestrel.prefix_cache"] = root.prefix_cache = pc

    # typed runtime tokens: plain NamedTuples with cache_key()/kv_length(); the reference's own file
    staged = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "kestrel" / "runtime" / "tokens.py"
    if staged.exists():
        rt = _package("kestrel.runtime")
        spec = importlib.util.spec_from_file_location("kestrel.runtime.tokens", staged)
        tokens = importlib.util.module_from_spec(spec)
        sys.modules["kestrel.runtime.tokens"] = rt.tokens = tokens
        spec.loader.exec_module(tokens)
        root.runtime = rt

    models = _package("kestrel.models")
    moondream = _package("kestrel.models.moondream")
    runtime = types.ModuleType("kestrel.models.moondream.runtime")

    class MoondreamRuntime:  # the model runtime is outside the paged-KV path
        pass

    runtime.MoondreamRuntime = MoondreamRuntime
    if "kestrel.runtime.tokens" in sys.modules:   # the runtime re-exports the typed tokens
        for name in ("TextToken", "CoordToken", "SizeToken"):
            setattr(runtime, name, getattr(sys.modules["kestrel.runtime.tokens"], name))
    sys.modules["kestrel.models.moondream.runtime"] = moondream.runtime = runtime
    root.models, models.moondream = models, moondream


install()
