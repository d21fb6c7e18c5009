"""Stages the reference's own modules for this path so that tests can run them unmodified.

TEST INFRASTRUCTURE ONLY.  Nothing under ``kestrel_b200/`` imports, reads or needs what this script
writes; the product never routes through it.

    python oracle/stage_reference.py [--reference /path/to/kestrel-checkout]

copies, byte for byte, from the reference tree into ``oracle/_ref/`` (git-ignored: the copies are
build outputs of this recipe, not sources of this repository):

* ``kestrel/kv_cache.py``, ``kestrel/ops/attention.py`` (+ ``ops/__init__.py``),
  ``kestrel/utils/buffers.py`` (+ ``utils/__init__.py``), ``kestrel/device.py``,
  ``kestrel/prefix_cache/*.py``, ``kestrel/runtime/tokens.py`` -- the host side of the paged-KV path,
  which binds its kernels from ``kestrel_kernels`` at import time (``kestrel/kv_cache.py:10-17``) and at
  call time (``kestrel/ops/attention.py:69``);
* ``tests/test_kv_pool.py``, ``tests/test_page_table.py``, ``tests/prefix_cache/*.py`` -- the reference's
  tests of that host side.

The tests under ``tests/`` then (a) register ``kestrel_b200.kernels`` as ``kestrel_kernels`` and drive the
staged ``PagedKVCache`` / ``PageTable`` / ``paged_attention`` / ``RadixPrefixCache`` on the GPU against the
oracle, and (b) run the staged reference tests against this repository's host mirror.  Both kinds skip
when ``oracle/_ref`` is absent.  ``kestrel/__init__.py`` is deliberately NOT staged (it imports every
model); the tests create the package object themselves (``tests/helpers.py``).
"""

from __future__ import annotations

import argparse
import hashlib
import json
import shutil
import sys
from pathlib import Path

import os

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
# a checkout named "reference" beside this repository, unless the environment names another place
DEFAULT_REFERENCE = os.environ.get("KESTREL_REFERENCE_DIR", str(HERE.parent.parent / "reference"))

MODULES = (
    "kestrel/kv_cache.py",
    "kestrel/device.py",
    "kestrel/ops/__init__.py",
    "kestrel/ops/attention.py",
    "kestrel/utils/__init__.py",
    "kestrel/utils/buffers.py",
    "kestrel/prefix_cache/__init__.py",
    "kestrel/prefix_cache/base.py",
    "kestrel/prefix_cache/eviction.py",
    "kestrel/prefix_cache/namespace.py",
    "kestrel/prefix_cache/radix_cache.py",
    "kestrel/prefix_cache/tokens.py",
    "kestrel/runtime/tokens.py",
)
TESTS = (
    "tests/test_kv_pool.py",
    "tests/test_page_table.py",
    "tests/prefix_cache/__init__.py",
    "tests/prefix_cache/test_radix_cache.py",
    "tests/prefix_cache/test_tokens.py",
)


def stage(reference: Path, dest: Path = DEST) -> dict:
    """Copy the files listed above; returns ``{relative path: sha256}`` (also written to
    ``dest/MANIFEST.json``).  A file the reference does not have is skipped and listed as ``None``."""
    reference = Path(reference)
    if not (reference / "kestrel" / "kv_cache.py").exists():
        raise FileNotFoundError(f"{reference} does not look like a kestrel checkout")
    if dest.exists():
        shutil.rmtree(dest)
    manifest: dict[str, str | None] = {}
    for rel in MODULES + TESTS:
        src = reference / rel
        if not src.exists():
            manifest[rel] = None
            continue
        out = dest / rel
        out.parent.mkdir(parents=True, exist_ok=True)
        data = src.read_bytes()
        out.write_bytes(data)
        manifest[rel] = hashlib.sha256(data).hexdigest()
    (dest / "MANIFEST.json").write_text(json.dumps(manifest, indent=1, sort_keys=True))
    return manifest


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    args = ap.parse_args()
    manifest = stage(Path(args.reference))
    missing = [k for k, v in manifest.items() if v is None]
    print(f"staged {len(manifest) - len(missing)} files into {DEST}" + (f"; missing: {missing}" if missing else ""))
    if missing:
        sys.exit(1)


if __name__ == "__main__":
    main()
