"""The reference's OWN host-side test files, run unmodified against this repository's mirror.

``oracle/stage_reference.py`` stages the reference's ``tests/test_kv_pool.py``, ``tests/test_page_table.py``
and ``tests/prefix_cache/*.py`` (byte copies, git-ignored); a child pytest collects them with the plugin
``tests/reference_alias.py``, which makes ``kestrel.kv_cache`` / ``kestrel.prefix_cache`` resolve to
``kestrel_b200``.  Every test must pass except the ones listed below, which cannot run here by design:
they call device ops on CPU tensors (this library has no CPU path; the same cases run on the GPU through
the reference's classes in ``tests/test_gpu_reference_dropin.py``) or exercise the Moondream model runtime,
which is outside the paged-KV path.
"""

from __future__ import annotations

import re
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
STAGED = ROOT / "oracle" / "_ref"

NEEDS_DEVICE_OPS_ON_CPU = {
    "test_page_table.py::test_populate_paged_kv_metadata_copies_active_pages_and_preserves_tail",
    "test_page_table.py::TestBackwardCompatibility::test_build_slot_mapping_still_works",
    "test_kv_pool.py::test_paged_cache_update_accepts_fused_projection_value_slice",
    "test_kv_pool.py::test_paged_cache_update_accepts_batched_decode_value_slice",
}
NEEDS_THE_MODEL_RUNTIME = {
    "test_page_table.py::TestDuplicatePrefill::test_duplicate_prefill_miss_does_not_lock_cache",
    "test_page_table.py::TestDuplicatePrefill::test_duplicate_prefill_partial_hit_keeps_prefix_lock",
    "test_page_table.py::TestDecodedPrefixRetention::test_retain_sequence_prefix_extends_cache_to_processed_generated_tokens",
    "test_page_table.py::TestDecodedPrefixRetention::test_retain_sequence_prefix_does_not_claim_duplicate_private_pages",
    "test_page_table.py::TestDecodedPrefixRetention::test_retain_sequence_prefix_skips_divergent_cached_prefix",
}


def _staged_tests() -> Path:
    """The staged reference tests; staged on the spot when a reference checkout is at hand."""
    if not (STAGED / "tests" / "test_page_table.py").exists():
        sys.path.insert(0, str(ROOT))
        from oracle import stage_reference

        if not (Path(stage_reference.DEFAULT_REFERENCE) / "kestrel" / "kv_cache.py").exists():
            pytest.skip("no staged reference files and no reference checkout to stage them from")
        stage_reference.stage(Path(stage_reference.DEFAULT_REFERENCE))
    return STAGED / "tests"


def _run(files: list[Path]) -> tuple[set[str], int]:
    proc = subprocess.run(
        [sys.executable, "-m", "pytest", *map(str, files), "-p", "tests.reference_alias", "-q", "-rf",
         "--rootdir", str(files[0].parent), "-c", "/dev/null", "-p", "no:cacheprovider"],
        cwd=ROOT, capture_output=True, text=True, timeout=600)
    failed = set()
    for line in proc.stdout.splitlines():
        m = re.match(r"FAILED\s+(\S+)", line)
        if m:
            node = m.group(1)
            failed.add(node[node.index("test_"):] if "/test_" in node else node)
    m = re.search(r"(\d+) passed", proc.stdout)
    assert m, f"child pytest produced no summary:\n{proc.stdout[-2000:]}\n{proc.stderr[-2000:]}"
    return failed, int(m.group(1))


def test_reference_radix_cache_and_token_tests_pass_on_the_mirror():
    tests = _staged_tests()
    failed, passed = _run([tests / "prefix_cache" / "test_radix_cache.py", tests / "prefix_cache" / "test_tokens.py"])
    assert failed == set(), failed
    assert passed >= 70


def test_reference_page_table_and_pool_tests_pass_on_the_mirror():
    tests = _staged_tests()
    failed, passed = _run([tests / "test_page_table.py", tests / "test_kv_pool.py"])
    unexpected = {f.split("/")[-1] for f in failed} - NEEDS_DEVICE_OPS_ON_CPU - NEEDS_THE_MODEL_RUNTIME
    assert unexpected == set(), unexpected
    assert passed >= 45
