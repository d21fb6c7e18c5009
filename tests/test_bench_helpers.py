"""Host-side pieces of ``bench.py`` that need no GPU: the kernel a workload lands on, the DRAM-traffic ratios read
from the profile summaries (and their staleness stamp), the algorithmic-byte formula."""

import hashlib
import importlib
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
bench = importlib.import_module("bench")


def test_every_decode_workload_names_its_kernel():
    want = {"cfg2": "paged_attn_kernel", "cfg3": "paged_attn_decode_kernel", "cfg4": "paged_attn_decode_kernel",
            "cfg5": "paged_attn_kernel", "cfg5_sq8": "paged_prefill_kernel", "cfg5_sq16": "paged_prefill_kernel"}
    for name, kernel in want.items():
        assert bench.split_kv_kernel_name(bench.WORKLOADS[name]) == kernel, name
    small = dict(bench.WORKLOADS["cfg5_sq8"], batch=16)      # 16 x 8 (sequence, KV head) pairs: fewer than the SMs
    assert bench.split_kv_kernel_name(small) == "paged_attn_rows32_kernel"
    fp8 = dict(bench.WORKLOADS["cfg5_sq16"], kv="fp8")       # 64 rows on an FP8 pool: two passes of the 32-row kernel
    assert bench.split_kv_kernel_name(fp8) == "paged_attn_rows32_kernel"


def test_traffic_ratios_come_from_the_profile_summaries():
    for (kernel, kv), rel in bench.TRAFFIC_PROFILES.items():
        got = bench.dram_traffic_ratio(kernel, kv)
        assert got["profile"] == rel and (ROOT / rel).exists()
        assert got["ratio"] is not None and 0.99 < got["ratio"] < 1.2, (kernel, kv, got)
        assert got["stale"] in (True, False)
    assert bench.dram_traffic_ratio("no_such_kernel", "bf16") == {"ratio": None, "profile": None, "stale": None}


def test_staleness_stamp_follows_the_source_file(tmp_path, monkeypatch):
    src = tmp_path / "k.cuh"
    src.write_text("// kernel\n")
    md = tmp_path / "p.md"
    md.write_text(f"kernel source sha256 (`k.cuh`) = {hashlib.sha256(src.read_bytes()).hexdigest()}\n"
                  "| DRAM traffic ÷ algorithmic bytes | **1.0100** |\n")
    monkeypatch.setattr(bench, "ROOT", tmp_path)
    monkeypatch.setitem(bench.TRAFFIC_PROFILES, ("k", "bf16"), "p.md")
    assert bench.dram_traffic_ratio("k", "bf16") == {"ratio": 1.01, "profile": "p.md", "stale": False}
    src.write_text("// kernel, edited\n")
    assert bench.dram_traffic_ratio("k", "bf16")["stale"] is True


def test_algorithmic_bytes_count_tokens_not_pages():
    lengths = torch.tensor([1, 17, 4096])
    got = bench.algorithmic_bytes(lengths, layers=2, kv_bytes=1, head_dim=128, sq=1, batch=3)
    kv = int(lengths.sum()) * 2 * bench.HKV * 128          # K + V, one byte per element
    assert got["attn_per_launch"] >= kv and got["attn_per_launch"] - kv < 64 * 1024
    assert got["per_step"] >= 2 * got["attn_per_launch"]
