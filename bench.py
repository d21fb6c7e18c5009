"""Benchmark of the paged-KV hot path: append + paged decode attention over a KV stack.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2|cfg3|cfg4|cfg5|cfg5_sq8|cfg5_sq16|ref_mha64_p1] [--impl reference]

One *step* is one decode step of the whole KV stack of the workload: decode metadata and slot
mapping once, then per layer the append of the new tokens' K/V rows (quantised to FP8 where the
workload says so) and the paged attention of the new queries over the grown context.  Inputs are
seeded synthetic tensors with the shapes and value distributions of the named configuration.

Default workload ``cfg3``: FP8 e4m3 KV with per-(layer, KV-head) scales, 24 layers, batch 256,
contexts U[4096, 32768], 32 query / 8 KV heads, head_dim 128, page size 16, inputs N(0,1) with
1 % outliers x20.  24 layers of that context need about 232 GB of KV, more than one GPU holds, so
the stack keeps as many *distinct* layer pools as fit (``config.n_layer_pools``) and layer ``i``
uses pool ``i mod n``: every layer still streams its whole KV from HBM (a pool is ~10 GB, far
beyond L2).

With N > 1 (launched by torchrun, one rank per GPU) every rank runs the same workload on its own
sequences (requests shard by sequence; no collective on the data path); the time is the max over
ranks and ``value`` is the sum over ranks: weak scaling.

The one JSON line printed by rank 0 carries the whole-job HBM GB/s (``value``), tokens/s, the
end-to-end number with host buffers (``e2e``), the roofline of the attention kernel, the clocks
seen during the timed region and a CPU baseline (the oracle timed on the host cores).
``--impl reference`` times the CPU restatement of the reference's torch path instead.

``--workload pf4|pf_long`` measure the prefill mode of the same op (rotary + append of a prompt chunk,
then paged attention of the chunk's queries over prefix + chunk): compute-bound, reported in TFLOP/s
against the measured bf16 tensor peak.  ``pf4`` is the prefill phase of configuration 4 (512 requests
on a shared 729-token prefix, suffixes U[32,256] appended in chunks of up to 128 tokens, D=64);
``pf_long`` is 32 sequences appending a 512-token chunk on 4096 cached tokens, D=128 (``pf_long_fp8``: the same
on FP8 e4m3 pools).
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
# DRAM read+write bytes of one attention launch divided by its algorithmic bytes come from the ncu captures
# summarised under profiles/ (each summary states the ratio and the sha256 of the kernel source it was taken
# with).  Traffic grows with the tokens attended, so a full launch is that ratio times its algorithmic bytes.
# ncu summary that holds the DRAM-traffic ratio of each attention kernel (a reduced launch of the same kernel)
TRAFFIC_PROFILES = {
    ("paged_attn_decode_kernel", "fp8"): "profiles/paged_attn_decode_kernel_fp8_cfg3_reduced.md",
    ("paged_attn_decode_kernel", "bf16"): "profiles/cfg4_shared_prefix_step.md",
    ("paged_attn_kernel", "bf16"): "profiles/paged_attn_kernel_bf16_cfg2.md",
    ("paged_attn_rows32_kernel", "bf16"): "profiles/paged_attn_rows32_kernel_bf16_cfg5_sq8_reduced.md",
    ("paged_prefill_kernel", "bf16"): "profiles/paged_prefill_kernel_bf16_key_split_cfg5_sq16_reduced.md",
}


def dram_traffic_ratio(kernel: str, kv: str, rel: str | None = None) -> dict:
    """{"ratio", "profile", "stale"}: the ratio a profile summary records, and whether the kernel source
    changed since (the summary names the source file and the sha256 it was captured with)."""
    import hashlib
    import re
    rel = rel or TRAFFIC_PROFILES.get((kernel, kv))
    out = {"ratio": None, "profile": rel, "stale": None}
    if rel is None or not (ROOT / rel).exists():
        return out
    text = (ROOT / rel).read_text()
    m = re.search(r"DRAM traffic . algorithmic bytes[^0-9]*([0-9]+\.[0-9]+)", text)
    if m:
        out["ratio"] = float(m.group(1))
    m = re.search(r"kernel source sha256 \(`([^`]+)`\)\s*=\s*([0-9a-f]{64})", text)
    if m and (ROOT / m.group(1)).exists():
        out["stale"] = hashlib.sha256((ROOT / m.group(1)).read_bytes()).hexdigest() != m.group(2)
    return out


WORKLOADS = {
    # name: batch, len range, layers, kv dtype, head_dim, seqlen_q, outliers, pool factor
    "cfg2": dict(batch=64, lo=1024, hi=8192, layers=1, kv="bf16", head_dim=128, sq=1, outliers=0.0, pool=1.25,
                 desc="bf16, batch 64, ctx U[1024,8192], 1 layer, 32/8 heads, D=128, page 16, pool 1.25x"),
    "cfg3": dict(batch=256, lo=4096, hi=32768, layers=24, kv="fp8", head_dim=128, sq=1, outliers=0.01, pool=1.02,
                 desc="FP8 e4m3 KV (per layer+head scales, quantise on append), 24 layers, batch 256, "
                      "ctx U[4096,32768], 32/8 heads, D=128, page 16, N(0,1)+1% outliers x20"),
    "cfg4": dict(batch=512, lo=32, hi=256, layers=1, kv="bf16", head_dim=64, sq=1, outliers=0.0, pool=1.25, prefix=729,
                 desc="bf16, 512 requests sharing a 729-token prefix (COW of the partial page) + suffix U[32,256], "
                      "decode steps, 32/8 heads, D=64, page 16"),
    "cfg5": dict(batch=256, lo=2048, hi=16384, layers=24, kv="bf16", head_dim=128, sq=4, outliers=0.0, pool=1.02,
                 desc="bf16, 24 layers, 256 sequences per GPU, ctx U[2048,16384], 4-token verify + 4-token append, "
                      "32/8 heads, D=128, page 16"),
}
WORKLOADS["cfg5_sq8"] = dict(WORKLOADS["cfg5"], sq=8,
                             desc=WORKLOADS["cfg5"]["desc"].replace("4-token verify + 4-token append",
                                                                    "8-token verify + 8-token append (32 packed rows per KV head: at this batch "
                                                                    "the tensor-memory kernel with its key split)"))
WORKLOADS["cfg5_sq16"] = dict(WORKLOADS["cfg5"], sq=16,
                              desc=WORKLOADS["cfg5"]["desc"].replace("4-token verify + 4-token append",
                                                                     "16-token verify + 16-token append (64 packed rows per KV head: "
                                                                     "the tensor-memory kernel with its key split)"))
# The reference's own pools: page size 1 (kestrel/config.py:164), MHA with 32 heads of 64
# (kestrel/models/moondream/config.py:25-31), 24 layers, bf16.  `heads` / `page` override the module's geometry
# while this workload is measured.
WORKLOADS["ref_mha64_p1"] = dict(batch=64, lo=1024, hi=8192, layers=24, kv="bf16", head_dim=64, sq=1, outliers=0.0,
                                 pool=1.25, heads=(32, 32), page=1,
                                 traffic_profile="profiles/paged_attn_decode_kernel_bf16_ref_mha64_p1_reduced.md",
                                 desc="the reference's own geometry: bf16, 24 layers, batch 64, ctx U[1024,8192], "
                                      "32/32 heads (MHA), D=64, page 1, pool 1.25x")
HQ, HKV, PAGE = 32, 8, 16

PREFILL_WORKLOADS = {
    "pf4": dict(batch=512, prefix=729, lo=32, hi=256, chunk=128, head_dim=64, rot=32,
                desc="prefill phase of cfg4: 512 requests on a shared, cached 729-token prefix, suffix U[32,256] in "
                     "chunks of <=128 tokens; rotary + append + paged attention per chunk, bf16, 32/8 heads, D=64, page 16"),
    "pf_long": dict(batch=32, prefix=4096, lo=512, hi=512, chunk=512, head_dim=128, rot=128,
                    desc="32 sequences append a 512-token chunk on 4096 cached tokens; rotary + append + paged "
                         "attention, bf16, 32/8 heads, D=128, page 16"),
}
PREFILL_WORKLOADS["pf_long_fp8"] = dict(PREFILL_WORKLOADS["pf_long"], kv="fp8",
                                        desc=PREFILL_WORKLOADS["pf_long"]["desc"].replace("bf16", "FP8 e4m3 pools (per-head scales), bf16 q"))
FALLBACK_BF16_TFLOPS = 1590.0


# ----------------------------------------------------------------------------------------------
# helpers
# ----------------------------------------------------------------------------------------------

def split_kv_kernel_name(cfg: dict) -> str:
    """The attention kernel the library picks for a decode / verify workload (rows = GQA group x query positions per
    KV head; the rule of ``use_prefill_kernel`` in csrc/paged_attention.cuh, 148 SMs)."""
    rows = (HQ // HKV) * cfg["sq"]
    fp8 = cfg["kv"] == "fp8"
    if rows >= (65 if fp8 else 33) or (not fp8 and cfg["head_dim"] == 128 and rows > 16 and cfg["batch"] * HKV >= 148):
        return "paged_prefill_kernel"
    if rows > 16:
        return "paged_attn_rows32_kernel"
    if rows <= 8 and (fp8 or cfg["head_dim"] == 64):
        return "paged_attn_decode_kernel"
    return "paged_attn_kernel"


def measured_hbm_peak() -> tuple[float, str]:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        def pump():
            for line in self.proc.stdout:
                self.lines.append(line.strip())
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


def algorithmic_bytes(lengths_after: torch.Tensor, *, layers: int, kv_bytes: int, head_dim: int, sq: int,
                      batch: int) -> dict:
    """Bytes one step must move, per the formula of the measurement plan: K+V actually attended (tokens,
    not pages), Q read, O written, compact page table + lengths read, appended rows read (bf16) and
    written (KV dtype), slot map."""
    tok = int(lengths_after.sum())
    kv = tok * 2 * HKV * head_dim * kv_bytes
    qo = 2 * batch * sq * HQ * head_dim * 2
    table = int(((lengths_after + PAGE - 1) // PAGE).sum()) * 4 + batch * 4
    append = batch * sq * 2 * HKV * head_dim * (2 + kv_bytes) + batch * sq * 8
    per_layer = kv + qo + table + append
    return {"per_layer": per_layer, "per_step": per_layer * layers, "attn_per_launch": kv + qo + table}


# ----------------------------------------------------------------------------------------------
# GPU workload
# ----------------------------------------------------------------------------------------------

class GpuWorkload:
    def __init__(self, name: str, device: torch.device, rank: int, total_steps: int, budget_frac: float = 0.78,
                 share_prefix: bool = True):
        from kestrel_b200.kv_cache import KVMemoryPool, PagedKVCache, PageTable, copy_kv_pages
        from kestrel_b200 import kernels

        self.kernels = kernels
        self.cfg = cfg = WORKLOADS[name]
        self.name, self.device = name, device
        self.B, self.D, self.sq, self.layers_n = cfg["batch"], cfg["head_dim"], cfg["sq"], cfg["layers"]
        self.kv_dtype = torch.float8_e4m3fn if cfg["kv"] == "fp8" else torch.bfloat16
        self.kv_bytes = 1 if cfg["kv"] == "fp8" else 2
        # context lengths and the page permutation are the same on every rank (the per-GPU work of a
        # weak-scaling run must not depend on the rank's draw); the K/V/Q data below is seeded per rank
        g = torch.Generator().manual_seed(1000 + (int(name[3]) if name[3].isdigit() else 6))
        prefix = cfg.get("prefix", 0)
        suffix = torch.randint(cfg["lo"], cfg["hi"] + 1, (self.B,), generator=g)
        self.len0 = suffix + prefix                      # context before the first timed/warm-up step
        grow = total_steps * self.sq + 1
        final = self.len0 + grow
        if prefix:
            shared_pages = prefix // PAGE
            own_pages = ((final + PAGE - 1) // PAGE - shared_pages)
            total_pages = int(own_pages.sum()) + shared_pages + 1
        else:
            total_pages = int(((final + PAGE - 1) // PAGE).sum())
        self.n_pages = int(total_pages * cfg["pool"]) + 16
        per_layer = 2 * self.n_pages * HKV * PAGE * self.D * self.kv_bytes
        free, _ = torch.cuda.mem_get_info(device)
        table_bytes = 3 * (self.B + 2) * self.n_pages * 4
        budget = min(int(free * budget_frac), 150 * 2 ** 30) - table_bytes - (2 << 30)
        self.n_pools = max(1, min(self.layers_n, budget // per_layer))
        self.pool = KVMemoryPool(device=device)
        shared_cache = None
        if prefix:
            from kestrel_b200.prefix_cache import ImageToken, PagedRadixCache, attach_cached_prefix
            shared_cache = PagedRadixCache(page_size=PAGE)
        self.pt = PageTable(n_pages=self.n_pages, page_size=PAGE, max_batch_size=self.B + 2, device=device,
                            prefix_cache=shared_cache)
        # pages scattered by a seeded permutation of the free list
        order = torch.randperm(len(self.pt.free_pages), generator=g).tolist()
        self.pt.free_pages = [self.pt.free_pages[i] for i in order]

        dg = torch.Generator(device=device).manual_seed(4242 + rank)
        self.dg = dg
        self.caches = []
        scales = None
        for l in range(self.n_pools):
            kw = {}
            if self.kv_dtype == torch.float8_e4m3fn:
                kw = dict(k_scale=[1.0] * HKV, v_scale=[1.0] * HKV)  # set after the absmax pass
            self.caches.append(PagedKVCache(self.pt, n_heads=HKV, head_dim=self.D, dtype=self.kv_dtype,
                                            pool=self.pool, **kw))
        # rows and pages
        self.rows = []
        if prefix:
            # the shared prefix lives in the radix cache; every request matches it, maps the 45 full pages
            # and gets a copy-on-write page for the partly filled 46th
            owner = self.pt.allocate()
            self.pt.reserve(owner, prefix)
            self.owner_row = owner
            image = [ImageToken(content_hash=1000 + rank, kv_length_=prefix)]
            assert shared_cache.insert(image, list(self.pt.page_table_cpu[owner])).inserted_pages == -(-prefix // PAGE)

            class _Text:
                def __init__(self, req, k): self.key = (0, req, k)
                def cache_key(self): return self.key
                def kv_length(self): return 1

            for b in range(self.B):
                if not self.pt.free_batch_idx:
                    raise RuntimeError("page table has too few rows")
                r = self.pt.allocate()
                n_suffix = int(suffix[b])
                prompt = image + [_Text(b, k) for k in range(n_suffix)]
                skip, n_shared, match = attach_cached_prefix(self.pt, shared_cache, r, prompt, prefix + n_suffix)
                assert skip == prefix and n_shared == prefix // PAGE
                shared_cache.unlock_prefill(match.last_node)
                self.pt.reserve(r, int(final[b]))
                self.rows.append(r)
        else:
            for b in range(self.B):
                r = self.pt.allocate()
                self.pt.reserve(r, int(final[b]))
                self.rows.append(r)
        self.pt.commit_block_table()
        self.batch_idx = torch.tensor(self.rows, dtype=torch.int64, device=device)
        # pages of the cached prefix that every request of the batch maps (0 without a prefix cache): the
        # attention call reads them once for the whole batch
        self.shared_pages = (self.pt.common_prefix_pages(self.rows, min_tokens=int(self.len0.min()))
                             if prefix and share_prefix else 0)
        self.shared_tokens = (prefix // PAGE) * PAGE if prefix else 0   # KV tokens on pages every request maps
        self._fill(prefix, copy_kv_pages)
        # per-step inputs, resident in HBM (one set per layer so no layer reuses another's rows)
        self.q = [self._randn(self.B, self.sq, HQ, self.D).to(torch.bfloat16) for _ in range(self.layers_n)]
        self.k_new = [self._randn(self.B, self.sq, HKV, self.D).to(torch.bfloat16) for _ in range(self.layers_n)]
        self.v_new = [self._randn(self.B, self.sq, HKV, self.D).to(torch.bfloat16) for _ in range(self.layers_n)]
        self.out = [torch.empty_like(q) for q in self.q]
        self.meta_pt = torch.zeros(self.B, self.n_pages, dtype=torch.int32, device=device)
        self.meta_sk = torch.zeros(self.B, dtype=torch.int32, device=device)
        self.pos = torch.zeros(self.B, self.sq, dtype=torch.int64, device=device)
        self.step_no = 0
        kernels.reserve_attention_workspace(batch=self.B, total_q=self.B * self.sq, n_q_heads=HQ, n_kv_heads=HKV,
                                            head_dim=self.D, device=device)
        # host staging for the end-to-end variant
        self.h_in = [torch.empty(self.B, self.sq, (HQ + 2 * HKV) * self.D, dtype=torch.bfloat16).pin_memory()
                     for _ in range(self.layers_n)]
        for h in self.h_in:
            h.normal_()
        self.d_in = [torch.empty(self.B, self.sq, (HQ + 2 * HKV) * self.D, dtype=torch.bfloat16, device=device)
                     for _ in range(2)]
        self.h_out = torch.empty(self.layers_n, self.B, self.sq, HQ, self.D, dtype=torch.bfloat16).pin_memory()
        self.h_pos = torch.zeros(self.B, self.sq, dtype=torch.int64).pin_memory()
        self.h2d_stream = torch.cuda.Stream(device=device)
        self.d2h_stream = torch.cuda.Stream(device=device)
        self.in_ready = [torch.cuda.Event(), torch.cuda.Event()]
        self.in_free = [torch.cuda.Event(), torch.cuda.Event()]
        self.out_done = [torch.cuda.Event(), torch.cuda.Event()]
        for ev in self.in_free:
            ev.record(torch.cuda.current_stream(device))
        self.attn_events: list[tuple[torch.cuda.Event, torch.cuda.Event]] = []
        self.launches_per_step = 2 + self.layers_n * (6 if self.shared_pages else 4)

    def _randn(self, *shape):
        x = torch.randn(*shape, generator=self.dg, device=self.device)
        if self.cfg["outliers"] > 0:
            m = torch.rand(*shape, generator=self.dg, device=self.device) < self.cfg["outliers"]
            x = torch.where(m, x * 20.0, x)
        return x

    def _fill(self, prefix: int, copy_kv_pages) -> None:
        """Store the initial contexts through the library's own append (quantising where needed)."""
        dev = self.device
        chunk_tokens = 1 << 18
        # flat (row, position) list of every context token
        if prefix:
            seqs = [(self.owner_row, 0, prefix)] + [(r, prefix, int(L)) for r, L in zip(self.rows, self.len0.tolist())]
        else:
            seqs = [(r, 0, int(L)) for r, L in zip(self.rows, self.len0.tolist())]
        rows = torch.cat([torch.full((e - s,), r, dtype=torch.int32) for r, s, e in seqs]).to(dev)
        pos = torch.cat([torch.arange(s, e, dtype=torch.int32) for r, s, e in seqs]).to(dev)
        slots = self.kernels.build_slot_mapping(self.pt.page_table, rows.view(-1, 1), pos.view(-1, 1), PAGE).view(-1)
        T = slots.numel()
        for l, cache in enumerate(self.caches):
            seeds = [(l * 1000003 + c) for c in range((T + chunk_tokens - 1) // chunk_tokens)]
            if self.kv_dtype == torch.float8_e4m3fn:
                kmax = torch.zeros(HKV, device=dev)
                vmax = torch.zeros(HKV, device=dev)
                for c, seed in enumerate(seeds):
                    n = min(chunk_tokens, T - c * chunk_tokens)
                    self.dg.manual_seed(seed)
                    k = self._randn(n, HKV, self.D).to(torch.bfloat16)
                    v = self._randn(n, HKV, self.D).to(torch.bfloat16)
                    kmax = torch.maximum(kmax, k.float().abs().amax(dim=(0, 2)))
                    vmax = torch.maximum(vmax, v.float().abs().amax(dim=(0, 2)))
                cache.k_scale_tensor.copy_(kmax / 448.0)
                cache.v_scale_tensor.copy_(vmax / 448.0)
            for c, seed in enumerate(seeds):
                n = min(chunk_tokens, T - c * chunk_tokens)
                self.dg.manual_seed(seed)
                k = self._randn(n, HKV, self.D).to(torch.bfloat16)
                v = self._randn(n, HKV, self.D).to(torch.bfloat16)
                sl = slots[c * chunk_tokens: c * chunk_tokens + n]
                cache.update(sl.view(1, n), k.view(1, n, HKV, self.D), v.view(1, n, HKV, self.D),
                             slot_mapping=sl.view(1, n))
            del k, v
        if prefix and prefix % PAGE:
            # the prefix was stored in the owner's pages; give every request its copy of the partial page.
            src, dst = self.pt.take_pending_page_copies()
            # cow_page ran before the owner's page was filled, so run the queued copies now
            copy_kv_pages(self.caches, src, dst)
            self.cow_pairs = len(dst)
        torch.cuda.synchronize(dev)
        self.dg.manual_seed(99)

    # ---- one step, inputs resident in HBM
    def lengths_after(self, step_no: int) -> torch.Tensor:
        return self.len0 + (step_no + 1) * self.sq

    def step_device(self, record_attn: bool = False) -> None:
        t = self.step_no
        base = (self.len0 + t * self.sq).to(self.device, non_blocking=True)
        self.pos.copy_(base.view(-1, 1) + torch.arange(self.sq, device=self.device).view(1, -1))
        self._run_layers(self.pos, record_attn, host=False)
        self.step_no += 1

    # ---- the same step captured once in a CUDA graph (the reference replays its decode step from a
    # graph too, kestrel/runtime/decode_graph.py:93-123); positions advance on the device
    def capture_graph(self) -> None:
        t = self.step_no
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            self.kernels.reserve_attention_workspace(batch=self.B, total_q=self.B * self.sq, n_q_heads=HQ,
                                                     n_kv_heads=HKV, head_dim=self.D, device=self.device)
            base = (self.len0 + t * self.sq).to(self.device)
            self.pos.copy_(base.view(-1, 1) + torch.arange(self.sq, device=self.device).view(1, -1))
            stream.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=stream):
                self._run_layers(self.pos, False, host=False)
                self.pos.add_(self.sq)
        torch.cuda.current_stream(self.device).wait_stream(stream)
        torch.cuda.synchronize(self.device)

    def step_graph(self) -> None:
        self.graph.replay()
        self.step_no += 1

    def time_attention_launch(self, reps: int) -> float:
        """Average duration (ms) of one attention call (plan + attention + merge launches) at the current
        context lengths: every layer's call captured in one graph, replayed ``reps`` times, CUDA events
        on the launching stream.  Eager per-call events would add tens of microseconds of launch latency."""
        scale = 1.0 / math.sqrt(self.D)
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))

        def body():
            for l in range(self.layers_n):
                cache = self.caches[l % self.n_pools]
                self.kernels.flash_attn_fwd(
                    self.q[l], cache.k_cache.permute(0, 2, 1, 3), cache.v_cache.permute(0, 2, 1, 3),
                    page_table=self.meta_pt, seqused_k=self.meta_sk, causal=True, softmax_scale=scale,
                    k_scale=cache.k_scale, v_scale=cache.v_scale, out=self.out[l],
                    shared_prefix_pages=self.shared_pages)

        with torch.cuda.stream(stream):
            self.kernels.reserve_attention_workspace(batch=self.B, total_q=self.B * self.sq, n_q_heads=HQ,
                                                     n_kv_heads=HKV, head_dim=self.D, device=self.device)
            body()
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                body()
        torch.cuda.current_stream(self.device).wait_stream(stream)
        g.replay()
        torch.cuda.synchronize(self.device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize(self.device)
        return e0.elapsed_time(e1) / (reps * self.layers_n)

    # ---- one step through the public API with host buffers
    def step_e2e(self) -> None:
        t = self.step_no
        for b, r in enumerate(self.rows):
            self.pt.reserve(r, int(self.len0[b]) + (t + 1) * self.sq)
        self.pt.commit_block_table(self.rows)
        self.h_pos.copy_((self.len0 + t * self.sq).view(-1, 1) + torch.arange(self.sq).view(1, -1))
        self.pos.copy_(self.h_pos, non_blocking=True)
        self._run_layers(self.pos, False, host=True)
        torch.cuda.current_stream(self.device).synchronize()
        self.step_no += 1

    def _run_layers(self, pos: torch.Tensor, record_attn: bool, host: bool) -> None:
        slots = self.pt.build_slot_mapping(self.batch_idx, pos)
        self.pt.populate_paged_kv_metadata(batch_idx=self.batch_idx, input_pos=pos[:, -1].to(torch.int32),
                                           out_page_table=self.meta_pt, out_seqused_k=self.meta_sk)
        scale = 1.0 / math.sqrt(self.D)
        compute = torch.cuda.current_stream(self.device)
        for l in range(self.layers_n):
            cache = self.caches[l % self.n_pools]
            if host:
                # inputs of layer l+1 cross PCIe on a copy stream while layer l computes
                if l == 0:
                    self._stage_in(0)
                if l + 1 < self.layers_n:
                    self._stage_in(l + 1)
                compute.wait_event(self.in_ready[l & 1])
                d = self.d_in[l & 1]
                q, k, v = d.split([HQ * self.D, HKV * self.D, HKV * self.D], dim=-1)
                q = q.view(self.B, self.sq, HQ, self.D)
                k = k.view(self.B, self.sq, HKV, self.D)
                v = v.view(self.B, self.sq, HKV, self.D)
            else:
                q, k, v = self.q[l], self.k_new[l], self.v_new[l]
            cache.update(pos, k, v, slot_mapping=slots)
            if record_attn:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            out, _ = self.kernels.flash_attn_fwd(
                q, cache.k_cache.permute(0, 2, 1, 3), cache.v_cache.permute(0, 2, 1, 3), page_table=self.meta_pt,
                seqused_k=self.meta_sk, causal=True, softmax_scale=scale, k_scale=cache.k_scale, v_scale=cache.v_scale,
                out=self.out[l], shared_prefix_pages=self.shared_pages)
            if record_attn:
                e1.record()
                self.attn_events.append((e0, e1))
            if host:
                self.in_free[l & 1].record(compute)          # the staging buffer may be refilled
                self.out_done[l & 1].record(compute)
                with torch.cuda.stream(self.d2h_stream):
                    self.d2h_stream.wait_event(self.out_done[l & 1])
                    self.h_out[l].copy_(out, non_blocking=True)
        if host:
            compute.wait_stream(self.d2h_stream)

    def _stage_in(self, l: int) -> None:
        """Host -> device copy of layer ``l``'s fused q/k/v rows into staging buffer ``l & 1`` on the copy
        stream, after the layer that used that buffer last has consumed it."""
        with torch.cuda.stream(self.h2d_stream):
            self.h2d_stream.wait_event(self.in_free[l & 1])
            self.d_in[l & 1].copy_(self.h_in[l], non_blocking=True)
            self.in_ready[l & 1].record(self.h2d_stream)

    def e2e_bytes(self) -> tuple[int, int]:
        h2d = self.layers_n * self.h_in[0].numel() * 2 + self.h_pos.numel() * 8
        d2h = self.h_out.numel() * 2
        return h2d, d2h


# ----------------------------------------------------------------------------------------------
# Prefill workload (compute-bound mode of the same op)
# ----------------------------------------------------------------------------------------------

def measured_bf16_peak() -> tuple[float, str]:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["bf16_tflops"]), "measured (burst)"
        except Exception:
            pass
    return FALLBACK_BF16_TFLOPS, "fallback"


class PrefillWorkload:
    """One *step* = one prefill pass: every chunk of every request is rotated, appended and attended.
    Chunks of one pass that belong to different requests run as one packed (``cu_seqlens_q``) call."""

    def __init__(self, name: str, device: torch.device, rank: int):
        from kestrel_b200.kv_cache import KVMemoryPool, PagedKVCache, PageTable
        from kestrel_b200 import kernels

        self.kernels, self.cfg, self.device = kernels, PREFILL_WORKLOADS[name], device
        cfg = self.cfg
        self.B, self.D, self.prefix, self.chunk = cfg["batch"], cfg["head_dim"], cfg["prefix"], cfg["chunk"]
        g = torch.Generator().manual_seed(2000)   # the same request lengths on every rank
        self.suffix = torch.randint(cfg["lo"], cfg["hi"] + 1, (self.B,), generator=g)
        own_pages = (self.prefix % PAGE + self.suffix + PAGE - 1) // PAGE        # pages a request writes
        shared_full = self.prefix // PAGE
        n_pages = int(own_pages.sum()) + (shared_full + 1) * (1 if name == "pf4" else self.B) + 16
        self.n_pages = int(n_pages * 1.25)
        self.pool = KVMemoryPool(device=device)
        self.pt = PageTable(n_pages=self.n_pages, page_size=PAGE, max_batch_size=self.B + 2, device=device)
        order = torch.randperm(len(self.pt.free_pages), generator=g).tolist()
        self.pt.free_pages = [self.pt.free_pages[i] for i in order]
        fp8 = cfg.get("kv") == "fp8"
        kw = dict(k_scale=[0.011] * HKV, v_scale=[0.012] * HKV) if fp8 else {}   # N(0,1) rows: absmax ~ 5 = 448 * 0.011
        self.cache = PagedKVCache(self.pt, n_heads=HKV, head_dim=self.D,
                                  dtype=torch.float8_e4m3fn if fp8 else torch.bfloat16, pool=self.pool, **kw)
        self.rows = []
        share = name == "pf4"
        owner = None
        if share:
            owner = self.pt.allocate()
            self.pt.reserve(owner, self.prefix)
            shared = list(self.pt.page_table_cpu[owner])[:shared_full]
        for b in range(self.B):
            r = self.pt.allocate()
            if share and shared_full:
                self.pt.map_pages(r, 0, shared)                 # the cached prefix pages, referenced by all
            self.pt.reserve(r, self.prefix + int(self.suffix[b]))
            self.rows.append(r)
        self.pt.commit_block_table()
        dg = torch.Generator(device=device).manual_seed(77 + rank)
        # the cached prefix (random K/V written straight into the pool pages)
        if fp8:   # codes of moderate magnitude (no NaN patterns)
            for c in (self.cache.k_cache, self.cache.v_cache):
                c.view(torch.uint8).copy_(torch.randint(0, 0x70, c.shape, generator=dg, device=device, dtype=torch.uint8)
                                          | (torch.randint(0, 2, c.shape, generator=dg, device=device, dtype=torch.uint8) << 7))
        else:
            self.cache.k_cache.copy_(torch.randn(self.cache.k_cache.shape, generator=dg, device=device, dtype=torch.bfloat16))
            self.cache.v_cache.copy_(torch.randn(self.cache.v_cache.shape, generator=dg, device=device, dtype=torch.bfloat16))
        # cos/sin table in the layout of kestrel/models/moondream/rope.py: cos of rot/2 frequencies, then sin
        inv_freq = 1.0 / (1.5e6 ** (torch.arange(0, cfg["rot"], 2, dtype=torch.float32) / cfg["rot"]))
        freqs = torch.arange(self.prefix + cfg["hi"] + 1, dtype=torch.float32).unsqueeze(1) * inv_freq
        self.table = torch.cat([freqs.cos(), freqs.sin()], dim=-1).to(device)
        # passes: chunk c of every request that still has tokens
        self.passes = []
        W = (HQ + 2 * HKV) * self.D
        n_chunks = int((int(self.suffix.max()) + self.chunk - 1) // self.chunk)
        for c in range(n_chunks):
            qlens = (self.suffix - c * self.chunk).clamp(min=0, max=self.chunk)
            live = (qlens > 0).nonzero().view(-1)
            ql = qlens[live]
            total = int(ql.sum())
            cu = torch.zeros(live.numel() + 1, dtype=torch.int32)
            cu[1:] = ql.cumsum(0)
            start = self.prefix + c * self.chunk
            pos = torch.cat([torch.arange(start, start + int(n)) for n in ql.tolist()])
            rows = torch.tensor([self.rows[i] for i in live.tolist()], dtype=torch.int64)
            row_of_tok = torch.repeat_interleave(rows, ql)
            seq_k = (start + ql).to(torch.int32)
            pairs = int((ql * start + ql * (ql + 1) // 2).sum())          # visible (query, key) pairs per head
            rows_dev = rows.to(device)
            ps = dict(
                total=total, cu=cu.to(device), max_q=int(ql.max()), pos=pos.to(device),
                slots=kernels.build_slot_mapping(self.pt.page_table, row_of_tok.to(device).view(-1, 1),
                                                 pos.to(device).view(-1, 1), PAGE).view(-1),
                page_table=self.pt.page_table[rows_dev].contiguous(), seqused_k=seq_k.to(device), pairs=pairs,
                qkv=torch.randn(total, W, generator=dg, device=device, dtype=torch.bfloat16),
                out=torch.empty(total, HQ, self.D, device=device, dtype=torch.bfloat16),
                h_qkv=torch.randn(total, W, dtype=torch.bfloat16).pin_memory(),
                h_out=torch.empty(total, HQ, self.D, dtype=torch.bfloat16).pin_memory())
            self.passes.append(ps)
        self.flops = sum(4 * self.D * HQ * ps["pairs"] for ps in self.passes)
        self.tokens = sum(ps["total"] for ps in self.passes)
        self.launches_per_step = 3 * len(self.passes)   # rope+append, plan, attention
        self.attn_bytes = sum(2 * ps["total"] * HQ * self.D * 2 for ps in self.passes)

    def _pass(self, ps, qkv, out, attn_only=False):
        q, k, v = qkv.split([HQ * self.D, HKV * self.D, HKV * self.D], dim=-1)
        q, k, v = q.unflatten(-1, (HQ, self.D)), k.unflatten(-1, (HKV, self.D)), v.unflatten(-1, (HKV, self.D))
        if not attn_only:
            self.kernels.rope_reshape_and_cache(ps["pos"], q, k, v, self.table, self.cache.k_cache.permute(0, 2, 1, 3),
                                                self.cache.v_cache.permute(0, 2, 1, 3), ps["slots"],
                                                self.cache._kv_cache_dtype, self.cache.k_scale_tensor.view(-1),
                                                self.cache.v_scale_tensor.view(-1), write_k=False)
        self.kernels.flash_attn_fwd(q, self.cache.k_cache.permute(0, 2, 1, 3), self.cache.v_cache.permute(0, 2, 1, 3),
                                    page_table=ps["page_table"], seqused_k=ps["seqused_k"], cu_seqlens_q=ps["cu"],
                                    max_seqlen_q=ps["max_q"], causal=True, out=out, k_scale=self.cache.k_scale,
                                    v_scale=self.cache.v_scale)

    def step_device(self, attn_only=False):
        for ps in self.passes:
            self._pass(ps, ps["qkv"], ps["out"], attn_only)

    def step_e2e(self):
        for ps in self.passes:
            ps["qkv"].copy_(ps["h_qkv"], non_blocking=True)
            self._pass(ps, ps["qkv"], ps["out"])
            ps["h_out"].copy_(ps["out"], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()

    def e2e_bytes(self):
        return (sum(ps["h_qkv"].numel() * 2 for ps in self.passes), sum(ps["h_out"].numel() * 2 for ps in self.passes))


def time_cpu_prefill(name: str, target_seconds: float = 12.0) -> dict:
    """The oracle (rotary, append, gather + attention in fp32 torch) on a few requests of the workload."""
    from oracle import paged_kv_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = PREFILL_WORKLOADS[name]
    D, prefix, chunk = cfg["head_dim"], cfg["prefix"], min(cfg["chunk"], cfg["hi"])
    nreq = 2
    g = torch.Generator().manual_seed(5)
    L = prefix + chunk
    pages = -(-L // PAGE)
    table = (torch.randperm(nreq * pages, generator=g) + 1).view(nreq, pages).to(torch.int32)
    kc = torch.randn(nreq * pages + 1, HKV, PAGE, D, generator=g)
    vc = torch.randn(nreq * pages + 1, HKV, PAGE, D, generator=g)
    cs = O.precompute_freqs_cis(cfg["rot"], L + 1, 1.5e6)
    q = torch.randn(nreq, chunk, HQ, D, generator=g).to(torch.bfloat16)
    k = torch.randn(nreq, chunk, HKV, D, generator=g).to(torch.bfloat16)
    v = torch.randn(nreq, chunk, HKV, D, generator=g).to(torch.bfloat16)
    pos = torch.arange(prefix, L).repeat(nreq)
    slots = O.build_slot_mapping(table, torch.arange(nreq), pos.view(nreq, chunk), PAGE).view(-1)

    def one():
        qr = O.rotary_embedding(pos, q.view(-1, HQ, D), cs).view(nreq, chunk, HQ, D)
        kr = O.rotary_embedding(pos, k.view(-1, HKV, D), cs)
        O.append(kc, vc, kr, v.view(-1, HKV, D), slots)
        return O.paged_attention(qr.float(), kc, vc, table, torch.full((nreq,), L, dtype=torch.int32))

    one()
    t0 = time.perf_counter()
    one()
    dt = time.perf_counter() - t0
    reps = max(1, min(20, int(target_seconds / max(dt, 1e-3))))
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        one()
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    flops = 4 * D * HQ * nreq * (chunk * prefix + chunk * (chunk + 1) // 2)
    return {"value": flops / med / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{nreq} requests x one {chunk}-token chunk on a {prefix}-token prefix, {reps} repetitions "
                      f"(oracle: torch CPU restatement, {cores} threads)", "tokens_per_s": nreq * chunk / med,
            "steps": reps, "ms_per_sample_step": med * 1e3}


def run_prefill(args) -> None:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = PREFILL_WORKLOADS[args.workload]
    if args.impl == "reference":
        if rank == 0:
            res = time_cpu_prefill(args.workload, 25.0)
            print(json.dumps({
                "impl": "reference", "metric": "paged append+prefill-attn TFLOP/s", "value": res["value"],
                "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": res["steps"], "warmup": args.warmup,
                "ms_per_step": res["ms_per_sample_step"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"{args.workload}: {cfg['desc']}", "timing": "host wall clock on a bounded sample"},
                "tokens_per_s": res["tokens_per_s"],
                "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": res["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}), flush=True)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the kernels have no CPU fallback)")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    from kestrel_b200 import _native
    from kestrel_b200.sharding import combine_step_stats
    _native.load()
    wl = PrefillWorkload(args.workload, device, rank)
    warm = max(3, args.warmup)

    def barrier():
        torch.cuda.synchronize(device)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    def timed(fn, n):
        for _ in range(warm):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        return e0.elapsed_time(e1)

    sampler = ClockSampler(physical_gpu_index(local))
    if rank == 0:
        sampler.start()
    ms = timed(wl.step_device, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    attn_ms = timed(lambda: wl.step_device(attn_only=True), args.steps) / args.steps
    e2e_ms = None if args.no_e2e else timed(wl.step_e2e, max(3, min(args.steps, 5)))
    flags = _native.device_status(local, clear=True)
    if flags[0] != 0:
        raise SystemExit(f"kernel diagnostics reported a problem: {flags}")
    ms_all, flops_all = combine_step_stats(ms, float(wl.flops) * args.steps, device)
    e2e_all = combine_step_stats(e2e_ms or 0.0, float(wl.flops) * max(3, min(args.steps, 5)), device)
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    peak, peak_kind = measured_bf16_peak()
    value = flops_all / (ms_all * 1e-3) / 1e12
    achieved = wl.flops / (attn_ms * 1e-3) / 1e12
    h2d, d2h = wl.e2e_bytes()
    line = {
        "metric": "paged append+prefill-attn TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": warm, "ms_per_step": ms_all / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": ("e4m3 K/V widened to f16 operands" if cfg.get("kv") == "fp8" else "bf16 operands") + ", fp32 accumulate and softmax",
        "data": "synthetic",
        "config": {"workload": f"{args.workload}: {cfg['desc']}", "passes_per_step": len(wl.passes),
                   "tokens_per_step": wl.tokens, "pool_pages": wl.n_pages, "launch": "eager",
                   "flops": "4 * head_dim * n_q_heads * visible (query, key) pairs (causal): useful work only",
                   "l2_policy": "K/V of a pass exceed L2 except the shared prefix of pf4, which is L2-resident by design"},
        "tokens_per_s": world * wl.tokens / (ms_all / args.steps * 1e-3),
        "gpu_launches": wl.launches_per_step * args.steps, "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "paged_prefill_kernel (+ its plan launch)", "achieved": achieved,
                     "peak": peak, "peak_kind": peak_kind, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": None,
                     "launch_ms_avg": attn_ms / len(wl.passes), "algorithmic_flops_per_step": wl.flops,
                     "timing": "attention calls of a step alone, CUDA events"},
    }
    if e2e_ms is not None:
        n = max(3, min(args.steps, 5))
        line["e2e"] = {"value": e2e_all[1] / (e2e_all[0] * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                       "d2h_bytes_per_step": d2h, "ms_per_step": e2e_all[0] / n, "steps": n}
    if world == 1 and not args.no_cpu_baseline:
        cb = time_cpu_prefill(args.workload)
        line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------------------
# CPU arm: the reference's own torch path where it has one (slot mapping, append), a vectorised torch
# restatement where it has none (FP8 quantise, metadata, attention), on a bounded sample of the workload
# ----------------------------------------------------------------------------------------------

def _staged_reference_kv_cache():
    """The reference's unmodified ``kestrel/kv_cache.py`` (staged under oracle/_ref by oracle/stage_reference.py)
    bound to a ``kestrel_kernels`` stub without kernels, which makes ``PagedKVCache.update`` take its torch
    path (``kestrel/kv_cache.py:216-220``).  Loaded under a private package name; None when nothing is staged."""
    import importlib
    import types
    root = ROOT / "oracle" / "_ref" / "kestrel"
    if not (root / "kv_cache.py").exists():
        return None
    saved = {k: sys.modules.get(k) for k in ("kestrel_kernels", "kestrel", "kestrel.kv_cache", "kestrel.device",
                                             "kestrel.utils", "kestrel.utils.buffers")}
    try:
        stub = types.ModuleType("kestrel_kernels")
        rt = types.SimpleNamespace(cache=types.SimpleNamespace(reshape_and_cache_flash=None, build_paged_kv_metadata=None))
        stub.get_runtime = lambda: rt
        sys.modules["kestrel_kernels"] = stub
        pkg = types.ModuleType("kestrel")
        pkg.__path__ = [str(root)]
        sys.modules["kestrel"] = pkg
        for k in ("kestrel.kv_cache", "kestrel.device", "kestrel.utils", "kestrel.utils.buffers"):
            sys.modules.pop(k, None)
        return importlib.import_module("kestrel.kv_cache")
    except Exception:
        return None
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


class CpuWorkload:
    """One layer of one decode step on ``sample_batch`` sequences drawn like the workload's.

    * slot mapping and bf16 append: the reference's own ``PageTable.build_slot_mapping`` /
      ``PagedKVCache.update`` torch path when the staged modules are present (``kind`` "reference+port"),
      else the same index arithmetic restated in torch (``kind`` "port");
    * FP8 quantise-on-append: ``(x / scale).clamp(-448, 448).to(float8_e4m3fn)`` (the reference's torch
      path refuses FP8, ``kestrel/kv_cache.py:212-215``);
    * metadata: the torch restatement of ``kestrel/models/qwen35/runtime.py:1165-1170``;
    * attention: per sequence, gather ITS pages only, dequantise with ``view(float8_e4m3fn).float()``,
      one batched matmul per product over the KV heads, fp32 softmax (the reference has no CPU attention).
    """

    def __init__(self, name: str, sample_batch: int):
        self.cfg = cfg = WORKLOADS[name]
        self.B = min(sample_batch, cfg["batch"])
        self.D, self.sq = cfg["head_dim"], cfg["sq"]
        self.fp8 = cfg["kv"] == "fp8"
        self.kv_bytes = 1 if self.fp8 else 2
        g = torch.Generator().manual_seed(1000 + (int(name[3]) if name[3].isdigit() else 6))
        prefix = cfg.get("prefix", 0)
        full = torch.randint(cfg["lo"], cfg["hi"] + 1, (cfg["batch"],), generator=g) + prefix
        self.len0 = full[: self.B]
        n_pages = int(((self.len0 + 64 + PAGE - 1) // PAGE).sum()) + 2
        self.n_pages = n_pages
        self.kc_mod = _staged_reference_kv_cache()
        kv_dtype = torch.float8_e4m3fn if self.fp8 else torch.bfloat16
        if self.kc_mod is not None:
            kc = self.kc_mod
            self.pt = kc.PageTable(n_pages=n_pages, page_size=PAGE, max_batch_size=self.B + 1, device="cpu")
            order = torch.randperm(len(self.pt.free_pages), generator=g).tolist()
            self.pt.free_pages = [self.pt.free_pages[i] for i in order]
            kw = dict(k_scale=0.2, v_scale=0.2) if self.fp8 else {}
            self.layer = kc.PagedKVCache(self.pt, n_heads=HKV, head_dim=self.D, dtype=kv_dtype,
                                         pool=kc.KVMemoryPool(device="cpu"), **kw)
            self.rows = [self.pt.allocate() for _ in range(self.B)]
            for r, L in zip(self.rows, self.len0.tolist()):
                self.pt.reserve(r, int(L) + 64)
            self.pt.commit_block_table(self.rows)
            self.table = self.pt.page_table
            self.kc, self.vc = self.layer.k_cache, self.layer.v_cache
        else:
            perm = (torch.randperm(n_pages - 1, generator=g) + 1).to(torch.int32)
            width = int(((self.len0 + 64 + PAGE - 1) // PAGE).max())
            self.table = torch.zeros(self.B + 1, width, dtype=torch.int32)
            cur = 0
            for b in range(self.B):
                n = int((self.len0[b] + 64 + PAGE - 1) // PAGE)
                self.table[b + 1, :n] = perm[cur:cur + n]
                cur += n
            self.rows = list(range(1, self.B + 1))
            self.kc = torch.zeros(n_pages, HKV, PAGE, self.D, dtype=kv_dtype)
            self.vc = torch.zeros_like(self.kc)
        shape = (n_pages, HKV, PAGE, self.D)
        if self.fp8:
            for c in (self.kc, self.vc):
                c.view(torch.uint8).copy_(torch.randint(0, 0x77, shape, generator=g, dtype=torch.uint8))
            self.ks = self.vs = 0.2
        else:
            self.kc.copy_(torch.randn(shape, generator=g).to(torch.bfloat16))
            self.vc.copy_(torch.randn(shape, generator=g).to(torch.bfloat16))
            self.ks = self.vs = 1.0
        self.batch_idx = torch.tensor(self.rows, dtype=torch.int64)
        self.q = torch.randn(self.B, self.sq, HQ, self.D, generator=g).to(torch.bfloat16)
        self.k_new = torch.randn(self.B, self.sq, HKV, self.D, generator=g).to(torch.bfloat16)
        self.v_new = torch.randn(self.B, self.sq, HKV, self.D, generator=g).to(torch.bfloat16)
        self.meta_pt = torch.zeros(self.B, self.table.shape[1], dtype=torch.int32)
        self.meta_sk = torch.zeros(self.B, dtype=torch.int32)
        self.out = torch.empty(self.B, self.sq, HQ, self.D, dtype=torch.bfloat16)
        self.step_no = 0

    @property
    def kind(self) -> str:
        return "reference+port" if self.kc_mod is not None else "port"

    def lengths_after(self, step_no: int) -> torch.Tensor:
        return self.len0 + (step_no % 8 + 1) * self.sq

    def _slot_mapping(self, pos: torch.Tensor) -> torch.Tensor:
        if self.kc_mod is not None:
            return self.pt.build_slot_mapping(self.batch_idx, pos)
        page = self.table[self.batch_idx.view(-1, 1).expand_as(pos).reshape(-1), (pos // PAGE).reshape(-1)]
        return (page.to(torch.int64) * PAGE + (pos % PAGE).reshape(-1)).view_as(pos)

    def _append(self, pos: torch.Tensor, slots: torch.Tensor) -> None:
        if self.fp8:
            flat = slots.reshape(-1)
            kq = (self.k_new.float() / self.ks).clamp(-448, 448).to(torch.float8_e4m3fn).view(-1, HKV, self.D)
            vq = (self.v_new.float() / self.vs).clamp(-448, 448).to(torch.float8_e4m3fn).view(-1, HKV, self.D)
            kview = self.kc.view(torch.uint8).permute(0, 2, 1, 3)
            vview = self.vc.view(torch.uint8).permute(0, 2, 1, 3)
            kview[flat // PAGE, flat % PAGE] = kq.view(torch.uint8)
            vview[flat // PAGE, flat % PAGE] = vq.view(torch.uint8)
        elif self.kc_mod is not None:
            self.layer.update(input_pos=pos, k_val=self.k_new, v_val=self.v_new, slot_mapping=slots)
        else:
            flat = slots.reshape(-1)
            self.kc.permute(0, 2, 1, 3)[flat // PAGE, flat % PAGE] = self.k_new.view(-1, HKV, self.D)
            self.vc.permute(0, 2, 1, 3)[flat // PAGE, flat % PAGE] = self.v_new.view(-1, HKV, self.D)

    def _metadata(self, pos: torch.Tensor) -> None:
        self.meta_sk.copy_(pos[:, -1].to(torch.int32) + 1)
        self.meta_pt.copy_(self.table[self.batch_idx])      # the restatement copies whole rows

    def _attention(self) -> None:
        group = HQ // HKV
        scale = 1.0 / math.sqrt(self.D)
        for b in range(self.B):
            L = int(self.meta_sk[b])
            pages = self.meta_pt[b, : -(-L // PAGE)].to(torch.int64)
            K = self.kc[pages].float().permute(1, 0, 2, 3).reshape(HKV, -1, self.D)[:, :L]      # [H_kv, L, D]
            V = self.vc[pages].float().permute(1, 0, 2, 3).reshape(HKV, -1, self.D)[:, :L]
            q = self.q[b].float().view(self.sq, HKV, group, self.D).permute(1, 0, 2, 3).reshape(HKV, self.sq * group, self.D)
            s = torch.matmul(q, K.transpose(1, 2)) * (scale * self.ks)                           # [H_kv, sq*g, L]
            if self.sq > 1:
                j = torch.arange(self.sq).repeat_interleave(group).view(1, -1, 1)
                s = s.masked_fill(torch.arange(L).view(1, 1, L) > (L - self.sq + j), float("-inf"))
            o = torch.matmul(torch.softmax(s, dim=-1), V) * self.vs                              # [H_kv, sq*g, D]
            self.out[b] = o.view(HKV, self.sq, group, self.D).permute(1, 0, 2, 3).reshape(self.sq, HQ, self.D).to(torch.bfloat16)

    def step(self) -> None:
        t = self.step_no % 8
        pos = (self.len0 + t * self.sq).view(-1, 1) + torch.arange(self.sq).view(1, -1)
        slots = self._slot_mapping(pos)
        self._append(pos, slots)
        self._metadata(pos)
        self._attention()
        self.step_no += 1

    def matmul_bound_seconds(self) -> float:
        """Time of the two batched matmuls alone on operands of this sample's shapes that are already
        gathered and fp32: what a torch CPU attention cannot beat on these cores."""
        group = HQ // HKV
        lens = self.lengths_after(0).tolist()
        ops = [(torch.randn(HKV, self.sq * group, self.D), torch.randn(HKV, int(L), self.D)) for L in lens]
        best = float("inf")
        for _ in range(3):
            t0 = time.perf_counter()
            for q, K in ops:
                s = torch.matmul(q, K.transpose(1, 2))
                torch.matmul(s, K)
            best = min(best, time.perf_counter() - t0)
        return best


def time_cpu(name: str, steps: int, warmup: int, target_seconds: float = 12.0) -> dict:
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = WORKLOADS[name]
    w = CpuWorkload(name, 8)
    for _ in range(max(1, min(warmup, 2))):
        w.step()
    t0 = time.perf_counter()
    w.step()
    one = time.perf_counter() - t0
    reps = max(3, min(max(steps, 3), int(target_seconds / max(one, 1e-3))))
    times = []
    byts = []
    for _ in range(reps):
        n = w.step_no
        t0 = time.perf_counter()
        w.step()
        times.append(time.perf_counter() - t0)
        byts.append(algorithmic_bytes(w.lengths_after(n), layers=1, kv_bytes=w.kv_bytes, head_dim=w.D, sq=w.sq,
                                      batch=w.B)["per_step"])
    med = statistics.median(times)
    gbs = statistics.median(byts) / med / 1e9
    bound = w.matmul_bound_seconds()
    return {"value": gbs, "unit": "GB/s", "cores": cores, "kind": w.kind,
            "sample": f"{w.B} of {cfg['batch']} sequences, 1 of {cfg['layers']} layers, {reps} steps; "
                      + ("slot mapping" + ("" if w.fp8 else " and append") + " by the reference's own torch path, "
                         if w.kc_mod is not None else "")
                      + f"{'FP8 quantise, ' if w.fp8 else ''}metadata and attention as vectorised torch, {cores} threads",
            "ms_per_sample_step": med * 1e3, "tokens_per_s": w.B * w.sq / med / cfg["layers"],
            "matmul_bound_gbs": statistics.median(byts) / bound / 1e9, "steps": reps}


def run_reference_arm(args) -> None:
    """``--impl reference``: the CPU arm alone (rank 0 only; other ranks exit without work)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    res = time_cpu(args.workload, args.steps, args.warmup, target_seconds=25.0)
    cfg = WORKLOADS[args.workload]
    line = {
        "impl": "reference", "metric": "paged append+decode-attn HBM GB/s", "value": res["value"], "unit": "GB/s",
        "n_gpus": args.gpus, "steps": res["steps"], "warmup": args.warmup, "ms_per_step": res["ms_per_sample_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": cfg["kv"], "data": "synthetic",
        "config": {"workload": f"{args.workload}: {cfg['desc']}", "timing": "host wall clock on a bounded sample"},
        "tokens_per_s": res["tokens_per_s"],
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample", "matmul_bound_gbs")},
        "e2e": {"value": res["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# yardstick arm: a library kernel on the same pools (not the reference, not on any product path)
# ----------------------------------------------------------------------------------------------

def _timed(fn, reps: int, device) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize(device)
    return e0.elapsed_time(e1) / reps


def _page_lists(rows_pages, lengths, device):
    """flashinfer's CSR description of the page lists: indptr, indices, tokens in the last page."""
    indptr, indices = [0], []
    for pages, L in zip(rows_pages, lengths):
        n = -(-int(L) // PAGE)
        indices.extend(pages[:n])
        indptr.append(len(indices))
    last = [(int(L) - 1) % PAGE + 1 for L in lengths]
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
    return t(indptr), t(indices), t(last)


def run_yardstick(args) -> None:
    """``--impl flashinfer``: the image's flashinfer paged attention (decode or prefill wrapper, HND layout)
    timed on the pools, page lists and queries of our arm, attention calls only, next to ours.  One GPU."""
    import flashinfer
    from kestrel_b200 import _native
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    ws = torch.empty(512 << 20, dtype=torch.uint8, device=device)
    if args.workload in PREFILL_WORKLOADS:
        wl = PrefillWorkload(args.workload, device, 0)
        if wl.cache.quantized:
            raise SystemExit("the prefill yardstick covers the 16-bit workloads")
        wl.step_device()                                   # fills the pools with the chunks' K/V
        ours_ms = _timed(lambda: wl.step_device(attn_only=True), max(3, args.steps), device)
        calls = []
        for ps in wl.passes:
            lens = ps["seqused_k"].tolist()
            indptr, indices, last = _page_lists(ps["page_table"].tolist(), lens, device)
            w = flashinfer.BatchPrefillWithPagedKVCacheWrapper(ws, "HND")
            w.plan(ps["cu"], indptr, indices, last, HQ, HKV, wl.D, PAGE, causal=True,
                   q_data_type=torch.bfloat16, kv_data_type=torch.bfloat16)
            q = ps["qkv"][:, :HQ * wl.D].unflatten(-1, (HQ, wl.D)).contiguous()
            calls.append((w, q))
        kv = (wl.cache.k_cache, wl.cache.v_cache)
        their_ms = _timed(lambda: [w.run(q, kv) for w, q in calls], max(3, args.steps), device)
        work, unit = wl.flops / 1e12, "TFLOP/s"
        per = "all attention calls of a step"
    else:
        wl = GpuWorkload(args.workload, device, 0, args.warmup + 6, share_prefix=False)
        for _ in range(max(1, args.warmup)):
            wl.step_device()
        ours_ms = wl.time_attention_launch(max(3, args.steps))
        lens = wl.lengths_after(wl.step_no - 1).tolist()
        indptr, indices, last = _page_lists([wl.pt.page_table_cpu[r] for r in wl.rows], lens, device)
        cache = wl.caches[0]
        fp8 = cache.quantized
        kw = dict(k_scale=float(cache.k_scale_tensor.view(-1)[0]), v_scale=float(cache.v_scale_tensor.view(-1)[0])) if fp8 else {}
        kv = (cache.k_cache, cache.v_cache)
        if wl.sq == 1:
            w = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws, "HND", use_tensor_cores=True)
            w.plan(indptr, indices, last, HQ, HKV, wl.D, PAGE, q_data_type=torch.bfloat16, kv_data_type=cache.k_cache.dtype)
            q = wl.q[0].view(wl.B, HQ, wl.D)
        else:
            w = flashinfer.BatchPrefillWithPagedKVCacheWrapper(ws, "HND")
            qo = torch.arange(0, (wl.B + 1) * wl.sq, wl.sq, dtype=torch.int32, device=device)
            w.plan(qo, indptr, indices, last, HQ, HKV, wl.D, PAGE, causal=True, q_data_type=torch.bfloat16,
                   kv_data_type=cache.k_cache.dtype)
            q = wl.q[0].view(wl.B * wl.sq, HQ, wl.D)
        their_ms = _timed(lambda: w.run(q, kv, **kw), max(3, args.steps), device)
        work = algorithmic_bytes(wl.lengths_after(wl.step_no - 1), layers=wl.layers_n, kv_bytes=wl.kv_bytes,
                                 head_dim=wl.D, sq=wl.sq, batch=wl.B)["attn_per_launch"] / 1e9
        unit, per = "GB/s", "one attention call (one layer)"
    flags = _native.device_status(0, clear=True)
    print(json.dumps({
        "impl": "flashinfer", "version": flashinfer.__version__, "metric": f"paged attention, {per}",
        "value": work / (their_ms * 1e-3), "unit": unit, "ms": their_ms,
        "ours": {"value": work / (ours_ms * 1e-3), "unit": unit, "ms": ours_ms},
        "n_gpus": 1, "config": {"workload": args.workload}, "device_status": list(flags),
        "note": "library kernel as a yardstick on the same pools and page lists; not the reference implementation",
    }), flush=True)


def unique_kv_tokens(wl, lengths_after: torch.Tensor) -> int:
    """KV tokens a step must fetch from HBM at least once: pages shared by the whole batch count once."""
    shared = wl.shared_tokens
    return int(lengths_after.sum()) - (wl.B - 1) * shared if shared else int(lengths_after.sum())


def measure_decode(name: str, args, device, rank: int, world: int, dist, *, steps: int, e2e_steps: int) -> dict | None:
    """Builds the workload, times ``steps`` steps (CUDA events, graph replay unless --no-graph), the attention
    calls alone (roofline) and ``e2e_steps`` steps through the public API with host buffers.  Every rank runs
    it; rank 0 gets the record, the others None."""
    from kestrel_b200 import _native
    local = device.index
    cfg = WORKLOADS[name]
    global HQ, HKV, PAGE
    saved_geometry = (HQ, HKV, PAGE)
    if "heads" in cfg:
        HQ, HKV = cfg["heads"]
    if "page" in cfg:
        PAGE = cfg["page"]
    try:
        return _measure_decode(name, cfg, args, device, rank, world, dist, steps=steps, e2e_steps=e2e_steps)
    finally:
        HQ, HKV, PAGE = saved_geometry


def _measure_decode(name: str, cfg: dict, args, device, rank: int, world: int, dist, *, steps: int, e2e_steps: int) -> dict | None:
    from kestrel_b200 import _native
    local = device.index
    warm = max(3, args.warmup)
    total_steps = 3 * warm + steps + e2e_steps + 4
    wl = GpuWorkload(name, device, rank, total_steps, share_prefix=not args.no_shared_prefix)

    def barrier():
        torch.cuda.synchronize(device)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    use_graph = not args.no_graph
    for _ in range(warm):
        wl.step_device()
    if use_graph:
        wl.capture_graph()
        wl.step_graph()   # one untimed replay (the graph continues where the eager warm-up stopped)
    step_fn = wl.step_graph if use_graph else wl.step_device
    barrier()
    sampler = ClockSampler(physical_gpu_index(local))
    if rank == 0:
        sampler.start()
    first_step = wl.step_no
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        step_fn()
    stop.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    elapsed_ms = start.elapsed_time(stop)
    ab = lambda lens: algorithmic_bytes(lens, layers=wl.layers_n, kv_bytes=wl.kv_bytes, head_dim=wl.D, sq=wl.sq, batch=wl.B)
    total_bytes = sum(ab(wl.lengths_after(first_step + i))["per_step"] for i in range(steps))
    # roofline of the dominant kernel: the attention calls alone, at the lengths of the last step
    attn_reps = max(3, min(200, int(400 / max(0.05, elapsed_ms / steps))))
    attn_avg_ms = wl.time_attention_launch(attn_reps)
    last = wl.lengths_after(wl.step_no - 1)
    attn_bytes = ab(last)["attn_per_launch"]
    tok_bytes = 2 * HKV * wl.D * wl.kv_bytes
    attn_unique = attn_bytes - (int(last.sum()) - unique_kv_tokens(wl, last)) * tok_bytes
    step_unique = ab(last)["per_step"] - wl.layers_n * (attn_bytes - attn_unique)

    e2e = None
    if e2e_steps:
        for _ in range(warm):
            wl.step_e2e()
        barrier()
        first_e2e = wl.step_no
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(e2e_steps):
            wl.step_e2e()
        t1.record()
        barrier()
        e2e = (t0.elapsed_time(t1), sum(ab(wl.lengths_after(first_e2e + i))["per_step"] for i in range(e2e_steps)))

    flags = _native.device_status(local, clear=True)
    if flags[0] != 0:
        raise SystemExit(f"kernel diagnostics reported a problem in {name}: {flags}")

    # whole job: every rank's bytes over the slowest rank's time; per-rank figures alongside
    from kestrel_b200.sharding import gather_rank_stats, whole_job_rate
    per = gather_rank_stats([elapsed_ms, total_bytes, e2e[0] if e2e else 0.0, e2e[1] if e2e else 0.0], device)
    h2d, d2h = wl.e2e_bytes()
    launches = wl.launches_per_step * steps
    n_pools, n_pages, shared_pages, layers_n, B, sq, D = wl.n_pools, wl.n_pages, wl.shared_pages, wl.layers_n, wl.B, wl.sq, wl.D
    kv_bytes = wl.kv_bytes
    step_fn = ab = None   # (both hold the workload)
    del wl
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    if rank != 0:
        return None

    peak, peak_kind = measured_hbm_peak()
    ms_all, rate_all, own_rates = whole_job_rate(per[:, 0], per[:, 1])
    value = rate_all / 1e9
    ms_per_step = ms_all / steps
    logical = attn_bytes / (attn_avg_ms * 1e-3) / 1e9
    achieved = attn_unique / (attn_avg_ms * 1e-3) / 1e9
    traffic = dram_traffic_ratio(split_kv_kernel_name(cfg), cfg["kv"])
    if "traffic_profile" in cfg:   # (a capture of this very geometry)
        traffic = dram_traffic_ratio(split_kv_kernel_name(cfg), cfg["kv"], rel=cfg["traffic_profile"])
    rec = {
        "value": value, "unit": "GB/s", "ms_per_step": ms_per_step, "steps": steps,
        "tokens_per_s": world * B * sq / (ms_per_step * 1e-3),
        "pct_of_8TBps": 100.0 * value / world / NOMINAL_HBM_GBS, "pct_of_measured_hbm": 100.0 * value / world / peak,
        "bytes_per_step_per_gpu": float(per[0, 1]) / steps,
        "per_rank": [{"ms_per_step": float(r[0]) / steps, "gbs": g / 1e9} for r, g in zip(per, own_rates)],
        "dtype": "fp8_e4m3 KV, bf16 q/out, f16 mma, fp32 softmax" if cfg["kv"] == "fp8" else "bf16",
        "config": {"workload": f"{name}: {cfg['desc']}", "n_layer_pools": n_pools, "layers": layers_n,
                   "pool_pages": n_pages, "sequences_per_gpu": B, "context_lengths": "same draw on every rank",
                   "launch": "CUDA graph replay" if use_graph else "eager", "shared_prefix_pages": shared_pages,
                   "l2_policy": "inputs larger than L2 (every layer streams a multi-GB pool)"
                   if n_pages * HKV * PAGE * D * kv_bytes * 2 > 256e6 else
                   "working set near L2 size; see tokens/s rather than GB/s"},
        "gpu_launches": launches, "clocks": clocks,
        "roofline": {"bound": "hbm",
                     "kernel": split_kv_kernel_name(cfg) + (" (no merge launch" if split_kv_kernel_name(cfg) == "paged_prefill_kernel" else " (+ its merge launch") + (", the prefix pass on paged_prefill_kernel" if shared_pages else "") + ")",
                     "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None if traffic["ratio"] is None else traffic["ratio"] * attn_unique,
                     "traffic_source": f"{traffic['profile']}: ncu dram__bytes_read+write of a reduced launch of the same "
                                       "kernel over its algorithmic bytes, scaled by tokens",
                     "traffic_profile_stale": traffic["stale"],
                     "launch_ms_avg": attn_avg_ms, "algorithmic_bytes_per_launch": attn_unique,
                     "timing": f"graph of {layers_n} attention calls replayed {attn_reps}x, CUDA events"},
    }
    if shared_pages:
        rec["unique_bytes_per_step"] = step_unique
        rec["unique_gbs"] = step_unique / (ms_per_step * 1e-3) / 1e9
        rec["roofline"]["logical_bytes_per_launch"] = attn_bytes
        rec["roofline"]["logical_gbs"] = logical
        rec["roofline"]["bytes"] = ("unique: the pages every request shares are counted once per launch, which is how "
                                    "often the kernel reads them; `value` counts them once per request (logical bytes)")
    if e2e is not None:
        e_ms, e_rate, _ = whole_job_rate(per[:, 2], per[:, 3])
        rec["e2e"] = {"value": e_rate / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                      "d2h_bytes_per_step": d2h, "ms_per_step": e_ms / e2e_steps, "steps": e2e_steps,
                      "tokens_per_s": world * B * sq / (e_ms / e2e_steps * 1e-3)}
    return rec


def measure_prefill_record(name: str, args, device, rank: int, world: int, dist) -> dict | None:
    """Sub-record of a prefill workload (compute-bound mode of the same op), timed like run_prefill."""
    from kestrel_b200 import _native
    wl = PrefillWorkload(name, device, rank)
    warm = max(3, args.warmup)
    steps = max(args.steps, 10)

    def timed(fn, n):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize(device)
        if dist is not None:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize(device)
        return e0.elapsed_time(e1) / n

    ms = timed(wl.step_device, steps)
    attn_ms = timed(lambda: wl.step_device(attn_only=True), steps)
    flags = _native.device_status(device.index, clear=True)
    if flags[0] != 0:
        raise SystemExit(f"kernel diagnostics reported a problem in {name}: {flags}")
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    flops, tokens, n_pass = wl.flops, wl.tokens, len(wl.passes)
    del wl
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    peak, peak_kind = measured_bf16_peak()
    ms_all = t.item()
    return {"metric": "paged append+prefill-attn TFLOP/s", "value": world * flops / (ms_all * 1e-3) / 1e12, "unit": "TFLOP/s",
            "ms_per_step": ms_all, "steps": steps, "tokens_per_s": world * tokens / (ms_all * 1e-3),
            "config": {"workload": f"{name}: {PREFILL_WORKLOADS[name]['desc']}", "passes_per_step": n_pass},
            "roofline": {"bound": "tensor", "kernel": "paged_prefill_kernel", "achieved": flops / (attn_ms * 1e-3) / 1e12,
                         "peak": peak, "peak_kind": peak_kind, "unit": "TFLOP/s",
                         "frac": flops / (attn_ms * 1e-3) / 1e12 / peak, "traffic": None,
                         "launch_ms_avg": attn_ms / n_pass, "algorithmic_flops_per_step": flops,
                         "timing": "attention calls of a step alone, CUDA events"}}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg3", choices=sorted(WORKLOADS) + sorted(PREFILL_WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "flashinfer"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch the timed steps eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-shared-prefix", action="store_true",
                    help="cfg4: read the cached prefix once per request (plain calls) instead of once per batch")
    ap.add_argument("--only", action="store_true",
                    help="measure the named workload alone (no `workloads` map with the other configurations)")
    ap.add_argument("--page-size", type=int, default=0, help="override the page size of the pools (default 16)")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch (profiling on a small case)")
    ap.add_argument("--layers", type=int, default=0, help="override the workload's layer count (profiling)")
    args = ap.parse_args()
    if args.page_size:
        global PAGE
        PAGE = args.page_size
        args.only = True
        for table in (WORKLOADS, PREFILL_WORKLOADS):
            for cfg in table.values():
                cfg["desc"] = cfg["desc"].replace("page 16", f"page {PAGE}")
    if args.impl == "flashinfer":
        run_yardstick(args)
        return
    if args.workload in PREFILL_WORKLOADS:
        run_prefill(args)
        return
    if args.batch or args.layers:
        args.only = True
        WORKLOADS[args.workload] = dict(WORKLOADS[args.workload])
        if args.batch:
            WORKLOADS[args.workload]["batch"] = args.batch
        if args.layers:
            WORKLOADS[args.workload]["layers"] = args.layers
        WORKLOADS[args.workload]["desc"] += f" [reduced for profiling: batch={WORKLOADS[args.workload]['batch']}, layers={WORKLOADS[args.workload]['layers']}]"
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.warmup < 3:
        args.warmup = 3

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the kernels have no CPU fallback)")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    from kestrel_b200 import _native
    _native.load()
    e2e_steps = 0 if args.no_e2e else max(3, min(args.steps, 5))
    head = measure_decode(args.workload, args, device, rank, world, dist, steps=args.steps, e2e_steps=e2e_steps)

    # the other configurations, same process, same box: sub-records under "workloads"
    extra = {}
    if not args.only:
        for name in ("cfg5", "cfg5_sq8", "cfg2", "cfg4", "ref_mha64_p1"):
            if name == args.workload:
                continue
            one_layer = WORKLOADS[name]["layers"] == 1
            rec = measure_decode(name, args, device, rank, world, dist, steps=max(args.steps, 50) if one_layer else args.steps,
                                 e2e_steps=0 if args.no_e2e else 3)
            if rec is not None:
                rec.pop("clocks", None)
                extra[name] = rec
        for name in ("pf_long", "pf_long_fp8", "pf4"):
            rec = measure_prefill_record(name, args, device, rank, world, dist)
            if rec is not None:
                extra[name] = rec
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    line = {"metric": "paged append+decode-attn HBM GB/s", "value": head["value"], "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": head["dtype"], "data": "synthetic"}
    for k in ("config", "tokens_per_s", "pct_of_8TBps", "pct_of_measured_hbm", "bytes_per_step_per_gpu", "per_rank",
              "gpu_launches", "clocks", "roofline", "e2e", "unique_bytes_per_step", "unique_gbs"):
        if k in head:
            line[k] = head[k]
    if extra:
        line["workloads"] = extra
        line["gpu_launches"] += sum(r.get("gpu_launches", 0) for r in extra.values())
    if world == 1 and not args.no_cpu_baseline:
        cb = time_cpu(args.workload, steps=50, warmup=1)
        line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample", "tokens_per_s", "matmul_bound_gbs")}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
