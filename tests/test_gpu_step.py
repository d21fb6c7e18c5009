"""Whole hot-path steps on the GPU through the public API (page table -> slot mapping -> append ->
metadata -> attention), shaped like the five benchmark configurations, checked against the oracle."""

import math

import pytest
import torch

from kestrel_b200 import _native
from kestrel_b200.attention import paged_attention
from kestrel_b200.kv_cache import KVMemoryPool, PagedKVCache, PageTable, copy_kv_pages
from oracle import paged_kv_oracle as O
from test_gpu_attention import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _clean_status():
    _native.device_status(torch.cuda.current_device(), clear=True)
    yield
    flags = _native.device_status(torch.cuda.current_device(), clear=True)
    assert flags[0] == 0, f"kernel diagnostics: {flags}"


class Stack:
    """n_layers paged caches on one page table, with fp32 CPU mirrors driven by the oracle."""

    def __init__(self, *, n_layers, n_pages, page_size, max_batch, hq, hkv, dim, dtype, kv_dtype=None, seed=0,
                 prefix_cache=None):
        self.g = torch.Generator().manual_seed(seed)
        self.hq, self.hkv, self.dim, self.P, self.dtype = hq, hkv, dim, page_size, dtype
        self.kv_dtype = kv_dtype or dtype
        self.pool = KVMemoryPool(device=DEV)
        self.pt = PageTable(n_pages=n_pages, page_size=page_size, max_batch_size=max_batch, device=DEV,
                            prefix_cache=prefix_cache)
        self.scales = []
        self.layers = []
        for l in range(n_layers):
            kw = {}
            if self.kv_dtype == torch.float8_e4m3fn:
                ks = (torch.rand(hkv, generator=self.g) * 0.02 + 0.01).tolist()
                vs = (torch.rand(hkv, generator=self.g) * 0.02 + 0.01).tolist()
                kw = dict(k_scale=ks, v_scale=vs)
                self.scales.append((torch.tensor(ks), torch.tensor(vs)))
            else:
                self.scales.append((None, None))
            self.layers.append(PagedKVCache(self.pt, n_heads=hkv, head_dim=dim, dtype=self.kv_dtype, pool=self.pool, **kw))
        mirror_dtype = torch.uint8 if self.kv_dtype == torch.float8_e4m3fn else torch.float32
        self.mk = [torch.zeros(n_pages, hkv, page_size, dim, dtype=mirror_dtype) for _ in range(n_layers)]
        self.mv = [torch.zeros(n_pages, hkv, page_size, dim, dtype=mirror_dtype) for _ in range(n_layers)]
        width = n_pages
        self.meta_pt = torch.zeros(max_batch, width, dtype=torch.int32, device=DEV)
        self.meta_sk = torch.zeros(max_batch, dtype=torch.int32, device=DEV)

    def rand(self, *shape):
        return torch.randn(*shape, generator=self.g).to(self.dtype)

    def step(self, rows, positions, shared_prefix_pages=0):
        """Append ``positions [B, S]`` new tokens for page-table rows ``rows`` and attend; returns max error."""
        B, S = positions.shape
        self.pt.commit_block_table(rows)
        batch_idx = torch.tensor(rows, dtype=torch.int64, device=DEV)
        pos_dev = positions.to(DEV)
        slots = self.pt.build_slot_mapping(batch_idx, pos_dev)
        self.pt.populate_paged_kv_metadata(batch_idx=batch_idx, input_pos=pos_dev[:, -1].to(torch.int32).contiguous(),
                                           out_page_table=self.meta_pt[:B], out_seqused_k=self.meta_sk[:B])
        table_cpu = self.pt._page_table_cpu_tensor.clone()
        slots_ref = O.build_slot_mapping(table_cpu, torch.tensor(rows), positions, self.P)
        assert torch.equal(slots.cpu(), slots_ref)
        ref_pt = torch.zeros(B, table_cpu.shape[1], dtype=torch.int32)
        ref_sk = torch.zeros(B, dtype=torch.int32)
        O.build_paged_kv_metadata(table_cpu, torch.tensor(rows), positions[:, -1], ref_pt, ref_sk, self.P)
        assert torch.equal(self.meta_sk[:B].cpu(), ref_sk)
        outs = []
        for l, layer in enumerate(self.layers):
            fused = self.rand(B, S, (self.hq + 2 * self.hkv) * self.dim).to(DEV)
            q, k, v = fused.split([self.hq * self.dim, self.hkv * self.dim, self.hkv * self.dim], dim=-1)
            q = q.view(B, S, self.hq, self.dim)
            k = k.view(B, S, self.hkv, self.dim)
            v = v.view(B, S, self.hkv, self.dim)
            layer.update(pos_dev, k, v, slot_mapping=slots)
            out = paged_attention(q.transpose(1, 2), paged_kv_layer=layer, page_table=self.meta_pt[:B],
                                  paged_kv_seqlens_k=self.meta_sk[:B], scaling=1.0 / math.sqrt(self.dim),
                                  shared_prefix_pages=shared_prefix_pages)
            ks, vs = self.scales[l]
            O.append(self.mk[l], self.mv[l], k.cpu().reshape(B * S, self.hkv, self.dim),
                     v.cpu().reshape(B * S, self.hkv, self.dim), slots_ref, k_scale=ks, v_scale=vs)
            want = O.paged_attention(q.cpu().float(), self.mk[l], self.mv[l], ref_pt, ref_sk, k_scale=ks, v_scale=vs)
            assert_close(out, want, f"layer {l}")
            outs.append(out)
        return outs

    def check_pools_bit_exact(self):
        for l, layer in enumerate(self.layers):
            if self.kv_dtype == torch.float8_e4m3fn:
                got_k, got_v = layer.k_cache.view(torch.uint8).cpu(), layer.v_cache.view(torch.uint8).cpu()
                assert torch.equal(got_k[1:], self.mk[l][1:]) and torch.equal(got_v[1:], self.mv[l][1:])
            else:
                assert torch.equal(layer.k_cache.float().cpu()[1:], self.mk[l][1:])
                assert torch.equal(layer.v_cache.float().cpu()[1:], self.mv[l][1:])


def _prefill(stack, rows, lengths, chunk=128, slack=8):
    """Append-prefill every row in ``chunk``-token pieces (single-row calls, Sq <= 16 per attention call
    is not needed here: only the append is exercised, attention is checked in the decode steps)."""
    for row, L in zip(rows, lengths):
        stack.pt.reserve(row, L + slack)
    stack.pt.commit_block_table(rows)
    for row, L in zip(rows, lengths):
        for start in range(0, L, chunk):
            n = min(chunk, L - start)
            pos = torch.arange(start, start + n).view(1, n)
            slots = stack.pt.build_slot_mapping(torch.tensor([row], device=DEV), pos.to(DEV))
            slots_ref = O.build_slot_mapping(stack.pt._page_table_cpu_tensor, torch.tensor([row]), pos, stack.P)
            assert torch.equal(slots.cpu(), slots_ref)
            for l, layer in enumerate(stack.layers):
                k = stack.rand(1, n, stack.hkv, stack.dim).to(DEV)
                v = stack.rand(1, n, stack.hkv, stack.dim).to(DEV)
                layer.update(pos.to(DEV), k, v, slot_mapping=slots)
                ks, vs = stack.scales[l]
                O.append(stack.mk[l], stack.mv[l], k.cpu()[0], v.cpu()[0], slots_ref, k_scale=ks, v_scale=vs)


def test_config1_shape_decode_steps():
    """4 sequences, contexts U[1,512], 32/8 heads, D=64, page 16, pool of 256 pages; 3 decode steps."""
    st = Stack(n_layers=1, n_pages=256, page_size=16, max_batch=6, hq=32, hkv=8, dim=64, dtype=torch.bfloat16, seed=1000)
    lengths = torch.randint(1, 513, (4,), generator=st.g).tolist()
    rows = [st.pt.allocate() for _ in lengths]
    _prefill(st, rows, lengths)
    for step in range(3):
        st.step(rows, torch.tensor([[L + step] for L in lengths]))
    st.check_pools_bit_exact()


def test_config3_shape_fp8_layers_small_batch():
    """FP8 e4m3 KV with per-(layer, head) scales, quantise-on-append, 3 layers, 6 sequences."""
    st = Stack(n_layers=3, n_pages=600, page_size=16, max_batch=8, hq=32, hkv=8, dim=128, dtype=torch.bfloat16,
               kv_dtype=torch.float8_e4m3fn, seed=1003)
    lengths = [1500, 17, 640, 1, 2047, 333]
    rows = [st.pt.allocate() for _ in lengths]
    _prefill(st, rows, lengths, chunk=512)
    for step in range(2):
        st.step(rows, torch.tensor([[L + step] for L in lengths]))
    st.check_pools_bit_exact()


def test_config5_shape_four_token_verify():
    """Each step appends 4 draft tokens per sequence and runs 4-query causal attention, 2 layers."""
    st = Stack(n_layers=2, n_pages=400, page_size=16, max_batch=8, hq=32, hkv=8, dim=128, dtype=torch.bfloat16, seed=1005)
    lengths = [900, 30, 1234, 61, 512]
    rows = [st.pt.allocate() for _ in lengths]
    _prefill(st, rows, lengths, chunk=512)
    for step in range(2):
        pos = torch.tensor([[L + 4 * step + j for j in range(4)] for L in lengths])
        st.step(rows, pos)
    st.check_pools_bit_exact()


def test_config4_shape_shared_prefix_with_cow():
    """One 729-token image prefix (45 full pages + 9 tokens) cached in the radix tree and reused by
    every request: the full pages are shared, the partly filled 46th page is copied on write before
    each request's first private token; then decode steps.  The oracle sees the same page table and
    the same appends, so pool contents must match bit for bit and attention within tolerance."""
    from kestrel_b200.prefix_cache import ImageToken, PagedRadixCache, attach_cached_prefix

    n_req, P, hq, hkv, D = 20, 16, 32, 8, 64
    prefix = 729
    cache = PagedRadixCache(page_size=P)
    st = Stack(n_layers=2, n_pages=900, page_size=P, max_batch=n_req + 2, hq=hq, hkv=hkv, dim=D, dtype=torch.bfloat16,
               seed=1004, prefix_cache=cache)
    suffix = torch.randint(32, 257, (n_req,), generator=st.g).tolist()
    image = [ImageToken(content_hash=42, kv_length_=prefix)]
    owner = st.pt.allocate()
    _prefill(st, [owner], [prefix], chunk=128, slack=0)
    shared = list(st.pt.page_table_cpu[owner])
    assert len(shared) == 46
    assert cache.insert(image, shared).inserted_pages == 46
    rows = []
    for i, s in enumerate(suffix):
        r = st.pt.allocate()

        class Text:  # request-specific suffix tokens
            def __init__(self, k): self.k = k
            def cache_key(self): return (0, i, self.k)
            def kv_length(self): return 1

        prompt = image + [Text(k) for k in range(s)]
        skip, n_shared, match = attach_cached_prefix(st.pt, cache, r, prompt, prefix + s)
        assert (skip, n_shared, match.partial_page_tokens) == (prefix, 45, 9)
        cache.unlock_prefill(match.last_node)
        rows.append(r)
    src_pages, dst_pages = st.pt.take_pending_page_copies()
    assert len(dst_pages) == n_req
    copy_kv_pages(st.layers, src_pages, dst_pages)
    for l in range(len(st.layers)):
        O.copy_pages([st.mk[l], st.mv[l]], src_pages, dst_pages)
    # private suffixes, appended in 128-token chunks starting inside the copied page
    for r, s in zip(rows, suffix):
        st.pt.reserve(r, prefix + s + 8)
    st.pt.commit_block_table(rows)
    for r, s in zip(rows, suffix):
        for start in range(prefix, prefix + s, 128):
            n = min(128, prefix + s - start)
            pos = torch.arange(start, start + n).view(1, n)
            slots = st.pt.build_slot_mapping(torch.tensor([r], device=DEV), pos.to(DEV))
            slots_ref = O.build_slot_mapping(st.pt._page_table_cpu_tensor, torch.tensor([r]), pos, P)
            for l, layer in enumerate(st.layers):
                k = st.rand(1, n, hkv, D).to(DEV)
                v = st.rand(1, n, hkv, D).to(DEV)
                layer.update(pos.to(DEV), k, v, slot_mapping=slots)
                O.append(st.mk[l], st.mv[l], k.cpu()[0], v.cpu()[0], slots_ref)
    for step in range(3):
        st.step(rows, torch.tensor([[prefix + s + step] for s in suffix]))
    # the same steps with the shared pages read once for the whole batch: the scheduler asks the page
    # table which leading pages all rows map alike
    n_common = st.pt.common_prefix_pages(rows, min_tokens=prefix + min(suffix))
    assert n_common == 45
    for step in range(3, 5):
        st.step(rows, torch.tensor([[prefix + s + step] for s in suffix]), shared_prefix_pages=n_common)
    st.check_pools_bit_exact()
    # the shared pages were never written after the prefix was stored
    for r in rows:
        assert st.pt.page_table_cpu[r][:45] == shared[:45] and st.pt.page_table_cpu[r][45] != shared[45]


def test_config3_full_batch_sampled_against_oracle():
    """Full-size single layer of the FP8 configuration (batch 256, contexts U[4096, 32768], about
    10 GB of K+V codes): the kernel runs on everything, a sample of sequences is checked against the
    oracle, and a physical re-paging of the pool (pages moved, table updated) must not change a bit."""
    g = torch.Generator().manual_seed(1003)
    B, hq, hkv, D, P = 256, 32, 8, 128, 16
    lengths = torch.randint(4096, 32769, (B,), generator=g)
    pages_per = (lengths + P - 1) // P
    total = int(pages_per.sum())
    n_pages = total + 64
    free = torch.cuda.mem_get_info()[0]
    need = 2 * n_pages * hkv * P * D
    if free < 2.6 * need:
        pytest.skip("not enough free HBM for the full-size case")
    perm = torch.randperm(n_pages - 1, generator=g) + 1
    width = int(pages_per.max())
    table = torch.zeros(B, width, dtype=torch.int32)
    cur = 0
    for b in range(B):
        n = int(pages_per[b])
        table[b, :n] = perm[cur:cur + n].to(torch.int32)
        cur += n
    dg = torch.Generator(device=DEV).manual_seed(5)
    k_pool = torch.randint(0, 256, (n_pages, hkv, P, D), generator=dg, dtype=torch.uint8, device=DEV)
    v_pool = torch.randint(0, 256, (n_pages, hkv, P, D), generator=dg, dtype=torch.uint8, device=DEV)
    k_pool[(k_pool & 0x7F) == 0x7F] = 0x30  # no NaN codes
    v_pool[(v_pool & 0x7F) == 0x7F] = 0x30
    k_pool &= 0xBF  # keep magnitudes below 2: realistic code range, finite softmax
    v_pool &= 0xBF
    q = torch.randn(B, 1, hq, D, generator=dg, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    ks = (torch.rand(hkv, generator=g) * 0.5 + 0.5)
    vs = (torch.rand(hkv, generator=g) * 0.5 + 0.5)
    from kestrel_b200 import kernels
    args = dict(page_table=table.to(DEV), seqused_k=lengths.to(torch.int32).to(DEV), causal=True,
                k_scale=ks.to(DEV), v_scale=vs.to(DEV))
    out, _ = kernels.flash_attn_fwd(q, k_pool.view(torch.float8_e4m3fn).permute(0, 2, 1, 3),
                                    v_pool.view(torch.float8_e4m3fn).permute(0, 2, 1, 3), **args)
    torch.cuda.synchronize()
    for b in (0, 17, 101, 255, int(lengths.argmax()), int(lengths.argmin())):
        L = int(lengths[b])
        pages = table[b, : int(pages_per[b])].to(DEV).long()
        kb = k_pool[pages].cpu()
        vb = v_pool[pages].cpu()
        local = torch.arange(int(pages_per[b]), dtype=torch.int32).view(1, -1)
        want = O.paged_attention(q[b:b + 1].float().cpu(), kb, vb, local, torch.tensor([L], dtype=torch.int32),
                                 k_scale=ks, v_scale=vs)
        assert_close(out[b:b + 1], want, f"sequence {b} (L={L})")
    # re-page: rotate every sequence's pages to other physical slots
    shift = torch.randperm(n_pages - 1, generator=g) + 1  # old page p (1-based) -> new page shift[p-1]
    new_k = torch.empty_like(k_pool)
    new_v = torch.empty_like(v_pool)
    idx = shift.to(DEV)
    new_k[idx] = k_pool[1:]
    new_v[idx] = v_pool[1:]
    del k_pool, v_pool
    lut = torch.zeros(n_pages, dtype=torch.int32)
    lut[1:] = shift.to(torch.int32)
    table2 = lut[table.long()]
    args["page_table"] = table2.to(DEV)
    out2, _ = kernels.flash_attn_fwd(q, new_k.view(torch.float8_e4m3fn).permute(0, 2, 1, 3),
                                     new_v.view(torch.float8_e4m3fn).permute(0, 2, 1, 3), **args)
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))
