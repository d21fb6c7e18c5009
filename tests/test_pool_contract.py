"""The pool layout and FP8 code contract, locked by a golden byte image.

A whole-model decode kernel reads and appends the same pools directly (the reference's megakernel path,
``kestrel/models/moondream/runtime.py:638-644``), so what the append leaves in memory is an interface:

* pool tensor ``[n_pages, H_kv, P, D]`` contiguous: element ``(page, head, token, d)`` lives at byte
  ``(((page * H_kv + head) * P + token) * D + d) * elt``;
* ``slot = page * P + token`` with the page taken from the sequence's page-table row;
* bf16 pools hold the projection's bytes unchanged; FP8 pools hold ``e4m3fn(satfinite(rn(x / scale)))``
  with the per-layer scalar scale.

``tests/golden/pool_image.npz`` (made by ``tests/golden/make_golden.py``) holds the bytes of a small bf16 pool
written by the reference's own torch path and of the FP8 pool the oracle defines on the same slots, after a
fixed sequence of prompt and decode appends.  The CPU test pins the oracle to it; the GPU test replays the
sequence through this library's classes and kernels and compares the raw pool bytes.
"""

import numpy as np
import pytest
import torch

from helpers import from_np
from oracle import paged_kv_oracle as O


def _steps(img):
    n = int(img["n_steps"][0])
    for i in range(n):
        yield (torch.from_numpy(img[f"step{i}_rows"]), torch.from_numpy(img[f"step{i}_pos"]),
               from_np(img[f"step{i}_fused"], "bfloat16"), torch.from_numpy(img[f"step{i}_slots"]))


def _split(fused, H, D, hq):
    k = fused[..., hq * D:(hq + H) * D].unflatten(-1, (H, D))
    v = fused[..., (hq + H) * D:].unflatten(-1, (H, D))
    return k, v


def test_oracle_reproduces_the_pool_image(golden_dir):
    img = np.load(golden_dir / "pool_image.npz")
    n_pages, P, H, D, hq = (int(x) for x in img["geometry"])
    ks, vs = (float(x) for x in img["scales"])
    table = torch.from_numpy(img["page_table"])
    kb = torch.zeros(n_pages, H, P, D, dtype=torch.bfloat16)
    vb = torch.zeros_like(kb)
    k8 = torch.zeros(n_pages, H, P, D, dtype=torch.uint8)
    v8 = torch.zeros_like(k8)
    for rows, pos, fused, slots in _steps(img):
        assert torch.equal(O.build_slot_mapping(table, rows, pos, P), slots)
        k, v = _split(fused, H, D, hq)
        O.append(kb, vb, k.reshape(-1, H, D), v.reshape(-1, H, D), slots.reshape(-1))
        O.append(k8, v8, k.reshape(-1, H, D), v.reshape(-1, H, D), slots.reshape(-1),
                 k_scale=torch.tensor([ks]), v_scale=torch.tensor([vs]))
    assert np.array_equal(kb.view(torch.uint8).numpy(), img["k_bf16"])
    assert np.array_equal(vb.view(torch.uint8).numpy(), img["v_bf16"])
    assert np.array_equal(k8.numpy(), img["k_e4m3"]) and np.array_equal(v8.numpy(), img["v_e4m3"])
    # the address formula, spelled out on the last appended token of the first step
    rows, pos, fused, slots = next(_steps(img))
    k, _ = _split(fused, H, D, hq)
    slot = int(slots[0, -1])
    page, token = divmod(slot, P)
    flat = img["k_bf16"].reshape(-1)
    for head in range(H):
        off = (((page * H + head) * P + token) * D) * 2
        want = k[0, -1, head].view(torch.uint8).numpy()
        assert np.array_equal(flat[off:off + D * 2], want)


@pytest.mark.gpu
@pytest.mark.parametrize("kv", ["bf16", "e4m3"])
def test_kernels_reproduce_the_pool_image(golden_dir, kv):
    from kestrel_b200 import _native
    from kestrel_b200.kv_cache import KVMemoryPool, PagedKVCache, PageTable

    img = np.load(golden_dir / "pool_image.npz")
    n_pages, P, H, D, hq = (int(x) for x in img["geometry"])
    ks, vs = (float(x) for x in img["scales"])
    dev = "cuda"
    pt = PageTable(n_pages=n_pages, page_size=P, max_batch_size=3, device=dev)
    # the recorded table (the reference drew its pages from a shuffled free list)
    pt._page_table_cpu_tensor.copy_(torch.from_numpy(img["page_table"]))
    pt._dirty_rows.update(range(3))
    pt.commit_block_table()
    kw = dict(k_scale=ks, v_scale=vs) if kv == "e4m3" else {}
    cache = PagedKVCache(pt, n_heads=H, head_dim=D, dtype=torch.float8_e4m3fn if kv == "e4m3" else torch.bfloat16,
                         pool=KVMemoryPool(device=dev), **kw)
    for rows, pos, fused, slots in _steps(img):
        got_slots = pt.build_slot_mapping(rows.to(dev), pos.to(dev))
        assert torch.equal(got_slots.cpu(), slots)
        k, v = _split(fused.to(dev), H, D, hq)          # strided views of the fused projection, as the models pass them
        cache.update(pos.to(dev), k, v, slot_mapping=got_slots)
    got_k = cache.k_cache.contiguous().view(torch.uint8).cpu().numpy()
    got_v = cache.v_cache.contiguous().view(torch.uint8).cpu().numpy()
    assert np.array_equal(got_k, img[f"k_{kv}"]) and np.array_equal(got_v, img[f"v_{kv}"])
    assert _native.device_status(torch.cuda.current_device(), clear=True)[0] == 0
