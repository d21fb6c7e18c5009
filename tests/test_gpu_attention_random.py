"""Seeded random shapes across every kernel switch of the paged attention op (transposed decode kernel, 16-row
and 32-row split-KV kernels, tensor-memory kernel with and without its key split, gather and TMA copy paths,
thread-per-item and warp-per-item merge), each checked against the fp32 CPU oracle with the tolerance of
``test_gpu_attention.py``."""

import random

import pytest
import torch

from helpers import make_paged_problem
from test_gpu_attention import _clean_status, assert_close, run_case  # noqa: F401  (autouse fixture)

pytestmark = pytest.mark.gpu


def _draw(seed):
    rng = random.Random(seed)
    head_dim = rng.choice([64, 128])
    group = rng.choice([1, 2, 4, 8])
    heads_kv = rng.choice([1, 2, 4])
    kv = rng.choice(["same", "same", "fp8"])
    page_size = rng.choice([1, 2, 4, 16, 16, 64])
    # query rows per KV head on either side of 8, 16, 32, 33, 64/65, 128, 256
    seqlen_q = rng.choice([1, 1, 2, 3, 4, 5, 8, 9, 16, 17, 24, 33, 40, 64, 70, 130])
    seqlen_q = max(1, min(seqlen_q, 300 // group))
    batch = rng.choice([1, 1, 2, 3, 5, 8, 12, 40])
    if batch == 40:                       # enough (sequence, KV head) pairs to reach the SM count
        heads_kv, seqlen_q = 4, min(seqlen_q, 8)
    shape = rng.choice(["short", "mixed", "long", "one_long"])
    lengths = []
    for b in range(batch):
        if shape == "short":
            L = rng.randint(0, 200)
        elif shape == "mixed":
            L = rng.choice([0, 1, rng.randint(1, 64), rng.randint(64, 700), rng.randint(700, 2500)])
        elif shape == "long":
            L = rng.randint(1500, 4000)
        else:
            L = rng.randint(6000, 12000) if b == 0 else rng.randint(1, 300)
        lengths.append(L)
    if batch == 40:
        lengths = [min(L, 600) for L in lengths]
    mode = rng.choice(["causal", "causal", "causal", "full", "window"])
    window = rng.choice([0, 7, 63, 500]) if mode == "window" else None
    use_sq = rng.random() < 0.25
    return dict(head_dim=head_dim, group=group, heads_kv=heads_kv, kv=kv, page_size=page_size, seqlen_q=seqlen_q,
                batch=batch, lengths=lengths, mode=mode, window=window, use_sq=use_sq, rng_seed=rng.randint(0, 1 << 30))


@pytest.mark.parametrize("seed", range(200))
def test_random_shape(seed):
    c = _draw(1000 + seed)
    dtype = torch.bfloat16 if seed % 3 else torch.float16
    p = make_paged_problem(seed=c["rng_seed"], batch=c["batch"], len_lo=0, len_hi=0, n_q_heads=c["group"] * c["heads_kv"],
                           n_kv_heads=c["heads_kv"], head_dim=c["head_dim"], page_size=c["page_size"],
                           seqlen_q=c["seqlen_q"], dtype=dtype, lengths=c["lengths"])
    seqused_q = None
    if c["use_sq"]:
        g = torch.Generator().manual_seed(c["rng_seed"])
        seqused_q = torch.randint(0, c["seqlen_q"] + 1, (c["batch"],), generator=g, dtype=torch.int32)
    out, want, lse, want_lse = run_case(p, dtype, kv=c["kv"], scales=(0.02, 0.03) if c["kv"] == "fp8" else None,
                                        causal=c["mode"] != "full", window=c["window"], seqused_q=seqused_q,
                                        return_lse=True)
    what = {k: v for k, v in c.items() if k != "lengths"}
    for b in range(c["batch"]):
        n = c["seqlen_q"] if seqused_q is None else int(seqused_q[b])
        if n == 0:
            continue
        if c["lengths"][b] == 0:          # no keys at all: zeros and a log-sum-exp of -inf
            assert (out[b, :n] == 0).all() and torch.isinf(lse[b, :, :n]).all(), (what, b)
            continue
        assert_close(out[b, :n], want[b, :n], f"{what} sequence {b} (L={c['lengths'][b]})")
        ref = want_lse[b, :, :n]
        got = lse[b, :, :n].cpu()
        fin = torch.isfinite(ref)
        assert torch.equal(torch.isfinite(got), fin), (what, b)
        if fin.any():
            assert torch.allclose(got[fin], ref[fin], atol=3e-3, rtol=1e-3), (what, b)
