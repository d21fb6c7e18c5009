"""The sampling hand-off (``sample_step_from_logits``) against the CPU oracle.

The reference's kernel lives in the absent wheel, so its arithmetic is parity-unpinned; what the reference tree
pins is the contract (greedy below 1e-6, log-probabilities over the whole vocabulary, the call shape), restated in
``oracle/sampling_oracle.py``.  Greedy rows must match bit for bit.  A drawn token must be a correct draw for the
row's uniform: inside the nucleus, its cumulative-mass interval containing ``u * mass`` -- up to 2e-5 of the mass,
because the kernel sums hardware exponentials in fixed point while the oracle sums float64 (rows whose nucleus
boundary is closer than that to ``top_p`` are ambiguous by construction and skipped).  Log-probabilities: 2e-3.
"""

import math

import pytest
import torch

from kestrel_b200 import _native, kernels
from oracle import sampling_oracle as S

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ambiguous(row, t, top_p, margin=1e-4):
    """True when the nucleus boundary falls within `margin` of top_p: either reading is a correct nucleus."""
    if t <= S.SAMPLING_EPS or top_p >= 1.0:
        return False
    p, _, Z, _ = S.nucleus(row.float(), t, top_p)
    csum = torch.cumsum(torch.sort(p, descending=True).values, 0) / Z
    return bool(((csum - top_p).abs() < margin).any())


@pytest.mark.parametrize("dtype,vocab", [(torch.bfloat16, 51200), (torch.float32, 51200), (torch.float16, 32000),
                                         (torch.bfloat16, 1003), (torch.float32, 151936)])
def test_draws_are_correct_for_their_uniform(dtype, vocab):
    g = torch.Generator().manual_seed(7 + vocab)
    B = 48
    logits = (torch.randn(B, vocab, generator=g) * 3.0).to(dtype)
    temps = torch.tensor([0.0, 1e-7, 0.3, 0.7, 1.0, 1.5] * 8)
    top_ps = torch.tensor([1.0, 0.95, 0.9, 0.5, 0.1, 0.0, 0.999, 0.3] * 6)
    u = torch.rand(B, generator=g)
    u[0], u[1], u[2] = 0.0, 0.9999999, 0.5
    out = torch.full((B,), -1, dtype=torch.int64, device=DEV)
    lp = torch.full((B,), float("nan"), device=DEV)
    ret = kernels.sample_step_from_logits(logits.to(DEV), temps.to(DEV), top_ps.to(DEV), out=out, logprobs_out=lp,
                                          uniforms=u.to(DEV))
    assert ret is out
    ids, lps = out.cpu(), lp.cpu()
    assert ((ids >= 0) & (ids < vocab)).all()
    want_ids, _ = S.sample_step_from_logits(logits, temps, top_ps, u)
    exact = 0
    for b in range(B):
        t, tp = float(temps[b]), float(top_ps[b])
        if t <= S.SAMPLING_EPS:
            assert int(ids[b]) == int(want_ids[b]) and float(lps[b]) == 0.0     # first arg-max, log-probability 0
            continue
        if not _ambiguous(logits[b], t, tp):
            why = S.check_sample(logits[b], t, tp, float(u[b]), int(ids[b]))
            assert why is None, (b, t, tp, why)
        exact += int(ids[b]) == int(want_ids[b])
        s = logits[b].double() / t
        ref_lp = float(s[int(ids[b])] - torch.logsumexp(s, 0))
        assert abs(float(lps[b]) - ref_lp) <= 2e-3, (b, float(lps[b]), ref_lp)
    assert exact >= 0.9 * (B - 16)          # (the oracle's own draw differs only where u * mass sits on an interval edge)
    # the same inputs give the same tokens
    again = kernels.sample_step_from_logits(logits.to(DEV), temps.to(DEV), top_ps.to(DEV), uniforms=u.to(DEV))
    assert torch.equal(again.cpu(), ids)
    assert _native.device_status(torch.cuda.current_device(), clear=True)[0] == 0


def test_greedy_takes_the_first_maximum():
    logits = torch.zeros(4, 64, dtype=torch.bfloat16)
    logits[0, [5, 9, 40]] = 3.0
    logits[1, 63] = 1.0
    logits[2] = -1.0
    logits[3, 0] = 2.0
    temps = torch.zeros(4)
    out = kernels.sample_step_from_logits(logits.to(DEV), temps.to(DEV), torch.ones(4, device=DEV),
                                          uniforms=torch.full((4,), 0.77, device=DEV))
    assert out.cpu().tolist() == [5, 63, 0, 0]


@pytest.mark.parametrize("top_p", [1.0, 0.8])
def test_draw_frequencies_follow_the_distribution(top_p):
    g = torch.Generator().manual_seed(11)
    V, N, t = 64, 16384, 0.8
    row = torch.randn(V, generator=g) * 2.0
    logits = row.to(torch.float32).repeat(N, 1)
    u = torch.rand(N, generator=g)
    ids = kernels.sample_step_from_logits(logits.to(DEV), torch.full((N,), t, device=DEV),
                                          torch.full((N,), top_p, device=DEV), uniforms=u.to(DEV)).cpu()
    p, keep, _, _ = S.nucleus(row, t, top_p)
    q = torch.where(keep, p, torch.zeros_like(p))
    q = (q / q.sum()).float()
    freq = torch.bincount(ids, minlength=V).float() / N
    assert (freq[~keep] == 0).all()
    tol = 4.5 * torch.sqrt(q * (1 - q) / N) + 1e-4
    assert ((freq - q).abs() <= tol).all(), (freq - q).abs().max()


def test_generator_call_shape_of_the_reference():
    """``sample_step_from_logits(logits, temps, top_ps, out=..., generator=..., logprobs_out=...)`` as the
    scheduler calls it (kestrel/scheduler/scheduler.py:2979-2991): reproducible for a seeded generator."""
    B, V = 8, 51200
    logits = torch.randn(B, V, device=DEV, dtype=torch.bfloat16)
    temps = torch.full((B,), 0.9, device=DEV)
    top_ps = torch.full((B,), 0.9, device=DEV)
    outs = []
    for _ in range(2):
        gen = torch.Generator(device=DEV).manual_seed(1234)
        out = torch.empty(B, dtype=torch.int64, device=DEV)
        lp = torch.empty(B, device=DEV)
        got = kernels.sample_step_from_logits(logits, temps, top_ps, out=out, generator=gen, logprobs_out=lp)
        assert got is out
        outs.append((out.cpu().clone(), lp.cpu().clone()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert (outs[0][1] <= 0).all() and torch.isfinite(outs[0][1]).all()
    rt = kernels.get_runtime()
    assert rt.sampling.sample_step_from_logits is kernels.sample_step_from_logits or callable(rt.sampling.sample_step_from_logits)


def test_bad_arguments_are_refused():
    lib = _native.load()
    rc = lib.kb200_sample_step_from_logits(None, _native.DTYPE_BF16, 1, 8, 8, None, None, None, None, None, 0, None)
    assert rc == -1
    x = torch.zeros(1, 8, device=DEV)
    rc = lib.kb200_sample_step_from_logits(x.data_ptr(), _native.DTYPE_F32, 1, (1 << 20) + 8, (1 << 20) + 8, x.data_ptr(),
                                           x.data_ptr(), x.data_ptr(), x.data_ptr(), None, 0, None)
    assert rc == -1 and "2^20" in lib.kb200_last_error().decode()
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        kernels.sample_step_from_logits(torch.zeros(1, 8), torch.zeros(1), torch.ones(1))
