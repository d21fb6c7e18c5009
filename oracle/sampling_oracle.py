"""CPU oracle of the sampling hand-off: ``sample_step_from_logits(logits, temperatures, top_ps, ...)``.

TEST INFRASTRUCTURE ONLY: imported by tests, never by ``kestrel_b200``.

The reference calls ``kestrel_kernels.sampling.sample_step_from_logits`` right after the decoder stack
(``kestrel/scheduler/scheduler.py:2986-2991``, ``kestrel/scheduler/spatial.py:105-123``); the kernel itself is in
the absent ``kestrel-kernels`` wheel, so its arithmetic is **parity unpinned**.  What the tree does pin is the
contract around it, restated here:

* ``temperatures <= 1e-6`` (``_SAMPLING_EPS``, ``scheduler.py:55``) means greedy: the arg-max of the logits,
  log-probability 0 (``_selected_logprobs_from_logits``, ``scheduler.py:3020-3042``);
* otherwise tokens are drawn from ``softmax(logits / temperature)`` restricted to the top-p nucleus, and the
  reported log-probability is ``logits[id] / T - logsumexp(logits / T)`` over the WHOLE vocabulary (same function);
* greedy requests are served with ``temperature 0, top_p 1`` (``scheduler.py:2949-2953``).

Defined here (the published nucleus-sampling rule, made deterministic): the nucleus is ``{i : p_i >= tau}`` where
``tau`` is the largest probability such that the tokens at or above it hold at least ``top_p`` of the mass (ties at
``tau`` all stay in); the token is the first index, in vocabulary order, whose running nucleus mass exceeds
``u * nucleus_mass`` for the row's uniform ``u`` in [0, 1).
"""

from __future__ import annotations

import torch

SAMPLING_EPS = 1e-6


def nucleus(logits_row: torch.Tensor, temperature: float, top_p: float):
    """``(p, keep, Z, m)`` in float64: unnormalised probabilities ``exp(x / T - m)``, the nucleus mask, their
    sum and the maximum of the scaled logits."""
    s = logits_row.to(torch.float64) / float(temperature)
    m = s.max()
    p = torch.exp(s - m)
    Z = p.sum()
    if top_p >= 1.0:
        return p, torch.ones_like(p, dtype=torch.bool), Z, m
    order = torch.argsort(p, descending=True, stable=True)
    csum = torch.cumsum(p[order], 0)
    k = int(torch.searchsorted(csum, torch.tensor(max(top_p, 0.0) * float(Z), dtype=torch.float64)).clamp(max=p.numel() - 1))
    tau = p[order[k]]
    return p, p >= tau, Z, m


def sample_step_from_logits(logits: torch.Tensor, temperatures: torch.Tensor, top_ps: torch.Tensor,
                            uniforms: torch.Tensor):
    """``logits [B, V]``, ``temperatures, top_ps, uniforms [B]`` -> ``(ids int64 [B], logprobs float32 [B])``."""
    B, V = logits.shape
    ids = torch.zeros(B, dtype=torch.int64)
    lps = torch.zeros(B, dtype=torch.float32)
    for b in range(B):
        row = logits[b].float()
        t = max(float(temperatures[b]), 0.0)
        if t <= SAMPLING_EPS:
            ids[b] = int(torch.argmax(row))
            lps[b] = 0.0
            continue
        p, keep, Z, m = nucleus(row, t, float(top_ps[b]))
        kept = torch.where(keep, p, torch.zeros_like(p))
        cdf = torch.cumsum(kept, 0)
        target = float(uniforms[b]) * float(cdf[-1])
        idx = int(torch.searchsorted(cdf, torch.tensor(target, dtype=torch.float64), right=True).clamp(max=V - 1))
        ids[b] = idx
        lps[b] = float(row[idx].double() / t - m - torch.log(Z))
    return ids, lps


def check_sample(logits_row: torch.Tensor, temperature: float, top_p: float, u: float, got_id: int,
                 rel_slack: float = 2e-5) -> str | None:
    """Is ``got_id`` a correct draw for this row?  Returns None when it is, else a description.  The kernel sums
    in another order and with hardware exponentials, so a draw is accepted when it is right for SOME threshold
    and target within ``rel_slack`` (relative to the mass) of the exact ones."""
    t = max(float(temperature), 0.0)
    if t <= SAMPLING_EPS:
        row = logits_row.float()
        return None if float(row[got_id]) == float(row.max()) else "greedy row did not return an arg-max"
    p, keep, Z, _ = nucleus(logits_row.float(), t, top_p)
    slack = rel_slack * float(Z)
    if not bool(keep[got_id]):
        # just below the threshold is fine when the nucleus mass is within the slack of top_p * Z
        above = float(p[p > p[got_id]].sum())
        if not (above < top_p * float(Z) + slack):
            return f"token {got_id} lies outside the nucleus (mass above it {above / float(Z):.6f}, top_p {top_p})"
    kept = torch.where(keep, p, torch.zeros_like(p))
    cdf = torch.cumsum(kept, 0)
    lo = float(cdf[got_id - 1]) if got_id > 0 else 0.0
    hi = float(cdf[got_id])
    target = float(u) * float(cdf[-1])
    # a token just outside the exact nucleus changes the running masses by at most the slack as well
    if lo - 2 * slack <= target <= hi + 2 * slack:
        return None
    return f"u*mass = {target:.9g} is not in token {got_id}'s interval [{lo:.9g}, {hi:.9g}]"
