"""The CPU oracle against the fixtures made from the reference's own torch path."""

import json
import math

import numpy as np
import pytest
import torch

from helpers import from_np, make_paged_problem
from oracle import paged_kv_oracle as O


@pytest.fixture(scope="module")
def vec(golden_dir):
    return np.load(golden_dir / "reference_vectors.npz")


@pytest.fixture(scope="module")
def meta(golden_dir):
    return json.loads((golden_dir / "reference_vectors.json").read_text())


def test_append_matches_reference(vec, meta):
    assert len(meta["append"]) >= 6
    for m in meta["append"]:
        n = m["name"]
        dt = m["dtype"]
        k = from_np(vec[f"append_{n}_k"], dt)
        v = from_np(vec[f"append_{n}_v"], dt)
        slots = torch.from_numpy(vec[f"append_{n}_slots"])
        want_k = from_np(vec[f"append_{n}_kcache"], dt)
        want_v = from_np(vec[f"append_{n}_vcache"], dt)
        kc = torch.zeros_like(want_k)
        vc = torch.zeros_like(want_v)
        O.append(kc, vc, k.reshape(-1, m["heads"], m["dim"]), v.reshape(-1, m["heads"], m["dim"]), slots)
        assert torch.equal(kc.view(torch.uint8), want_k.view(torch.uint8)), n
        assert torch.equal(vc.view(torch.uint8), want_v.view(torch.uint8)), n


def test_append_skips_negative_slots():
    kc = torch.zeros(2, 1, 4, 2)
    vc = torch.zeros(2, 1, 4, 2)
    k = torch.arange(6, dtype=torch.float32).view(3, 1, 2) + 1
    O.append(kc, vc, k, k, torch.tensor([1, -1, 6]))
    assert kc[0, 0, 1].tolist() == [1, 2] and kc[1, 0, 2].tolist() == [5, 6]
    assert kc.abs().sum() == 1 + 2 + 5 + 6


def test_slot_mapping_matches_reference(vec, meta):
    for m in meta["slots"]:
        n = m["name"]
        got = O.build_slot_mapping(torch.from_numpy(vec[f"slots_{n}_table"]), torch.from_numpy(vec[f"slots_{n}_batch"]),
                                   torch.from_numpy(vec[f"slots_{n}_pos"]), m["page_size"])
        assert got.dtype == torch.int64
        assert torch.equal(got, torch.from_numpy(vec[f"slots_{n}_out"])), n


def test_metadata_matches_reference_test_vector(vec):
    out_pt = torch.full((2, 16), -99, dtype=torch.int32)
    out_sk = torch.full((2,), -1, dtype=torch.int32)
    O.build_paged_kv_metadata(torch.from_numpy(vec["meta_table"]), torch.from_numpy(vec["meta_batch"]),
                              torch.from_numpy(vec["meta_pos"]), out_pt, out_sk, 4)
    assert torch.equal(out_pt, torch.from_numpy(vec["meta_out_table"]))
    assert torch.equal(out_sk, torch.from_numpy(vec["meta_out_seqused"]))
    assert out_sk.tolist() == [8, 9]


def test_fp8_encoder_equals_torch_cast_for_all_bf16_values():
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16)
    x = bits.view(torch.bfloat16).float()
    finite = torch.isfinite(x)
    x = x[finite]
    want = x.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    got = torch.from_numpy(O.fp8_e4m3_encode(x.numpy()))
    assert torch.equal(got, want)


def test_fp8_encoder_equals_torch_cast_on_scaled_random_fp32():
    g = torch.Generator().manual_seed(7)
    x = torch.randn(200_000, generator=g) * torch.logspace(-4, 3, 200_000)
    scale = torch.tensor(0.0371)
    y = x / scale
    want = y.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    got = O.fp8_quantise(x, scale)
    assert torch.equal(got, want)
    # ties-to-even and saturation spot checks (value -> code)
    probe = torch.tensor([17.0, 19.0, 449.0, 465.0, 1000.0, -1000.0, 2.0 ** -10, 2.0 ** -9, 3 * 2.0 ** -10, 0.0])
    codes = O.fp8_quantise(probe, 1.0)
    dec = torch.from_numpy(O.fp8_e4m3_decode(codes.numpy()))
    assert dec.tolist() == [16.0, 20.0, 448.0, 448.0, 448.0, -448.0, 0.0, 2.0 ** -9, 2.0 ** -8, 0.0]


def test_fp8_decode_is_inverse_on_all_codes():
    codes = np.arange(256, dtype=np.uint8)
    vals = O.fp8_e4m3_decode(codes)
    want = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    ok = ~np.isnan(want)
    assert np.array_equal(vals[ok], want[ok]) and np.isnan(vals[~ok]).all()
    back = O.fp8_e4m3_encode(vals[ok])
    keep = codes[ok]
    assert np.array_equal(back[keep != 0x80], keep[keep != 0x80])  # -0 encodes as 0x80 too
    assert back[keep == 0x80][0] == 0x80


def test_fp8_per_head_scales():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(5, 4, 8, generator=g)
    s = torch.tensor([0.01, 0.02, 0.5, 1.0])
    got = O.fp8_quantise(x, s)
    for h in range(4):
        assert torch.equal(got[:, h], O.fp8_quantise(x[:, h], float(s[h])))


def test_attention_oracle_equals_dense_sdpa():
    p = make_paged_problem(seed=5, batch=3, len_lo=1, len_hi=70, n_q_heads=8, n_kv_heads=2, head_dim=16, page_size=4,
                           seqlen_q=3)
    out = O.paged_attention(p["q"], p["k_pool"], p["v_pool"], p["page_table"], p["seqused_k"])
    for b, L in enumerate(p["lengths"]):
        K = O.gather_kv(p["k_pool"], p["page_table"][b], L).repeat_interleave(4, dim=1)
        V = O.gather_kv(p["v_pool"], p["page_table"][b], L).repeat_interleave(4, dim=1)
        sq = 3
        mask = torch.ones(sq, L, dtype=torch.bool).tril(diagonal=L - sq)
        ref = torch.nn.functional.scaled_dot_product_attention(
            p["q"][b].transpose(0, 1), K.transpose(0, 1), V.transpose(0, 1), attn_mask=mask)
        ref = ref.transpose(0, 1)
        # rows that see no key (L < sq) are zero in the oracle; SDPA gives NaN there
        rows = torch.arange(sq) + (L - sq) >= 0
        assert torch.allclose(out[b][rows], ref[rows], atol=1e-5, rtol=1e-5)
        assert (out[b][~rows] == 0).all()


def test_attention_oracle_window_and_fp8():
    p = make_paged_problem(seed=6, batch=2, len_lo=40, len_hi=90, n_q_heads=4, n_kv_heads=2, head_dim=8, page_size=16)
    full = O.paged_attention(p["q"], p["k_pool"], p["v_pool"], p["page_table"], p["seqused_k"])
    wide = O.paged_attention(p["q"], p["k_pool"], p["v_pool"], p["page_table"], p["seqused_k"], window_left=10_000)
    assert torch.allclose(full, wide)
    one = O.paged_attention(p["q"], p["k_pool"], p["v_pool"], p["page_table"], p["seqused_k"], window_left=0)
    for b, L in enumerate(p["lengths"]):
        last = O.gather_kv(p["v_pool"], p["page_table"][b], L)[L - 1].repeat_interleave(2, dim=0)
        assert torch.allclose(one[b, 0], last, atol=1e-6)
    ks = torch.tensor([0.05, 0.07])
    kq = O.fp8_quantise(p["k_pool"].permute(0, 2, 1, 3), ks).permute(0, 2, 1, 3).contiguous()
    vq = O.fp8_quantise(p["v_pool"].permute(0, 2, 1, 3), ks).permute(0, 2, 1, 3).contiguous()
    deq = O.paged_attention(p["q"], kq, vq, p["page_table"], p["seqused_k"], k_scale=ks, v_scale=ks)
    assert (deq - full).abs().max() < 0.15
    as_f8 = O.paged_attention(p["q"], kq.view(torch.float8_e4m3fn), vq.view(torch.float8_e4m3fn), p["page_table"],
                              p["seqused_k"], k_scale=ks, v_scale=ks)
    assert torch.equal(as_f8, deq)


def test_lse_and_empty_sequences():
    p = make_paged_problem(seed=8, batch=3, len_lo=1, len_hi=20, n_q_heads=2, n_kv_heads=2, head_dim=8, page_size=4,
                           lengths=[5, 0, 17])
    out, lse = O.paged_attention(p["q"], p["k_pool"], p["v_pool"], p["page_table"], p["seqused_k"], return_lse=True)
    assert (out[1] == 0).all() and torch.isinf(lse[1]).all()
    K = O.gather_kv(p["k_pool"], p["page_table"][0], 5)
    s = torch.einsum("hd,lhd->hl", p["q"][0, 0], K) / math.sqrt(8)
    assert torch.allclose(lse[0, :, 0], torch.logsumexp(s, dim=-1), atol=1e-5)


def test_copy_pages_and_decode_step():
    p = make_paged_problem(seed=9, batch=2, len_lo=17, len_hi=40, n_q_heads=4, n_kv_heads=2, head_dim=8, page_size=16)
    k2 = p["k_pool"].clone()
    O.copy_pages([k2], [int(p["page_table"][0, 0])], [0])
    assert torch.equal(k2[0], p["k_pool"][int(p["page_table"][0, 0])])
    # decode_step: append at position L (the page table already has room unless L % 16 == 0)
    lens = [L - 1 for L in p["lengths"]]
    rows = torch.zeros(3, p["page_table"].shape[1], dtype=torch.int32)
    rows[1:] = p["page_table"]
    g = torch.Generator().manual_seed(1)
    k_new = torch.randn(2, 1, 2, 8, generator=g)
    v_new = torch.randn(2, 1, 2, 8, generator=g)
    kc, vc = p["k_pool"].clone(), p["v_pool"].clone()
    out, used = O.decode_step(p["q"], k_new, v_new, kc, vc, rows, torch.tensor([1, 2]),
                              torch.tensor(lens).view(2, 1))
    assert used.tolist() == p["lengths"]
    for b in range(2):
        got = O.gather_kv(kc, p["page_table"][b], p["lengths"][b])[-1]
        assert torch.equal(got, k_new[b, 0])
    assert out.shape == (2, 1, 4, 8) and torch.isfinite(out).all()


# ---------------------------------------------------------------------------
# rotary embedding and the per-step metadata
# ---------------------------------------------------------------------------

def test_rope_table_matches_reference(golden_dir):
    vec = np.load(golden_dir / "rope_vectors.npz")
    rot, end, theta = vec["table_args"].tolist()
    got = O.precompute_freqs_cis(int(rot), int(end), float(theta))
    want = torch.from_numpy(vec["table"])
    assert got.shape == want.shape and got.dtype == torch.float32
    # cos/sin come from the host's libm: allow the last bit
    assert (got - want).abs().max().item() <= 2.0 ** -23


def test_rope_matches_reference_rotate_half_in_fp32(golden_dir):
    vec = np.load(golden_dir / "rope_vectors.npz")
    x, pos, want = (torch.from_numpy(vec[k]) for k in ("x", "pos", "y"))
    got = O.rotary_embedding(pos, x, torch.from_numpy(vec["table"]))
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))
    # elements past the rotated width pass through
    rot = vec["table"].shape[1]
    assert torch.equal(got[..., rot:], x[..., rot:])


def test_rope_rounds_once_to_the_row_dtype():
    g = torch.Generator().manual_seed(5)
    table = O.precompute_freqs_cis(32, 128, 1.5e6)
    x = torch.randn(9, 2, 64, generator=g).to(torch.bfloat16)
    pos = torch.randint(0, 128, (9,), generator=g)
    got = O.rotary_embedding(pos, x, table)
    assert got.dtype == torch.bfloat16
    assert torch.equal(got, O.rotary_embedding(pos, x.float(), table).to(torch.bfloat16))
    assert torch.equal(O.rotary_embedding(torch.zeros(9, dtype=torch.long), x, table), x)  # angle 0


def test_decode_step_metadata_is_metadata_then_slot_mapping(vec):
    table = torch.from_numpy(vec["meta_table"])
    batch = torch.from_numpy(vec["meta_batch"])
    pos = torch.from_numpy(vec["meta_pos"])
    out_pt = torch.full((2, 16), -99, dtype=torch.int32)
    out_sk = torch.zeros(2, dtype=torch.int32)
    slots, positions = O.build_decode_step_metadata(table, batch, pos, out_pt, out_sk, 4, n_new=3)
    assert torch.equal(out_pt, torch.from_numpy(vec["meta_out_table"]))
    assert torch.equal(out_sk, torch.from_numpy(vec["meta_out_seqused"]))
    assert positions.tolist() == [[5, 6, 7], [6, 7, 8]]
    assert torch.equal(slots, O.build_slot_mapping(table, batch, positions, 4))


def test_sampling_oracle_known_answers():
    """Nucleus rule and inverse-CDF draw on a vocabulary of three: probabilities 0.5 / 0.3 / 0.2."""
    from oracle import sampling_oracle as S

    logits = torch.log(torch.tensor([[0.5, 0.3, 0.2]])).repeat(6, 1)
    temps = torch.tensor([1.0, 1.0, 1.0, 1.0, 0.0, 1.0])
    top_ps = torch.tensor([1.0, 1.0, 0.7, 0.7, 1.0, 0.0])
    u = torch.tensor([0.49, 0.81, 0.62, 0.63, 0.99, 0.99])
    ids, lps = S.sample_step_from_logits(logits, temps, top_ps, u)
    # whole vocabulary: cdf 0.5 / 0.8 / 1.0; nucleus 0.7 -> {0, 1} with mass 0.8: cdf 0.5 / 0.8, target u * 0.8
    assert ids.tolist() == [0, 2, 0, 1, 0, 0]
    assert abs(float(lps[1]) - math.log(0.2)) < 1e-6 and float(lps[4]) == 0.0
    assert S.check_sample(logits[2], 1.0, 0.7, 0.62, 0) is None
    assert S.check_sample(logits[2], 1.0, 0.7, 0.62, 1) is not None
    assert S.check_sample(logits[2], 1.0, 0.7, 0.9, 2) is not None      # outside the nucleus
