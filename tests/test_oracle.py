"""CPU checks of the oracle (oracle/evo_ref.py): the committed fixture, analytic
known-answer cases, an fp64 self-check, and an independent cross-check against
torch's scaled_dot_product_attention."""
import math
import os

import numpy as np
import torch

from oracle import evo_ref

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "cfg1_golden.npz")


def test_golden_fixture_config1():
    g = np.load(GOLDEN)
    q, k, v, mask, bias, d_o = evo_ref.make_workload("cfg1_cpu_fp32")
    sums = np.array([t.double().sum().item() for t in (q, k, v, mask, bias, d_o)])
    np.testing.assert_allclose(sums, g["input_sums"], rtol=1e-12)
    r = evo_ref.evo_attention_fwd_bwd_ref(q, k, v, mask, bias, d_o)
    rows = g["rows"].tolist()
    for n in ("o", "dq", "dk", "dv"):
        np.testing.assert_allclose(r[n][:, rows].numpy(), g[n], rtol=0, atol=2e-5, err_msg=n)
    np.testing.assert_allclose(r["dbias"].numpy(), g["dbias"], rtol=0, atol=2e-5)
    lse = evo_ref.evo_lse_ref(q, k, mask, bias, dtype=torch.float64)
    np.testing.assert_allclose(lse[:, 0].numpy(), g["lse_row0"], rtol=0, atol=1e-9)


def test_fp64_self_consistency():
    q, k, v, mask, bias, d_o = evo_ref.make_workload("cfg1_cpu_fp32")
    a = evo_ref.evo_attention_fwd_bwd_ref(q, k, v, mask, bias, d_o, dtype=torch.float32)
    b = evo_ref.evo_attention_fwd_bwd_ref(q, k, v, mask, bias, d_o, dtype=torch.float64, s_chunk=5)
    for n in a:
        ma, rl = evo_ref.parity(b[n], a[n])
        assert ma < 1e-4 and rl < 1e-5, (n, ma, rl)


def test_against_sdpa():
    """Independent implementation: torch SDPA with attn_mask = bias + mask."""
    q, k, v, mask, bias, _ = evo_ref.make_inputs(2, 3, 40, 2, 16, seed=3, mask_kind="bernoulli0.9")
    o = evo_ref.evo_attention_ref(q, k, v, mask, bias)
    qt, kt, vt = (t.transpose(-2, -3) for t in (q, k, v))            # [B,S,H,N,D]
    am = (bias + mask).expand(2, 3, 2, 40, 40)
    o2 = torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, attn_mask=am).transpose(-2, -3)
    assert evo_ref.max_abs_err(o2, o) < 1e-5


def test_kat_uniform_softmax():
    """q = 0, bias = 0: softmax is uniform over the valid residues, so O is
    their mean of V and dBias = P o (dP - delta)."""
    B, S, N, H, D = 1, 2, 16, 2, 8
    g = torch.Generator().manual_seed(0)
    v = torch.randn((B, S, N, H, D), generator=g)
    k = torch.randn((B, S, N, H, D), generator=g)
    q = torch.zeros((B, S, N, H, D))
    bias = torch.zeros((B, 1, H, N, N))
    valid = torch.ones((B, S, N), dtype=torch.bool)
    valid[:, 0, 10:] = False
    mask = torch.where(valid, 0.0, -1e9).reshape(B, S, 1, 1, N)
    o = evo_ref.evo_attention_ref(q, k, v, mask, bias)
    for s, cnt in ((0, 10), (1, 16)):
        mean = v[:, s, :cnt].mean(dim=1, keepdim=True)               # [B,1,H,D]
        assert torch.allclose(o[:, s], mean.expand(B, N, H, D), atol=1e-6)
    lse = evo_ref.evo_lse_ref(q, k, mask, bias)
    assert torch.allclose(lse[:, 0], torch.full((B, H, N), math.log(10.0)), atol=1e-5)


def test_kat_single_valid_residue():
    """Only residue 3 valid: O = V[3] for every query, dV only at residue 3,
    dQ = dK = dBias = 0 (softmax is a constant one-hot)."""
    B, S, N, H, D = 1, 1, 8, 2, 4
    q, k, v, _, bias, d_o = evo_ref.make_inputs(B, S, N, H, D, seed=11)
    valid = torch.zeros((B, S, N), dtype=torch.bool)
    valid[..., 3] = True
    mask = torch.where(valid, 0.0, -1e9).reshape(B, S, 1, 1, N)
    r = evo_ref.evo_attention_fwd_bwd_ref(q, k, v, mask, bias, d_o)
    assert torch.allclose(r["o"], v[:, :, 3:4].expand_as(v), atol=1e-6)
    assert r["dq"].abs().max() < 1e-6 and r["dk"].abs().max() < 1e-6
    assert r["dbias"].abs().max() < 1e-6
    assert torch.allclose(r["dv"][:, :, 3], d_o.sum(dim=2), atol=1e-5)
    assert r["dv"][:, :, :3].abs().max() == 0 and r["dv"][:, :, 4:].abs().max() < 1e-12


def test_kat_diagonal_bias():
    """A large bias on the diagonal makes attention the identity: O ~= V."""
    B, S, N, H, D = 1, 2, 12, 2, 8
    q, k, v, mask, bias, _ = evo_ref.make_inputs(B, S, N, H, D, seed=2)
    bias = bias + 200.0 * torch.eye(N).reshape(1, 1, 1, N, N)
    o = evo_ref.evo_attention_ref(q, k, v, mask, bias)
    assert torch.allclose(o, v, atol=1e-5)


def test_dbias_is_sum_over_rows_unscaled():
    """dBias = sum_s P o (dP - delta), without the softmax scale
    (evo_h100/tk_evoattention.cu:824-833)."""
    B, S, N, H, D = 1, 3, 10, 2, 8
    q, k, v, mask, bias, d_o = evo_ref.make_inputs(B, S, N, H, D, seed=4, mask_kind="bernoulli0.9")
    r = evo_ref.evo_attention_fwd_bwd_ref(q, k, v, mask, bias, d_o, dtype=torch.float64)
    qt, kt, vt, dot = (t.double().transpose(-2, -3) for t in (q, k, v, d_o))
    logits = (qt / math.sqrt(D)) @ kt.transpose(-1, -2) + bias.double() + mask.double()
    p = torch.softmax(logits, -1)
    dp = dot @ vt.transpose(-1, -2)
    delta = (dot * (p @ vt)).sum(-1, keepdim=True)
    ds = p * (dp - delta)
    assert torch.allclose(r["dbias"], ds.sum(dim=1, keepdim=True), atol=1e-12)
    assert torch.allclose(r["dq"].transpose(-2, -3), (ds @ kt) / math.sqrt(D), atol=1e-12)
    assert torch.allclose(r["dk"].transpose(-2, -3), (ds.transpose(-1, -2) @ qt) / math.sqrt(D), atol=1e-12)
    assert torch.allclose(r["dv"].transpose(-2, -3), p.transpose(-1, -2) @ dot, atol=1e-12)


def test_row_sharded_inputs_match_unsharded():
    full = evo_ref.make_workload("cfg3_triangle", S_override=8)
    lo = evo_ref.make_workload("cfg3_triangle", 0, 5, S_override=8)
    hi = evo_ref.make_workload("cfg3_triangle", 5, 8, S_override=8)
    for i in (0, 1, 2, 3, 5):     # q, k, v, mask, d_o are sharded over S
        assert torch.equal(torch.cat([lo[i], hi[i]], dim=1), full[i])
    assert torch.equal(lo[4], full[4]) and torch.equal(hi[4], full[4])   # bias replicated


def test_workload_shapes_and_flops():
    B, S, N, H, D = evo_ref.WORKLOADS["cfg2_msa_row"][:5]
    assert (B, S, N, H, D) == (1, 512, 384, 8, 32)
    assert abs(evo_ref.flops_fwd_bwd(B, S, N, H, D) - 2.706e11) / 2.706e11 < 1e-3
    assert abs(evo_ref.algorithmic_bytes(B, S, N, H, D) - 1.231e9) / 1.231e9 < 2e-3
    m = evo_ref.make_mask("tail10pct", 1, 2, 768, torch.Generator().manual_seed(0))
    assert int((m < 0).sum()) == 2 * 77


def test_gate_matches_manual_product_rule():
    """The gated form of the oracle: out = sigmoid(gate) * O; its gradients against the product rule
    applied by hand to the un-gated oracle."""
    B, S, N, H, D = 1, 2, 16, 2, 8
    q, k, v, mask, bias, d_out = evo_ref.make_inputs(B, S, N, H, D, 1.0, 1.0, "bernoulli0.9", seed=5)
    gate = torch.randn((B, S, N, H, D), generator=torch.Generator().manual_seed(6))
    got = evo_ref.evo_attention_fwd_bwd_ref(q, k, v, mask, bias, d_out, dtype=torch.float64, gate=gate)
    sig = torch.sigmoid(gate.double())
    plain = evo_ref.evo_attention_fwd_bwd_ref(q, k, v, mask, bias, d_out.double() * sig, dtype=torch.float64)
    assert torch.allclose(got["o"], plain["o"] * sig, atol=1e-12)
    for n in ("dq", "dk", "dv", "dbias"):
        assert torch.allclose(got[n], plain[n], atol=1e-10), n
    assert torch.allclose(got["dgate"], d_out.double() * plain["o"] * sig * (1 - sig), atol=1e-12)
