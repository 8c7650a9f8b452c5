"""Seeded synthetic workloads for EvoAttention: the five benchmark
configurations (shapes, value distributions, masks, seeds), the input
generator, and the algorithmic FLOP / byte model.

These stand in for AlphaFold-3 / MegaFold MSA-row and triangle attention
shapes; no dataset is involved.  All draws come from CPU generators, so a GPU
run and a CPU check see identical values, and every S row has its own
sub-seed, so a rank can materialise just its shard of rows.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

WORKLOADS = {
    # name: (B, S, N, H, D, qkv_std, bias_std, mask kind)
    "cfg1_cpu_fp32":      (1, 32, 64, 4, 32, 1.0, 1.0, "bernoulli0.9"),
    "cfg2_msa_row":       (1, 512, 384, 8, 32, 0.5, 1.0, "tail0to32"),
    "cfg3_triangle":      (1, 384, 384, 4, 32, 0.5, 1.0, "valid"),
    "cfg4_large_msa":     (1, 1024, 768, 8, 32, 0.5, 2.0, "tail10pct"),
    "cfg5_long_triangle": (1, 1024, 1024, 4, 64, 0.5, 1.0, "bernoulli0.95"),
    # not benchmark configurations: the two wide head dims of the reference's kernels and test grids
    # (evo_h100/test_tk_evoattention.py:89-95) at a size that fills the GPU, for timing them
    "wide_d128":          (1, 128, 768, 4, 128, 0.5, 1.0, "tail10pct"),
    "wide_d96":           (1, 128, 768, 4, 96, 0.5, 1.0, "tail10pct"),
}
WORKLOAD_SEEDS = {"cfg1_cpu_fp32": 1001, "cfg2_msa_row": 1002, "cfg3_triangle": 1003,
                  "cfg4_large_msa": 1004, "cfg5_long_triangle": 1005, "wide_d128": 1006, "wide_d96": 1007}


def make_mask(kind: str, B: int, S: int, N: int, gen: torch.Generator) -> torch.Tensor:
    """Additive residue mask [B,S,1,1,N] fp32: 0 valid, -1e9 padded
    (evo_h100/test_tk_evoattention.py:37-39)."""
    valid = torch.ones((B, S, N), dtype=torch.bool)
    if kind == "valid":
        pass
    elif kind.startswith("bernoulli"):
        p = float(kind[len("bernoulli"):])
        valid = torch.rand((B, S, N), generator=gen) < p
        valid[..., 0] = True                       # residue 0 forced valid
    elif kind == "tail0to32":
        for b in range(B):
            t = int(torch.randint(0, 33, (1,), generator=gen).item())
            if t:
                valid[b, :, N - t:] = False
    elif kind == "tail10pct":
        t = int(math.ceil(0.1 * N))
        valid[:, :, N - t:] = False
    elif kind == "randint":                        # the reference tests' own mask draw
        valid = torch.randint(0, 2, (B, S, N), generator=gen).bool()
        valid[..., 0] = True
    else:
        raise ValueError(kind)
    m = torch.where(valid, torch.zeros(()), torch.full((), -1e9))
    return m.reshape(B, S, 1, 1, N).to(torch.float32)


def make_inputs(B, S, N, H, D, qkv_std=1.0, bias_std=1.0, mask_kind="valid",
                seed=0, s_lo: int = 0, s_hi: Optional[int] = None):
    """fp32 CPU tensors (q, k, v, res_mask, pair_bias, d_o) drawn from a CPU
    generator so that the GPU run and the CPU oracle see identical values.

    `s_lo:s_hi` selects a contiguous shard of the S axis: each S row is drawn
    from its own sub-seed, so any rank can materialise just its rows and the
    union over ranks equals the unsharded draw."""
    if s_hi is None:
        s_hi = S
    g = torch.Generator().manual_seed(seed)
    bias = torch.randn((B, 1, H, N, N), generator=g) * bias_std
    mask = make_mask(mask_kind, B, S, N, g)[:, s_lo:s_hi].contiguous()
    rows = s_hi - s_lo
    q = torch.empty((B, rows, N, H, D))
    k = torch.empty_like(q)
    v = torch.empty_like(q)
    d_o = torch.empty_like(q)
    for s in range(s_lo, s_hi):
        gs = torch.Generator().manual_seed(seed * 1_000_003 + 17 * s + 1)
        blk = torch.randn((4, B, N, H, D), generator=gs)
        q[:, s - s_lo] = blk[0] * qkv_std
        k[:, s - s_lo] = blk[1] * qkv_std
        v[:, s - s_lo] = blk[2] * qkv_std
        d_o[:, s - s_lo] = blk[3]
    return q, k, v, mask, bias, d_o


def make_workload(name: str, s_lo: int = 0, s_hi: Optional[int] = None,
                  S_override: Optional[int] = None):
    B, S, N, H, D, qs, bs, mk = WORKLOADS[name]
    if S_override is not None:
        S = S_override
    return make_inputs(B, S, N, H, D, qs, bs, mk, WORKLOAD_SEEDS[name], s_lo, s_hi)


def flops_fwd_bwd(B, S, N, H, D) -> float:
    """Algorithmic FLOPs: fwd 4, bwd 10 per (B,S,H) N^2 D (evo_h100/benchmark.py:49-56)."""
    return 14.0 * B * S * H * N * N * D


def algorithmic_bytes(B, S, N, H, D) -> float:
    E = B * S * N * H * D
    return 24.0 * E + 8.0 * B * S * H * N + 8.0 * B * H * N * N + 4.0 * B * S * N
