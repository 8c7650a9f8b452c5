"""CPU oracle for EvoAttention forward + backward (TEST INFRASTRUCTURE, not product).

PARITY UNPINNED: the reference tree holds no golden vectors, no known-answer
tests and no eager implementation of this path; its own tests compare against
a third-party Triton kernel that is not vendored.  This file restates the
documented math of the reference

    logits = (Q * softmax_scale) @ K^T + pair_bias + res_mask
    O      = softmax(logits, dim=-1) @ V

(evo_h100/README.md:29-40, evo_h100/tk_evoattention.cu:13-15) in eager PyTorch
on the caller layout of evo_h100/tk_evo_attention_layer.py:5-11, and is pinned
only by analytic known-answer cases, an fp64 self-check and an independent
cross-check against torch.nn.functional.scaled_dot_product_attention (see
tests/test_oracle.py), plus the committed fixtures under tests/golden/ that it
generated itself.

Only tests/, the smoke entry and the benchmark's cpu-baseline / reference arm
may import this module; the product path never does.

Layouts (B = batch, S = MSA / triangle rows, N = residues, H = heads, D = head dim):
    q, k, v   [B, S, N, H, D]
    res_mask  [B, S, 1, 1, N]   additive (0 valid, -1e9 padded)
    pair_bias [B, 1, H, N, N]   broadcast over S
    o         [B, S, N, H, D]
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch


def _scale(D: int, softmax_scale: Optional[float]) -> float:
    # evo_h100/tk_evoattention.cu:988-990 -- a scale <= 0 means 1/sqrt(head_dim);
    # evo_h100/tk_evo_attention_layer.py:105 -- the layer always passes 1/sqrt(true D).
    if softmax_scale is None or softmax_scale <= 0.0:
        return 1.0 / math.sqrt(D)
    return float(softmax_scale)


def evo_attention_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                      res_mask: torch.Tensor, pair_bias: torch.Tensor,
                      softmax_scale: Optional[float] = None,
                      dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Eager forward in `dtype` (fp32 or fp64); differentiable.

    Follows evo_h100/README.md:29-40: transpose to [B,S,H,N,D]
    (tk_evo_attention_layer.py:81-88), logits = (q*scale) @ k^T + bias + mask,
    softmax over the kv axis, times v, transpose back (layer.py:112-113).
    """
    B, S, N, H, D = q.shape
    sc = _scale(D, softmax_scale)
    qt = q.to(dtype).transpose(-2, -3)          # [B,S,H,N,D]
    kt = k.to(dtype).transpose(-2, -3)
    vt = v.to(dtype).transpose(-2, -3)
    logits = torch.matmul(qt * sc, kt.transpose(-1, -2))     # [B,S,H,N,N]
    logits = logits + pair_bias.to(dtype) + res_mask.to(dtype)
    p = torch.softmax(logits, dim=-1)
    o = torch.matmul(p, vt)                                  # [B,S,H,N,D]
    return o.transpose(-2, -3).contiguous()


def evo_lse_ref(q, k, res_mask, pair_bias, softmax_scale=None,
                dtype=torch.float32) -> torch.Tensor:
    """Natural-log log-sum-exp of the logits, [B,S,H,N] (evo_h100/README.md:244-252)."""
    B, S, N, H, D = q.shape
    sc = _scale(D, softmax_scale)
    qt = q.to(dtype).transpose(-2, -3)
    kt = k.to(dtype).transpose(-2, -3)
    logits = torch.matmul(qt * sc, kt.transpose(-1, -2))
    logits = logits + pair_bias.to(dtype) + res_mask.to(dtype)
    return torch.logsumexp(logits, dim=-1)


def evo_attention_fwd_bwd_ref(q, k, v, res_mask, pair_bias, d_o,
                              softmax_scale=None, dtype=torch.float32,
                              s_chunk: int = 32, gate=None) -> Dict[str, torch.Tensor]:
    """Forward + backward through autograd, chunked over S to bound memory.

    With `gate` (the shape of q) the output is sigmoid(gate) * O, the gating that follows
    this attention in the AlphaFold-3 / MegaFold blocks (the reference applies it outside
    its kernel); d_o is then the gradient of that gated output, "o" in the result is the
    gated output and "dgate" the gradient of the gate logits.

    Rows of S are independent attention problems that share only the read-only
    pair bias, so dBias is the sum of the per-chunk bias gradients
    (dBias = sum_s P o (dP - Delta), unscaled: evo_h100/README.md:410-414,
    evo_h100/tk_evoattention.cu:824-833).  No gradient for the mask
    (tk_evo_attention_layer.py:180).

    Returns fp32/fp64 tensors: o, dq, dk, dv [B,S,N,H,D], dbias [B,1,H,N,N].
    """
    B, S, N, H, D = q.shape
    o = torch.empty((B, S, N, H, D), dtype=dtype)
    dq = torch.empty_like(o)
    dk = torch.empty_like(o)
    dv = torch.empty_like(o)
    dbias = torch.zeros((B, 1, H, N, N), dtype=dtype)
    dgate = torch.empty_like(o) if gate is not None else None
    for s0 in range(0, S, s_chunk):
        s1 = min(S, s0 + s_chunk)
        qc = q[:, s0:s1].detach().to(dtype).requires_grad_(True)
        kc = k[:, s0:s1].detach().to(dtype).requires_grad_(True)
        vc = v[:, s0:s1].detach().to(dtype).requires_grad_(True)
        bc = pair_bias.detach().to(dtype).requires_grad_(True)
        oc = evo_attention_ref(qc, kc, vc, res_mask[:, s0:s1], bc, softmax_scale, dtype)
        if gate is not None:
            gc = gate[:, s0:s1].detach().to(dtype).requires_grad_(True)
            oc = oc * torch.sigmoid(gc)
        oc.backward(d_o[:, s0:s1].to(dtype))
        if gate is not None:
            dgate[:, s0:s1] = gc.grad
        o[:, s0:s1] = oc.detach()
        dq[:, s0:s1] = qc.grad
        dk[:, s0:s1] = kc.grad
        dv[:, s0:s1] = vc.grad
        dbias += bc.grad
    out = {"o": o, "dq": dq, "dk": dk, "dv": dv, "dbias": dbias}
    if gate is not None:
        out["dgate"] = dgate
    return out


# ---------------------------------------------------------------------------
# parity metrics (the bar: max-abs <= 2e-2 and relative-L2 <= 1e-2 for bf16 inputs)
# ---------------------------------------------------------------------------
MAX_ABS_TOL = 2e-2
REL_L2_TOL = 1e-2


def max_abs_err(ref: torch.Tensor, got: torch.Tensor) -> float:
    return (ref.double() - got.double()).abs().max().item()


def rel_l2_err(ref: torch.Tensor, got: torch.Tensor) -> float:
    num = (ref.double() - got.double()).norm().item()
    den = ref.double().norm().item()
    return num / max(den, 1e-30)


def parity(ref: torch.Tensor, got: torch.Tensor) -> Tuple[float, float]:
    return max_abs_err(ref, got), rel_l2_err(ref, got)


# ---------------------------------------------------------------------------
# workloads: shapes, seeds, input generators and the FLOP / byte model live with
# the product (megakernel-exploration_b200/evo_workloads.py); re-exported here so
# tests can reach everything through the oracle.
# ---------------------------------------------------------------------------
import os as _os
import sys as _sys

_PKG = _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))),
                     "megakernel-exploration_b200")
if _PKG not in _sys.path:
    _sys.path.insert(0, _PKG)
from evo_workloads import (WORKLOADS, WORKLOAD_SEEDS, algorithmic_bytes, flops_fwd_bwd,  # noqa: E402,F401
                           make_inputs, make_mask, make_workload)
