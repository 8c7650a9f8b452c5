"""torch.autograd.Function over the B200 EvoAttention kernels.

Drop-in for evo_h100/tk_evo_attention_layer.py of the reference: same module
name, same class, same call

    O = TKEvoAttention.apply(Q, K, V, res_mask, pair_bias)

Input shapes (reference layer.py:5-11):
    Q, K, V   : (B, N_SEQ, N_CTX, H, D)   bf16 (other float dtypes are cast)
    res_mask  : (B, N_SEQ, 1, 1, N_CTX)   additive; any dtype, cast to bf16
    pair_bias : (B, 1, H, N_CTX, N_CTX)   any float, cast to bf16
Output:
    O         : (B, N_SEQ, N_CTX, H, D)   bf16
Backward returns (dQ, dK, dV, None, d_pair_bias) in the caller layouts
(reference layer.py:180); there is no gradient for the mask.

Differences from the reference, all internal:
  * the kernels read and write the caller layout directly, so there are no
    transposes and no zero-padding of D (reference layer.py:81-102,112-113);
  * native head dims are 32 and 64; D=16 is zero-padded to 32 here; D=96/128
    raise ValueError (the reference pads them to 128, layer.py:47-56);
  * d_pair_bias is accumulated in fp32 and returned in the dtype of pair_bias
    (the reference rounds it to bf16 first, layer.py:176);
  * an optional sixth argument `process_group` shards the independent N_SEQ axis
    over ranks: every rank passes its own rows of Q/K/V/res_mask and the full
    (replicated) pair_bias, and backward all-reduces d_pair_bias over the group.

There is no CPU or eager fallback: without libevoattn.so and a CUDA device this
module raises.
"""
from __future__ import annotations

import os
import sys

import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
if HERE not in sys.path:
    sys.path.insert(0, HERE)

import _evoattn  # noqa: E402  (ctypes binding of libevoattn.so)

# Head dims the kernels support natively; smaller ones are zero-padded up.
TK_SUPPORTED_DIMS = (32, 64)


def _next_supported_dim(d: int) -> int:
    for t in TK_SUPPORTED_DIMS:
        if d <= t:
            return t
    raise ValueError(
        f"head_dim {d} exceeds max supported head_dim {TK_SUPPORTED_DIMS[-1]} "
        f"(D=96/128 are not yet supported by the sm_100a kernels)"
    )


def _bf16c(x: torch.Tensor) -> torch.Tensor:
    if x.dtype != torch.bfloat16:
        x = x.to(torch.bfloat16)
    return x.contiguous()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check_device(t: torch.Tensor) -> None:
    if not t.is_cuda:
        raise RuntimeError("TKEvoAttention needs CUDA tensors (there is no CPU path)")


def _device_ctx(t: torch.Tensor):
    return torch.cuda.device(t.device)


class TKEvoAttention(torch.autograd.Function):
    """Evo / triangle attention: softmax(Q K^T / sqrt(D) + pair_bias + res_mask) V."""

    @staticmethod
    def forward(ctx, Q, K, V, res_mask, pair_bias, process_group=None):
        B, N_SEQ, N_CTX, H, D = Q.shape
        assert K.shape == (B, N_SEQ, N_CTX, H, D), f"K shape mismatch: {K.shape}"
        assert V.shape == (B, N_SEQ, N_CTX, H, D), f"V shape mismatch: {V.shape}"
        assert res_mask.shape == (B, N_SEQ, 1, 1, N_CTX), (
            f"res_mask shape mismatch: expected (B,N_SEQ,1,1,N_CTX)={(B, N_SEQ, 1, 1, N_CTX)}, got {res_mask.shape}"
        )
        assert pair_bias.shape == (B, 1, H, N_CTX, N_CTX), (
            f"pair_bias shape mismatch: expected (B,1,H,N,N)={(B, 1, H, N_CTX, N_CTX)}, got {pair_bias.shape}"
        )
        padded_D = _next_supported_dim(D)
        _check_device(Q)
        if N_CTX % 8 != 0:
            raise ValueError(f"N_CTX must be a multiple of 8, got {N_CTX}")

        q, k, v = _bf16c(Q), _bf16c(K), _bf16c(V)
        if padded_D != D:
            pad = padded_D - D
            q = F.pad(q, (0, pad)).contiguous()
            k = F.pad(k, (0, pad)).contiguous()
            v = F.pad(v, (0, pad)).contiguous()
        bias = _bf16c(pair_bias.reshape(B, H, N_CTX, N_CTX))
        mask = _bf16c(res_mask.reshape(B, N_SEQ, N_CTX))

        # softmax_scale is 1/sqrt(true D), not 1/sqrt(padded D) (reference layer.py:105)
        softmax_scale = 1.0 / (D ** 0.5)

        o = torch.empty_like(q)
        # rounding residual of O, kept for backward only (accurate delta -> accurate dBias)
        o_resid = torch.empty_like(q) if any(ctx.needs_input_grad) else None
        lse = torch.empty((B, N_SEQ, H, N_CTX), dtype=torch.float32, device=q.device)
        dims = _evoattn.EvoDims(B, N_SEQ, N_CTX, H, padded_D)
        with _device_ctx(q):
            _evoattn.fwd(dims, q, k, v, bias, mask, o, o_resid, lse, softmax_scale, _stream())

        ctx.save_for_backward(q, k, v, bias, mask, o, o_resid, lse)
        ctx.softmax_scale = softmax_scale
        ctx.true_D = D
        ctx.padded_D = padded_D
        ctx.dims = (B, N_SEQ, N_CTX, H)
        ctx.bias_dtype = pair_bias.dtype
        ctx.process_group = process_group
        ctx.n_inputs = 6 if process_group is not None else 5
        return o[..., :D].contiguous() if padded_D != D else o

    @staticmethod
    def backward(ctx, dO):
        q, k, v, bias, mask, o, o_resid, lse = ctx.saved_tensors
        B, N_SEQ, N_CTX, H = ctx.dims
        D, padded_D = ctx.true_D, ctx.padded_D

        d_o = _bf16c(dO)
        if padded_D != D:
            d_o = F.pad(d_o, (0, padded_D - D)).contiguous()

        dq = torch.empty_like(q)
        dk = torch.empty_like(q)
        dv = torch.empty_like(q)
        dbias = torch.empty((B, H, N_CTX, N_CTX), dtype=torch.float32, device=q.device)
        dims = _evoattn.EvoDims(B, N_SEQ, N_CTX, H, padded_D)
        ws = torch.empty(_evoattn.bwd_workspace_bytes(dims), dtype=torch.uint8, device=q.device)
        with _device_ctx(q):
            _evoattn.bwd(dims, q, k, v, bias, mask, o, o_resid, lse, d_o, dq, dk, dv, dbias, ws,
                         ctx.softmax_scale, _stream())

        if ctx.process_group is not None:
            # rows of N_SEQ are sharded over the group; pair_bias is replicated
            import torch.distributed as dist
            dist.all_reduce(dbias, op=dist.ReduceOp.SUM, group=ctx.process_group)

        if padded_D != D:
            dq, dk, dv = (t[..., :D].contiguous() for t in (dq, dk, dv))
        d_pair_bias = dbias.unsqueeze(1)
        if ctx.bias_dtype != torch.float32:
            d_pair_bias = d_pair_bias.to(ctx.bias_dtype)
        grads = (dq, dk, dv, None, d_pair_bias)
        return grads + (None,) if ctx.n_inputs == 6 else grads


class EvoAttention(torch.nn.Module):
    """Module form of TKEvoAttention; `process_group` shards N_SEQ over ranks."""

    def __init__(self, process_group=None):
        super().__init__()
        self.process_group = process_group

    def forward(self, Q, K, V, res_mask, pair_bias):
        if self.process_group is None:
            return TKEvoAttention.apply(Q, K, V, res_mask, pair_bias)
        return TKEvoAttention.apply(Q, K, V, res_mask, pair_bias, self.process_group)
