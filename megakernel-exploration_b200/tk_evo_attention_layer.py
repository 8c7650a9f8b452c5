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
  * head dims 16, 32 and 64 run without any padding copy (16 on the D=32 kernels,
    whose loads zero-fill and whose stores clip the missing columns); other D <= 64
    are zero-padded up to the next of those here; D=96/128 raise ValueError (the
    reference pads them to 128, layer.py:47-56);
  * d_pair_bias is accumulated in fp32 and returned in the dtype of pair_bias
    (the reference rounds it to bf16 first, layer.py:176);
  * an optional sixth argument `process_group` shards the independent N_SEQ axis
    over ranks: every rank passes its own rows of Q/K/V/res_mask and the full
    (replicated) pair_bias, and backward all-reduces d_pair_bias over the group;
  * an optional seventh argument `gate` (the shape of Q: the logits of the sigmoid
    gate that follows this attention in the AlphaFold-3 / MegaFold blocks) makes the
    call return sigmoid(gate) * O, formed in the forward kernel's epilogue, and
    backward return the gate's gradient as well.

HostStreamedEvoAttention (end of this file) is an addition without a reference
counterpart: forward + backward for callers whose tensors live in host memory,
with the copies overlapped with the kernels.

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

# SMs the dQ/dK/dV kernel leaves to the d_pair_bias all-reduce that runs beside it.  The collective
# only overlaps if its kernel fits on them: create the process group with new_dbias_group() (or run
# with NCCL_MAX_CTAS set to this number).  Measured on 8 B200s, config 4 split over S: 1.55 ms per
# step without the reservation, 1.48 ms with 4 SMs and 4 collective CTAs; with more collective CTAs
# than reserved SMs the reservation only costs (1.56-1.60 ms).  On 2 B200s, 512 rows of config 2 per
# GPU: 1.337 ms per step without the reservation (the small-CTA collective then runs after the
# kernel), 1.287 ms with it; config 4 split in two 4.50 against 4.31 ms.
ALLREDUCE_RESERVED_SMS = int(os.environ.get("EVO_ALLREDUCE_RESERVED_SMS", "4"))
# smallest group for which SMs are reserved
ALLREDUCE_MIN_GROUP = int(os.environ.get("EVO_ALLREDUCE_MIN_GROUP", "2"))


def new_dbias_group(ranks=None, ctas: int = 0, timeout=None):
    """A process group for the d_pair_bias all-reduce whose NCCL kernels use at most `ctas` CTAs
    (default ALLREDUCE_RESERVED_SMS), so that they fit beside the dQ/dK/dV kernel.  Collective over
    all ranks of the default group, like torch.distributed.new_group.  `timeout` (a timedelta) is the
    group's limit for one collective: with it, a rank that never joins the backward's all-reduce ends
    the others' wait with an error instead of holding them for the backend's default half hour."""
    import torch.distributed as dist
    ctas = ctas or max(ALLREDUCE_RESERVED_SMS, 1)
    kw = {} if timeout is None else {"timeout": timeout}
    if dist.get_backend() == "nccl":
        opts = dist.ProcessGroupNCCL.Options()
        opts.config.max_ctas = ctas
        opts.config.min_ctas = 1
        return dist.new_group(ranks=ranks, pg_options=opts, **kw)
    return dist.new_group(ranks=ranks, **kw)

# Head dims the library takes as they are; others below 128 are zero-padded up to the next one.
TK_SUPPORTED_DIMS = (16, 32, 64, 96, 128)


def _next_supported_dim(d: int) -> int:
    for t in TK_SUPPORTED_DIMS:
        if d <= t:
            return t
    raise ValueError(
        f"head_dim {d} exceeds max supported head_dim {TK_SUPPORTED_DIMS[-1]}"
    )


def _bf16c(x: torch.Tensor) -> torch.Tensor:
    if x.dtype != torch.bfloat16:
        x = x.to(torch.bfloat16)
    return x.contiguous()


# bf16 copies of fp32 pair-bias tensors: a model calls the layer with the same pair bias for every
# block of a stack and, in evaluation, for every step, and the fp32 -> bf16 cast is the single largest
# cost the reference measured around its forward (evo_h100/README.md:655-669).  An entry is served only
# to the very tensor object it was made from (held by weak reference, so a new tensor that happens to
# reuse the address of a freed one never matches) and only while its version counter, which every
# in-place write bumps, is unchanged.
_BIAS_CACHE: "dict[int, tuple]" = {}
_BIAS_CACHE_MAX = 8


def _bias_bf16(pair_bias: torch.Tensor, B: int, H: int, N: int) -> torch.Tensor:
    """pair_bias (B, 1, H, N, N) as a contiguous bf16 (B, H, N, N) tensor, cast at most once per version."""
    import weakref
    pb = pair_bias.reshape(B, H, N, N)
    if pb.dtype == torch.bfloat16:
        return pb.contiguous()
    key = id(pair_bias)
    hit = _BIAS_CACHE.get(key)
    if hit is not None and hit[0]() is pair_bias and hit[1] == pair_bias._version:
        return hit[2]
    out = pb.detach().to(torch.bfloat16).contiguous()
    for k in [k for k, v in _BIAS_CACHE.items() if v[0]() is None]:      # entries of dead tensors
        del _BIAS_CACHE[k]
    if len(_BIAS_CACHE) >= _BIAS_CACHE_MAX:
        _BIAS_CACHE.pop(next(iter(_BIAS_CACHE)))
    _BIAS_CACHE[key] = (weakref.ref(pair_bias), pair_bias._version, out)
    return out


def _shared_view_strides(Q, K, V):
    """Strides (elements) if Q, K, V are bf16 views that the kernels can read in place: identical
    strides, contiguous head dim, 16-byte-aligned steps, (B, N_SEQ) flattenable, and DENSE (a
    permutation of a contiguous tensor: no holes, no overlap).  None for contiguous tensors (the
    plain path) and for anything else (which is copied).  A view with holes -- q, k, v chunked out
    of one fused projection, for instance -- is copied: outputs allocated with its strides would
    carry the holes along and O would come back non-contiguous where the reference's never is."""
    if Q.is_contiguous() or any(t.dtype != torch.bfloat16 for t in (Q, K, V)):
        return None
    st = Q.stride()
    if K.stride() != st or V.stride() != st or st[4] != 1:
        return None
    B, S = Q.shape[0], Q.shape[1]
    for ext, s in zip(Q.shape[:4], st[:4]):
        if ext > 1 and (s <= 0 or s % 8 != 0):
            return None
    if B > 1 and S > 1 and st[0] != S * st[1]:
        return None
    # dense: sorted by stride, every axis of extent > 1 steps by exactly the span of the inner ones
    span = 1
    for s_, ext in sorted((s_, ext) for s_, ext in zip(st, Q.shape) if ext > 1):
        if s_ != span:
            return None
        span *= ext
    if any(t.data_ptr() % 16 for t in (Q, K, V)):
        return None
    return tuple(st)


def _inplace_view_strides(Q, K, V):
    """Strides (elements) if Q, K, V are bf16 views that the kernels can READ in place: identical
    strides, contiguous head dim, 16-byte-aligned steps, (B, N_SEQ) flattenable, no overlap inside a
    tensor.  Holes are fine: q, k, v sliced out of one fused projection [B, N_SEQ, N_CTX, 3, H, D]
    qualify, and are read where they lie while O and the gradients are written contiguously (the
    reference copies each of them twice, transpose and pad, layer.py:81-102).  None otherwise."""
    if any(t.dtype != torch.bfloat16 for t in (Q, K, V)):
        return None
    st = Q.stride()
    if K.stride() != st or V.stride() != st or st[4] != 1:
        return None
    B, S = Q.shape[0], Q.shape[1]
    for ext, s_ in zip(Q.shape[:4], st[:4]):
        if ext > 1 and (s_ <= 0 or s_ % 8 != 0):
            return None
    if B > 1 and S > 1 and st[0] != S * st[1]:
        return None
    span = 1
    for s_, ext in sorted((s_, ext) for s_, ext in zip(st, Q.shape) if ext > 1):
        if s_ < span:
            return None
        span = s_ * ext
    if any(t.data_ptr() % 16 for t in (Q, K, V)):
        return None
    return tuple(st)


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
    def forward(ctx, Q, K, V, res_mask, pair_bias, process_group=None, gate=None):
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
        if gate is not None:
            assert gate.shape == (B, N_SEQ, N_CTX, H, D), f"gate shape mismatch: {gate.shape}"
            if padded_D != D:
                raise ValueError(f"the fused gate needs a head dim the library takes as it is {TK_SUPPORTED_DIMS}, got {D}")
        if N_CTX % 8 != 0:
            raise ValueError(f"N_CTX must be a multiple of 8, got {N_CTX}")

        # Views such as the "ending node" triangle attention (N_SEQ and N_CTX swapped in memory) are
        # read and written in place; the reference transposes and copies (layer.py:81-102).
        strides = _shared_view_strides(Q, K, V) if padded_D == D else None
        # Views with holes (q, k, v sliced out of a fused projection) are read in place as well; only
        # the tensors this call allocates are then contiguous.
        in_strides = strides
        if strides is None and padded_D == D and not Q.is_contiguous():
            in_strides = _inplace_view_strides(Q, K, V)
        q, k, v = (Q, K, V) if in_strides is not None else (_bf16c(Q), _bf16c(K), _bf16c(V))
        if padded_D != D:
            pad = padded_D - D
            q = F.pad(q, (0, pad)).contiguous()
            k = F.pad(k, (0, pad)).contiguous()
            v = F.pad(v, (0, pad)).contiguous()
        bias = _bias_bf16(pair_bias, B, H, N_CTX)
        mask = _bf16c(res_mask.reshape(B, N_SEQ, N_CTX))

        # softmax_scale is 1/sqrt(true D), not 1/sqrt(padded D) (reference layer.py:105)
        softmax_scale = 1.0 / (D ** 0.5)

        like = (lambda: torch.empty_strided(q.shape, strides, dtype=q.dtype, device=q.device)) \
            if strides is not None else (lambda: torch.empty(q.shape, dtype=q.dtype, device=q.device))
        o = like()
        g = o_gated = None
        if gate is not None:
            # the gate travels in the layout of q
            same_layout = (tuple(gate.stride()) == strides) if strides is not None else gate.is_contiguous()
            if gate.dtype == torch.bfloat16 and same_layout and gate.data_ptr() % 16 == 0:
                g = gate
            else:
                g = like()
                g.copy_(gate)
            o_gated = like()
        # rounding residual of O, kept for backward only (accurate delta -> accurate dBias)
        o_resid = like() if any(ctx.needs_input_grad) else None
        lse = torch.empty((B, N_SEQ, H, N_CTX), dtype=torch.float32, device=q.device)
        dims = _evoattn.EvoDims(B, N_SEQ, N_CTX, H, padded_D)
        with _device_ctx(q):
            st_ = _evoattn.EvoStrides(*strides[:4]) if strides is not None else None
            if in_strides != strides:
                _evoattn.fwd_views(dims, _evoattn.EvoStrides(*in_strides[:4]), st_, q, k, v, bias, mask, g, o, o_gated,
                                   o_resid, lse, softmax_scale, _stream())
            elif g is not None:
                _evoattn.fwd_gated(dims, st_, q, k, v, bias, mask, g, o, o_gated, o_resid, lse, softmax_scale, _stream())
            elif strides is not None:
                _evoattn.fwd_strided(dims, st_, q, k, v, bias, mask, o, o_resid, lse, softmax_scale, _stream())
            else:
                _evoattn.fwd(dims, q, k, v, bias, mask, o, o_resid, lse, softmax_scale, _stream())
        ctx.strides = strides
        ctx.in_strides = in_strides
        ctx.gated = g is not None

        if g is not None:
            ctx.save_for_backward(q, k, v, bias, mask, o, o_resid, lse, g)
        else:
            ctx.save_for_backward(q, k, v, bias, mask, o, o_resid, lse)
        ctx.softmax_scale = softmax_scale
        ctx.true_D = D
        ctx.padded_D = padded_D
        ctx.dims = (B, N_SEQ, N_CTX, H)
        ctx.bias_dtype = pair_bias.dtype
        ctx.process_group = process_group
        ctx.n_inputs = 7 if gate is not None else (6 if process_group is not None else 5)
        if g is not None:
            return o_gated
        return o[..., :D].contiguous() if padded_D != D else o

    @staticmethod
    def backward(ctx, dO):
        if ctx.gated:
            q, k, v, bias, mask, o, o_resid, lse, g = ctx.saved_tensors
        else:
            q, k, v, bias, mask, o, o_resid, lse = ctx.saved_tensors
            g = None
        B, N_SEQ, N_CTX, H = ctx.dims
        D, padded_D = ctx.true_D, ctx.padded_D

        strides = ctx.strides
        if strides is not None:
            like = lambda: torch.empty_strided(q.shape, strides, dtype=q.dtype, device=q.device)
            if dO.dtype == torch.bfloat16 and tuple(dO.stride()) == strides and dO.data_ptr() % 16 == 0:
                d_o = dO
            else:
                d_o = like()
                d_o.copy_(dO)
        else:
            like = lambda: torch.empty(q.shape, dtype=q.dtype, device=q.device)
            d_o = _bf16c(dO)
            if padded_D != D:
                d_o = F.pad(d_o, (0, padded_D - D)).contiguous()

        dq, dk, dv = like(), like(), like()
        d_gate = like() if g is not None else None
        dbias = torch.empty((B, H, N_CTX, N_CTX), dtype=torch.float32, device=q.device)
        dims = _evoattn.EvoDims(B, N_SEQ, N_CTX, H, padded_D)
        ws_bytes = _evoattn.bwd_gated_workspace_bytes(dims) if g is not None else _evoattn.bwd_workspace_bytes(dims)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
        st_ = _evoattn.EvoStrides(*strides[:4]) if strides is not None else None
        args = (dims, st_, q, k, v, bias, mask, o, o_resid, lse, d_o, dq, dk, dv, dbias, ws, ctx.softmax_scale)
        with _device_ctx(q):
            if ctx.in_strides != strides:
                # q, k, v read through their own view; everything else in the layout of `strides`
                import torch.distributed as dist
                vargs = (dims, _evoattn.EvoStrides(*ctx.in_strides[:4]), st_, st_, q, k, v, bias, mask, g, o, o_resid,
                         lse, d_o, dq, dk, dv, d_gate, dbias, ws, ctx.softmax_scale)
                if ctx.process_group is None:
                    _evoattn.bwd_views(*vargs, _evoattn.BWD_PHASE_DBIAS | _evoattn.BWD_PHASE_DQKV, 0, _stream())
                else:
                    _evoattn.bwd_views(*vargs, _evoattn.BWD_PHASE_DBIAS, 0, _stream())
                    work = dist.all_reduce(dbias, op=dist.ReduceOp.SUM, group=ctx.process_group, async_op=True)
                    reserve = ALLREDUCE_RESERVED_SMS if dist.get_world_size(ctx.process_group) >= ALLREDUCE_MIN_GROUP else 0
                    _evoattn.bwd_views(*vargs, _evoattn.BWD_PHASE_DQKV, reserve, _stream())
                    work.wait()
            elif g is not None:
                both = _evoattn.BWD_PHASE_DBIAS | _evoattn.BWD_PHASE_DQKV
                gargs = (dims, st_, q, k, v, bias, mask, g, o, o_resid, lse, d_o, dq, dk, dv, d_gate, dbias, ws,
                         ctx.softmax_scale)
                if ctx.process_group is None:
                    _evoattn.bwd_gated(*gargs, both, 0, _stream())
                else:
                    import torch.distributed as dist
                    _evoattn.bwd_gated(*gargs, _evoattn.BWD_PHASE_DBIAS, 0, _stream())
                    work = dist.all_reduce(dbias, op=dist.ReduceOp.SUM, group=ctx.process_group, async_op=True)
                    reserve = ALLREDUCE_RESERVED_SMS if dist.get_world_size(ctx.process_group) >= ALLREDUCE_MIN_GROUP else 0
                    _evoattn.bwd_gated(*gargs, _evoattn.BWD_PHASE_DQKV, reserve, _stream())
                    work.wait()
            elif ctx.process_group is None:
                _evoattn.bwd_phased(*args, _evoattn.BWD_PHASE_DBIAS | _evoattn.BWD_PHASE_DQKV, 0, _stream())
            else:
                # Rows of N_SEQ are sharded over the group and pair_bias is replicated: d_pair_bias is
                # summed over the ranks.  It is complete after the first phase, so its all-reduce runs
                # (on the collective's own stream, on the SMs the second phase leaves free) while
                # dQ/dK/dV are computed.
                import torch.distributed as dist
                _evoattn.bwd_phased(*args, _evoattn.BWD_PHASE_DBIAS, 0, _stream())
                work = dist.all_reduce(dbias, op=dist.ReduceOp.SUM, group=ctx.process_group, async_op=True)
                reserve = ALLREDUCE_RESERVED_SMS if dist.get_world_size(ctx.process_group) >= ALLREDUCE_MIN_GROUP else 0
                _evoattn.bwd_phased(*args, _evoattn.BWD_PHASE_DQKV, reserve, _stream())
                work.wait()

        if padded_D != D:
            dq, dk, dv = (t[..., :D].contiguous() for t in (dq, dk, dv))
        d_pair_bias = dbias.unsqueeze(1)
        if ctx.bias_dtype != torch.float32:
            d_pair_bias = d_pair_bias.to(ctx.bias_dtype)
        grads = (dq, dk, dv, None, d_pair_bias)
        if ctx.n_inputs == 7:
            return grads + (None, d_gate)
        return grads + (None,) if ctx.n_inputs == 6 else grads


class EvoAttention(torch.nn.Module):
    """Module form of TKEvoAttention; `process_group` shards N_SEQ over ranks."""

    def __init__(self, process_group=None):
        super().__init__()
        self.process_group = process_group

    def forward(self, Q, K, V, res_mask, pair_bias, gate=None):
        if gate is not None:
            return TKEvoAttention.apply(Q, K, V, res_mask, pair_bias, self.process_group, gate)
        if self.process_group is None:
            return TKEvoAttention.apply(Q, K, V, res_mask, pair_bias)
        return TKEvoAttention.apply(Q, K, V, res_mask, pair_bias, self.process_group)


class HostStreamedEvoAttention:
    """Forward + backward for callers whose tensors live in HOST memory.

    The reference has no such entry point: its callers hold device tensors and its
    benchmark times device-resident calls only (evo_h100/benchmark.py:76-124).  A
    host-buffer caller that simply copies everything in, runs the layer and copies
    everything out spends ten times longer on the two copies than on the kernels,
    and the copies do not overlap.  Rows of N_SEQ are independent problems, so this
    class cuts N_SEQ into chunks and runs three streams: chunk c+1 is copied in
    while chunk c is computed and chunk c-1 is copied out (both PCIe directions
    busy at once); d_pair_bias is summed over the chunks on the device and copied
    out once.

        eng = HostStreamedEvoAttention(device, chunk_rows=64)
        eng.run(q, k, v, res_mask, pair_bias, dO, out)   # all host tensors

    q, k, v, dO: bf16 (B, N_SEQ, N_CTX, H, D), D in TK_SUPPORTED_DIMS; res_mask: bf16
    (B, N_SEQ, 1, 1, N_CTX) or (B, N_SEQ, N_CTX); pair_bias: bf16 (B, 1, H, N, N) or
    (B, H, N, N).  `out` = dict(o, dq, dk, dv: bf16 like q; dbias: fp32 like
    pair_bias).  Host tensors should be pinned (page-locked), otherwise the copies
    are synchronous.  With `process_group`, every rank passes its own rows and the
    full pair_bias; d_pair_bias is all-reduced before it is copied out.
    """

    def __init__(self, device, chunk_rows: int = 64, process_group=None):
        self.dev = torch.device(device)
        if self.dev.type != "cuda":
            raise RuntimeError("HostStreamedEvoAttention needs a CUDA device: there is no CPU path")
        self.chunk_rows = int(chunk_rows)
        self.pg = process_group
        self.s_in, self.s_cmp, self.s_out = (torch.cuda.Stream(self.dev) for _ in range(3))
        self._key = None

    def _buffers(self, B, N, H, D):
        key = (B, N, H, D)
        if self._key == key:
            return
        R, dev, bf = self.chunk_rows, self.dev, torch.bfloat16
        dims = _evoattn.EvoDims(1, R, N, H, D)
        self.sets = []
        for _ in range(2):
            s = {n: torch.empty((1, R, N, H, D), dtype=bf, device=dev)
                 for n in ("q", "k", "v", "do", "o", "ores", "dq", "dk", "dv")}
            s["mask"] = torch.empty((1, R, N), dtype=bf, device=dev)
            s["lse"] = torch.empty((1, R, H, N), dtype=torch.float32, device=dev)
            s["dbias"] = torch.empty((1, H, N, N), dtype=torch.float32, device=dev)
            s["ws"] = torch.empty(_evoattn.bwd_workspace_bytes(dims), dtype=torch.uint8, device=dev)
            s["ev_in"], s["ev_cmp"], s["ev_out"] = (torch.cuda.Event() for _ in range(3))
            self.sets.append(s)
        self.bias = torch.empty((B, H, N, N), dtype=bf, device=dev)
        self.dbias = torch.empty((B, H, N, N), dtype=torch.float32, device=dev)
        self._key = key

    def run(self, q, k, v, res_mask, pair_bias, d_o, out):
        B, S, N, H, D = q.shape
        if D not in TK_SUPPORTED_DIMS:
            raise ValueError(f"head_dim {D}: the host-streamed path takes D in {TK_SUPPORTED_DIMS}")
        for t in (q, k, v, d_o):
            assert t.shape == (B, S, N, H, D) and t.dtype == torch.bfloat16 and not t.is_cuda
        mask = res_mask.reshape(B, S, N)
        bias = pair_bias.reshape(B, H, N, N)
        assert mask.dtype == torch.bfloat16 and bias.dtype == torch.bfloat16
        dbias_out = out["dbias"].reshape(B, H, N, N)
        self._buffers(B, N, H, D)
        R = self.chunk_rows
        cur = torch.cuda.current_stream(self.dev)
        for s_ in (self.s_in, self.s_cmp, self.s_out):
            s_.wait_stream(cur)
        with torch.cuda.stream(self.s_in):
            self.bias.copy_(bias, non_blocking=True)
        with torch.cuda.stream(self.s_cmp):
            self.dbias.zero_()
        c = 0
        for b in range(B):
            for s0 in range(0, S, R):
                r = min(R, S - s0)
                st = self.sets[c & 1]
                dims = _evoattn.EvoDims(1, r, N, H, D)
                with torch.cuda.stream(self.s_in):
                    if c >= 2:
                        self.s_in.wait_event(st["ev_out"])      # this set's previous results are out
                    for n, h in (("q", q), ("k", k), ("v", v), ("do", d_o)):
                        st[n][:, :r].copy_(h[b:b + 1, s0:s0 + r], non_blocking=True)
                    st["mask"][:, :r].copy_(mask[b:b + 1, s0:s0 + r], non_blocking=True)
                    st["ev_in"].record(self.s_in)
                with torch.cuda.stream(self.s_cmp):
                    self.s_cmp.wait_event(st["ev_in"])
                    h_ = self.s_cmp.cuda_stream
                    # a chunk with fewer rows uses the leading rows of the (contiguous) buffers
                    _evoattn.fwd(dims, st["q"], st["k"], st["v"], self.bias[b:b + 1], st["mask"], st["o"],
                                 st["ores"], st["lse"], 0.0, h_)
                    _evoattn.bwd(dims, st["q"], st["k"], st["v"], self.bias[b:b + 1], st["mask"], st["o"],
                                 st["ores"], st["lse"], st["do"], st["dq"], st["dk"], st["dv"], st["dbias"],
                                 st["ws"], 0.0, h_)
                    self.dbias[b:b + 1].add_(st["dbias"])
                    st["ev_cmp"].record(self.s_cmp)
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(st["ev_cmp"])
                    for n in ("o", "dq", "dk", "dv"):
                        out[n][b:b + 1, s0:s0 + r].copy_(st[n][:, :r], non_blocking=True)
                    st["ev_out"].record(self.s_out)
                c += 1
        with torch.cuda.stream(self.s_cmp):
            if self.pg is not None:
                import torch.distributed as dist
                dist.all_reduce(self.dbias, group=self.pg)
            dbias_out.copy_(self.dbias, non_blocking=True)
        for s_ in (self.s_in, self.s_cmp, self.s_out):
            cur.wait_stream(s_)
