"""The allocation-free backward entry point (evo_bwd_static_scratch).

Some hosts hand all device memory out up front -- a server whose pool owns the
GPU, a plugin inside such a process -- and then nothing may call the allocator.
For them the library carries its own fixed scratch array.  This test calls that
entry point through the C ABI twice in a row (the array keeps the previous
call's contents, so the second call checks that stale scratch does no harm) and
compares every output with the regular evo_bwd on the same inputs.  dK and dV
must agree bit for bit.  dQ and dBias are sums of fp32 reduce-adds whose order
can differ from launch to launch, so they are compared within 2^-7 (dQ, bf16)
and 1e-4 (dBias, fp32) -- the same slack the parity tests allow between two
runs of the regular entry point.  The second call runs a smaller problem than
the first, so the array still holds the larger problem's data beyond the new
extents, and the amount of free device memory is read before and after that
call: it must not move, which is the property the entry point exists for.  The
test also checks that an oversized problem is refused.

Collected last on purpose (file name), so that a failure here cannot hide the
result of any other test in a run that stops at the first failure.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(B, S, N, H, D, seed):
    from oracle import evo_ref
    q, k, v, mask, bias, d_o = evo_ref.make_inputs(B, S, N, H, D, 0.5, 1.0, "tail0to32", seed=seed)
    dev, bf = "cuda", torch.bfloat16
    return ([t.to(dev, bf) for t in (q, k, v, d_o)] +
            [bias.reshape(B, H, N, N).to(dev, bf), mask.reshape(B, S, N).to(dev, bf)])


def test_static_scratch_backward_matches_regular_backward():
    import _evoattn
    st = torch.cuda.current_stream().cuda_stream
    # ragged N, S not a multiple of the row chunk; the second problem is smaller than the first
    for call, (B, S, N, H, D) in enumerate([(1, 7, 264, 3, 32), (1, 4, 136, 2, 32)]):
        dims = _evoattn.EvoDims(B, S, N, H, D)
        assert _evoattn.bwd_workspace_bytes(dims) <= _evoattn.lib().evo_bwd_static_scratch_capacity()
        qd, kd, vd, dod, bd, md = _inputs(B, S, N, H, D, seed=100 + call)
        o, ores = torch.empty_like(qd), torch.empty_like(qd)
        lse = torch.empty((B, S, H, N), dtype=torch.float32, device="cuda")
        _evoattn.fwd(dims, qd, kd, vd, bd, md, o, ores, lse, 0.0, st)

        ref = [torch.empty_like(qd) for _ in range(3)] + [torch.empty((B, H, N, N), device="cuda")]
        ws = torch.empty(_evoattn.bwd_workspace_bytes(dims), dtype=torch.uint8, device="cuda")
        _evoattn.bwd(dims, qd, kd, vd, bd, md, o, ores, lse, dod, *ref, ws, 0.0, st)

        got = [torch.full_like(qd, float("nan")) for _ in range(3)] + \
              [torch.full((B, H, N, N), float("nan"), device="cuda")]
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        _evoattn.bwd_static_scratch(dims, qd, kd, vd, bd, md, o, ores, lse, dod, *got, 0.0, st)
        torch.cuda.synchronize()
        free_after = torch.cuda.mem_get_info()[0]
        _evoattn.device_status()
        if call > 0:
            # the first call on a device looks the array's address up (and may load the module's
            # data); from then on a call must leave the device's free memory exactly as it was
            assert free_after == free_before, f"device memory moved by {free_before - free_after} bytes"

        dq_r, dk_r, dv_r, db_r = ref
        dq_g, dk_g, dv_g, db_g = got
        assert torch.equal(dk_g, dk_r) and torch.equal(dv_g, dv_r), f"call {call}: dK/dV differ"
        assert (dq_g.float() - dq_r.float()).abs().max().item() <= 2.0 ** -7, f"call {call}: dQ"
        assert (db_g - db_r).abs().max().item() <= 1e-4, f"call {call}: dBias"
        assert torch.isfinite(db_g).all() and torch.isfinite(dq_g.float()).all()


def test_static_scratch_rejects_oversized_problem():
    import _evoattn
    big = _evoattn.EvoDims(1, 512, 384, 8, 32)          # needs ~210 MB of scratch
    assert _evoattn.bwd_workspace_bytes(big) > _evoattn.lib().evo_bwd_static_scratch_capacity()
    x = torch.empty(16, device="cuda")
    with pytest.raises(_evoattn.EvoAttnError) as ei:
        _evoattn.bwd_static_scratch(big, x, x, x, x, x, x, x, x, x, x, x, x, x, 0.0,
                                    torch.cuda.current_stream().cuda_stream)
    assert ei.value.code == -9
