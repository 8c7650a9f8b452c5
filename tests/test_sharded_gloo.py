"""S-sharded data parallelism on CPU ranks (gloo, world size 2).

The rows of S are independent problems and the pair bias is replicated, so each
rank runs the operator on its own rows and backward all-reduces dBias over the
group.  This test drives the real TKEvoAttention wiring (argument handling,
gradient count, process-group all-reduce) with the two C-ABI calls replaced by
the CPU oracle -- a test double, since the kernels themselves need a GPU -- and
checks that the sharded result equals the unsharded one.
"""
import contextlib
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _install_cpu_doubles():
    for p in (ROOT, os.path.join(ROOT, "megakernel-exploration_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import _evoattn
    import tk_evo_attention_layer as L
    from oracle import evo_ref

    def fake_fwd(dims, q, k, v, bias, mask, o, o_resid, lse, scale, stream):
        B, S, N, H = dims.B, dims.S, dims.N, dims.H
        b5, m5 = bias.float().reshape(B, 1, H, N, N), mask.float().reshape(B, S, 1, 1, N)
        o.copy_(evo_ref.evo_attention_ref(q.float(), k.float(), v.float(), m5, b5, scale))
        lse.copy_(evo_ref.evo_lse_ref(q.float(), k.float(), m5, b5, scale))

    calls = []

    def fake_bwd_phased(dims, strides, q, k, v, bias, mask, o, o_resid, lse, d_o, dq, dk, dv, dbias, ws, scale,
                        phases, reserved_sms, stream):
        # phase 1 (prep + dBias) and phase 2 (dQ/dK/dV) as the layer issues them around the all-reduce
        assert strides is None
        calls.append((phases, reserved_sms))
        B, S, N, H = dims.B, dims.S, dims.N, dims.H
        b5, m5 = bias.float().reshape(B, 1, H, N, N), mask.float().reshape(B, S, 1, 1, N)
        with torch.enable_grad():      # the oracle differentiates; autograd is off inside backward()
            r = evo_ref.evo_attention_fwd_bwd_ref(q.float(), k.float(), v.float(), m5, b5, d_o.float(), scale)
        if phases & _evoattn.BWD_PHASE_DBIAS:
            dbias.copy_(r["dbias"].reshape(B, H, N, N))
        if phases & _evoattn.BWD_PHASE_DQKV:
            dq.copy_(r["dq"]); dk.copy_(r["dk"]); dv.copy_(r["dv"])

    _evoattn.fwd, _evoattn.bwd_phased = fake_fwd, fake_bwd_phased
    L._bwd_calls = calls
    _evoattn.bwd_workspace_bytes = lambda dims: 256
    L._check_device = lambda t: None
    L._device_ctx = lambda t: contextlib.nullcontext()
    L._stream = lambda: 0
    return L, evo_ref


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    L, evo_ref = _install_cpu_doubles()
    B, S, N, H, D = 1, 6, 24, 2, 32
    rows = S // world
    lo = rank * rows
    q, k, v, mask, bias, d_o = evo_ref.make_inputs(B, S, N, H, D, seed=9, mask_kind="bernoulli0.9",
                                                   s_lo=lo, s_hi=lo + rows)
    Q, K, V = (t.to(torch.bfloat16).requires_grad_(True) for t in (q, k, v))
    PB = bias.clone().requires_grad_(True)
    O = L.EvoAttention(process_group=L.new_dbias_group())(Q, K, V, mask, PB)
    O.backward(d_o.to(torch.bfloat16))
    # with a process group the backward is issued in two phases around the all-reduce, and the second
    # phase leaves SMs to the collective
    assert [c[0] for c in L._bwd_calls] == [1, 2] and L._bwd_calls[1][1] == L.ALLREDUCE_RESERVED_SMS   # SMs left to the collective
    torch.save({"o": O.detach().float(), "dq": Q.grad.float(), "dk": K.grad.float(), "dv": V.grad.float(),
                "dbias": PB.grad.float()}, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_s_sharded_equals_unsharded(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    L, evo_ref = _install_cpu_doubles()
    B, S, N, H, D = 1, 6, 24, 2, 32
    q, k, v, mask, bias, d_o = evo_ref.make_inputs(B, S, N, H, D, seed=9, mask_kind="bernoulli0.9")
    bf = lambda t: t.to(torch.bfloat16).float()
    ref = evo_ref.evo_attention_fwd_bwd_ref(bf(q), bf(k), bf(v), bf(mask), bf(bias), bf(d_o))
    for n in ("o", "dq", "dk", "dv"):
        got = torch.cat([p[n] for p in parts], dim=1)
        assert evo_ref.max_abs_err(ref[n], got) < 2e-2, n       # bf16 outputs
    # every rank holds the full dBias after the all-reduce, and it matches the unsharded sum
    assert torch.equal(parts[0]["dbias"], parts[1]["dbias"])
    assert evo_ref.max_abs_err(ref["dbias"], parts[0]["dbias"]) < 1e-4


def test_five_argument_call_returns_five_grads():
    L, evo_ref = _install_cpu_doubles()
    q, k, v, mask, bias, d_o = evo_ref.make_inputs(1, 2, 16, 2, 16, seed=1)     # D=16 is padded to 32
    Q, K, V = (t.to(torch.bfloat16).requires_grad_(True) for t in (q, k, v))
    PB = bias.clone().requires_grad_(True)
    O = L.TKEvoAttention.apply(Q, K, V, mask, PB)
    assert O.shape == (1, 2, 16, 2, 16) and O.dtype == torch.bfloat16
    O.backward(d_o.to(torch.bfloat16))
    assert Q.grad.shape == Q.shape and PB.grad.shape == PB.shape and PB.grad.dtype == torch.float32
    bf = lambda t: t.to(torch.bfloat16).float()
    ref = evo_ref.evo_attention_fwd_bwd_ref(bf(q), bf(k), bf(v), bf(mask), bf(bias), bf(d_o))
    assert evo_ref.max_abs_err(ref["dq"], Q.grad.float()) < 2e-2


def _worker_missing_rank(rank, world, port, out_dir):
    """Rank 1 runs the forward and then never joins the backward's all-reduce (a rank that died or fell
    behind between steps).  Rank 0 must get an error from the collective within the group's time limit,
    not wait for ever."""
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    L, evo_ref = _install_cpu_doubles()
    B, S, N, H, D = 1, 4, 16, 2, 32
    rows = S // world
    q, k, v, mask, bias, d_o = evo_ref.make_inputs(B, S, N, H, D, seed=5, s_lo=rank * rows, s_hi=(rank + 1) * rows)
    Q, K, V = (t.to(torch.bfloat16).requires_grad_(True) for t in (q, k, v))
    PB = bias.clone().requires_grad_(True)
    O = L.EvoAttention(process_group=L.new_dbias_group(timeout=datetime.timedelta(seconds=4)))(Q, K, V, mask, PB)
    if rank == 0:
        t0 = time.time()
        try:
            O.backward(d_o.to(torch.bfloat16))
            verdict = "no error"
        except Exception as e:                      # the collective's time limit, surfaced by work.wait()
            verdict = f"raised {type(e).__name__} after {time.time() - t0:.1f}s"
        with open(os.path.join(out_dir, "rank0.txt"), "w") as f:
            f.write(verdict)
    else:
        deadline = time.time() + 30                 # absent from the all-reduce until rank 0 has given up
        while not os.path.exists(os.path.join(out_dir, "rank0.txt")) and time.time() < deadline:
            time.sleep(0.2)
    # no barrier, no orderly shutdown of a group with a failed collective
    os._exit(0)


def test_missing_rank_ends_the_all_reduce_with_an_error(tmp_path):
    world = 2
    mp.spawn(_worker_missing_rank, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    verdict = (tmp_path / "rank0.txt").read_text()
    assert verdict.startswith("raised"), verdict
    seconds = float(verdict.split("after ")[1].rstrip("s"))
    assert seconds < 20, verdict
