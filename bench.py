"""EvoAttention fwd+bwd benchmark (one JSON line on stdout, printed by rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload cfg2_msa_row] [--scaling weak|strong]

A step is one forward + backward of the workload through
TKEvoAttention.apply on seeded synthetic inputs.  N=1 runs benchmark config 2
(B=1, S=512, N=384, H=8, D=32, bf16).  N>1 (under torchrun, one rank per GPU)
shards the independent S axis over ranks with the pair bias replicated and an
NCCL all-reduce of dBias in backward: "weak" keeps S rows per GPU fixed,
"strong" splits the workload's S over the ranks.

value      whole-job TFLOP/s, algorithmic FLOPs 14*B*S*H*N^2*D, inputs resident in HBM
e2e        same metric with host (pinned) buffers through HostStreamedEvoAttention.run:
           H2D of q,k,v,dO,mask,bias and D2H of O,dQ,dK,dV,dBias inside the timed
           region, overlapped with the kernels chunk by chunk of S rows
roofline   backward dQ/dK/dV kernel: its 10*B*S*H*N^2*D FLOPs / its CUDA-event time,
           against the measured sustained bf16 GEMM peak
cpu_baseline / --impl reference   the eager PyTorch restatement on the host cores
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "megakernel-exploration_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import evo_workloads as wl  # noqa: E402

# DRAM bytes per S row of one evo_bwd_kernel launch, from the ncu capture summarised under profiles/
# (160.77 MB read + 53.59 MB written at 128 rows of cfg2).
NCU_DRAM_BYTES_PER_ROW = {"cfg2_msa_row": (160.77e6 + 53.59e6) / 128}

METRIC = "EvoAttention fwd+bwd TFLOP/s"
UNIT = "TFLOP/s"


def _peaks():
    """Measured dense bf16 peaks of this pool's B200s: `burst` for a kernel timed by itself,
    `sustained` for one inside a seconds-long loop under the power cap."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"burst": float(p["bf16_tflops"]), "sustained": float(p["bf16_tflops_sustained"]),
                "source": "measured cuBLAS bf16, burst (MEASURED_PEAKS.json): the timed loop is a fraction of a "
                          "second at full clock"}
    return {"burst": 1590.0, "sustained": 1400.0, "source": "fallback figures of an earlier measurement on this pool"}


def _strong_cfg4(world, rank, dev, pg, TKEvoAttention, barrier, steps):
    """Config 4 (B=1, S=1024, N=768, H=8, D=32) on one GPU (rank 0 alone, the others wait) and split over
    all ranks along S, in the same process: {"ms_1gpu", "ms_Ngpu", "speedup"}."""
    import torch.distributed as dist
    name = "cfg4_large_msa"
    B, S, N, H, D = wl.WORKLOADS[name][:5]
    if S % world:
        return None
    bf = torch.bfloat16

    def make(lo, hi):
        q, k, v, mask, bias, d_o = wl.make_workload(name, lo, hi)
        t = [x.to(dev, bf) for x in (q, k, v, d_o)] + [mask.to(dev, bf), bias.to(dev, bf)]
        for x in (t[0], t[1], t[2], t[5]):
            x.requires_grad_(True)
        return t

    def run(t, group, n):
        Q, K, V, DO, M, PB = t

        def one():
            for x in (Q, K, V, PB):
                x.grad = None
            o = TKEvoAttention.apply(Q, K, V, M, PB) if group is None else TKEvoAttention.apply(Q, K, V, M, PB, group)
            o.backward(DO)

        for _ in range(3):
            one()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            one()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    ms1 = torch.zeros(1, device=dev)
    if rank == 0:
        t = make(0, S)
        ms1[0] = run(t, None, steps)
        del t
        torch.cuda.empty_cache()
    barrier()
    dist.broadcast(ms1, 0)
    rows = S // world
    t = make(rank * rows, (rank + 1) * rows)
    barrier()
    msn = torch.tensor([run(t, pg, steps)], device=dev)
    dist.all_reduce(msn, op=dist.ReduceOp.MAX)
    del t
    torch.cuda.empty_cache()
    return {"workload": name, "S_total": S, "S_per_gpu": rows, "steps": steps, "ms_1gpu": ms1.item(),
            "ms_Ngpu": msn.item(), "speedup": ms1.item() / msn.item(),
            "note": "device-resident fwd+bwd per step; N-GPU time is the max over ranks"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the
    timed region runs (reading only)."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self._nv is not None:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr is not None:
            self._thr.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def _cpu_fwd_bwd(name: str, rows: int, repeats: int):
    """Eager oracle on the host cores over `rows` S rows of the workload; returns
    (TFLOP/s, seconds per pass, threads)."""
    from oracle import evo_ref
    B, S, N, H, D = wl.WORKLOADS[name][:5]
    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v, mask, bias, d_o = wl.make_workload(name, 0, rows)
    evo_ref.evo_attention_fwd_bwd_ref(q[:, :4], k[:, :4], v[:, :4], mask[:, :4], bias, d_o[:, :4])  # warm-up
    ts = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        evo_ref.evo_attention_fwd_bwd_ref(q, k, v, mask, bias, d_o, s_chunk=32)
        ts.append(time.perf_counter() - t0)
    sec = min(ts)
    return wl.flops_fwd_bwd(B, rows, N, H, D) / sec / 1e12, sec, torch.get_num_threads()


def run_reference(args, rank: int, world: int):
    """The reference's path on the host CPU: its documented math restated in eager
    PyTorch (the reference kernel itself needs ThunderKittens and an sm_90a GPU).
    Each step is one forward + backward over a bounded sample of the workload's S rows
    (rows are independent problems, so TFLOP/s on a row subset is the workload's rate)."""
    if rank != 0:
        return
    name = args.workload
    B, S, N, H, D = wl.WORKLOADS[name][:5]
    if args.rows:
        S = args.rows
    S_total = S * world if args.scaling == "weak" else S
    S_per_gpu = S if args.scaling == "weak" else S // world
    torch.set_num_threads(os.cpu_count() or 1)
    from oracle import evo_ref
    rows = max(1, min(S, args.cpu_rows))
    q, k, v, mask, bias, d_o = wl.make_workload(name, 0, rows)
    # one untimed pass (thread pool, allocator), then size the sample: the whole run stays within a few
    # minutes, and never drops below 16 rows (smaller samples time the framework, not the math)
    evo_ref.evo_attention_fwd_bwd_ref(q, k, v, mask, bias, d_o, s_chunk=32)
    t0 = time.perf_counter()
    evo_ref.evo_attention_fwd_bwd_ref(q, k, v, mask, bias, d_o, s_chunk=32)
    per_pass = time.perf_counter() - t0
    budget = 150.0 / max(args.steps + args.warmup, 1)
    if per_pass > budget and rows > 16:
        rows = max(16, int(rows * budget / per_pass))
        q, k, v, mask, bias, d_o = wl.make_workload(name, 0, rows)
    vals = []
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        evo_ref.evo_attention_fwd_bwd_ref(q, k, v, mask, bias, d_o, s_chunk=32)
        dt = time.perf_counter() - t0
        if i >= args.warmup:
            vals.append(dt)
    sec = statistics.median(vals)
    tf = wl.flops_fwd_bwd(B, rows, N, H, D) / sec / 1e12
    sample = f"{rows} of {S_total} S rows of {name} per step (rows are independent), fp32 eager, S-chunked by 32"
    out = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": _config(name, B, S_total, S_per_gpu, N, H, D, world),
        "cpu_baseline": {"value": tf, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": tf, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(out), flush=True)


def _config(name, B, S_total, S_per_gpu, N, H, D, world):
    """The `config` object both arms print (same keys, same values)."""
    return {"workload": name, "B": B, "S_total": S_total, "S_per_gpu": S_per_gpu, "N": N, "H": H, "D": D,
            "parallelism": f"S-sharded x{world}, pair bias replicated, NCCL all-reduce of dBias",
            "l2": "each step streams > 126 MB (inputs larger than L2)"}


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch.distributed as dist
    import _evoattn
    from tk_evo_attention_layer import TKEvoAttention

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    pg = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        # the only collective of the path: the d_pair_bias all-reduce, on a group whose kernels are small
        # enough to run beside the dQ/dK/dV kernel
        from tk_evo_attention_layer import new_dbias_group
        pg = new_dbias_group()

    name = args.workload
    B, S, N, H, D = wl.WORKLOADS[name][:5]
    if args.rows:
        S = args.rows
    if args.scaling == "weak":
        rows, S_total = S, S * world
        lo = rank * S
    else:
        assert S % world == 0, "strong scaling needs S divisible by the number of GPUs"
        rows, S_total = S // world, S
        lo = rank * rows
    q, k, v, mask, bias, d_o = wl.make_workload(name, lo, lo + rows, S_override=S_total)
    bf = torch.bfloat16
    # host side: pinned bf16 / fp32 buffers (what a host-buffer caller would hold)
    h_in = [t.to(bf).pin_memory() for t in (q, k, v, d_o)] + [mask.to(bf).pin_memory(), bias.to(bf).pin_memory()]
    d_in = [t.to(dev, non_blocking=True) for t in h_in]
    Q, K, V, DO, M, PB = d_in
    for t in (Q, K, V, PB):
        t.requires_grad_(True)
    h_out = [torch.empty((B, rows, N, H, D), dtype=bf).pin_memory() for _ in range(4)]
    h_out.append(torch.empty((B, 1, H, N, N), dtype=torch.float32).pin_memory())
    h2d = sum(t.numel() * t.element_size() for t in h_in)
    d2h = sum(t.numel() * t.element_size() for t in h_out)

    def step():
        for t in (Q, K, V, PB):
            t.grad = None
        if pg is None:
            O = TKEvoAttention.apply(Q, K, V, M, PB)
        else:
            O = TKEvoAttention.apply(Q, K, V, M, PB, pg)
        O.backward(DO)
        return O

    # host-buffer callers: the package's streamed entry point (H2D, kernels and D2H of S-row chunks overlap)
    from tk_evo_attention_layer import HostStreamedEvoAttention
    eng = HostStreamedEvoAttention(dev, chunk_rows=args.e2e_chunk_rows, process_group=pg)
    e2e_out = dict(zip(("o", "dq", "dk", "dv", "dbias"), h_out))

    def step_e2e():
        hq, hk, hv, hdo, hm, hb = h_in
        eng.run(hq, hk, hv, hm, hb, hdo, e2e_out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """Total milliseconds of `steps` calls (one event pair around the whole loop, max over ranks) and the
        per-step milliseconds (an event at every step boundary, this rank)."""
        barrier()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        ev[0].record()
        for i in range(steps):
            fn()
            ev[i + 1].record()
        barrier()
        ms = torch.tensor([ev[0].elapsed_time(ev[steps])], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        per = [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)]
        return ms.item(), per

    headline = step
    if args.graph:
        # the step captured once in a CUDA graph (its NCCL all-reduce included) and replayed: for
        # workloads whose per-GPU share is launch-bound.  The leaves are first used on the capture's
        # side stream: autograd accumulates a leaf's gradient on the stream of its first use.
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(args.warmup, 3)):
                step()
        torch.cuda.current_stream().wait_stream(side)
        barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            step()
        barrier()
        headline = graph.replay
    for _ in range(max(args.warmup, 3)):
        headline()
    _evoattn.device_status()
    # headline: nothing but the steps inside the timed region
    with ClockSampler(local_rank) as cs:
        ms_total, per_step = timed(headline, args.steps)
    _evoattn.device_status()
    # a second, short loop with the library's per-kernel events, for the roofline figures only
    prof_steps = max(3, min(args.steps, 20))
    _evoattn.profile_enable(True)
    timed(step, prof_steps)
    _evoattn.profile_enable(False)
    fwd_ms, fwd_n = _evoattn.profile_read(0)
    bwd_ms, bwd_n = _evoattn.profile_read(1)
    db_ms, db_n = _evoattn.profile_read(2)
    _evoattn.device_status()

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        step_e2e()
    ms_e2e, _ = timed(step_e2e, e2e_steps)
    _evoattn.device_status()

    # ---- N > 1: the overlapped, phased backward against a plain all-reduce of the partial dBias ----
    multi_gpu_check = None
    if world > 1:
        PB32 = PB.detach().float().requires_grad_(True)            # fp32 leaf: d_pair_bias comes back in fp32

        def grads(group):
            for t in (Q, K, V, PB32):
                t.grad = None
            o = TKEvoAttention.apply(Q, K, V, M, PB32) if group is None else TKEvoAttention.apply(Q, K, V, M, PB32, group)
            o.backward(DO)
            return [t.grad.detach().clone() for t in (Q, K, V, PB32)]

        got = grads(pg)                                             # phased backward, overlapped all-reduce
        part = grads(None)                                          # this rank's rows alone, no group
        dist.all_reduce(part[3], op=dist.ReduceOp.SUM)              # default group, blocking
        db_err = (got[3].float() - part[3].float()).abs().max()
        dq_err = (got[0].float() - part[0].float()).abs().max()
        same = torch.tensor([float(torch.equal(got[1], part[1]) and torch.equal(got[2], part[2]))], device=dev)
        stats = torch.stack([db_err, dq_err, 1.0 - same[0]])
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        db_e, dq_e, diff = (float(x) for x in stats.tolist())
        multi_gpu_check = {"dbias_max_abs": db_e, "dq_max_abs": dq_e, "dk_dv_bit_identical": diff == 0.0,
                           "ok": bool(db_e <= 1e-3 and dq_e <= 2.0 ** -6 and diff == 0.0),
                           "what": "d_pair_bias of the phased backward with the overlapped all-reduce against "
                                   "the same rows without a group followed by a blocking all-reduce (fp32, "
                                   "<= 1e-3); dK/dV bit-identical, dQ within one bf16 step; max over ranks"}
        for t in (Q, K, V, PB):
            t.grad = None

    # ---- N > 1: strong scaling of config 4 (S = 1024 split over the ranks) in the same run ----
    strong = None
    if world > 1 and not args.no_strong_cfg4 and name == "cfg2_msa_row" and args.scaling == "weak" and not args.rows:
        strong = _strong_cfg4(world, rank, dev, pg, TKEvoAttention, barrier, max(3, min(args.steps, 20)))

    flops_step = wl.flops_fwd_bwd(B, S_total, N, H, D)          # whole job, all ranks
    ms_step = ms_total / args.steps
    value = flops_step / (ms_step * 1e-3) / 1e12
    e2e_value = flops_step / (ms_e2e / e2e_steps * 1e-3) / 1e12

    peaks = _peaks()
    bwd_flops_launch = 10.0 * B * rows * H * N * N * D           # this rank's launch
    bwd_avg_ms = bwd_ms / max(bwd_n, 1)
    achieved = bwd_flops_launch / (bwd_avg_ms * 1e-3) / 1e12 if bwd_n else None
    roofline = {
        "kernel": "evo_bwd_kernel", "bound": "tensor", "achieved": achieved, "peak": peaks["burst"], "unit": "TFLOP/s",
        "frac": (achieved / peaks["burst"]) if achieved else None,
        "frac_of_sustained_peak": (achieved / peaks["sustained"]) if achieved else None,
        "traffic": (NCU_DRAM_BYTES_PER_ROW[name] * rows) if name in NCU_DRAM_BYTES_PER_ROW else None,
        "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch at 128 S rows "
                          "(summary under profiles/), scaled by rows: every S row is touched once",
        "peak_source": peaks["source"],
        "avg_launch_ms": bwd_avg_ms, "launches_timed": bwd_n,
        "fwd_kernel": {"avg_launch_ms": fwd_ms / max(fwd_n, 1), "launches_timed": fwd_n,
                       "achieved": (4.0 * B * rows * H * N * N * D) / (fwd_ms / max(fwd_n, 1) * 1e-3) / 1e12 if fwd_n else None},
        "dbias_kernel": {"avg_launch_ms": db_ms / max(db_n, 1), "launches_timed": db_n,
                         "achieved": (4.0 * B * rows * H * N * N * D) / (db_ms / max(db_n, 1) * 1e-3) / 1e12 if db_n else None},
    }

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        S = wl.WORKLOADS[name][1]
        tf, sec, cores = _cpu_fwd_bwd(name, min(S, args.cpu_rows), 2)
        cpu = {"value": tf, "unit": UNIT, "cores": cores, "kind": "port",
               "sample": f"{min(S, args.cpu_rows)} of {S} S rows of {name}, fp32 eager PyTorch, best of 2 "
                         f"({sec:.2f} s per pass)"}

    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": _config(name, B, S_total, rows, N, H, D, world),
            "pct_of_2250_dense_bf16": 100.0 * value / (2250.0 * world),
            "ms_per_step_median": statistics.median(per_step), "ms_per_step_min": min(per_step),
            "clocks": cs.summary(),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "bytes_are": "per rank (the value is the whole job)",
                    "ms_per_step": ms_e2e / e2e_steps, "steps": e2e_steps},
            "gpu_launches": 5 * args.steps,   # forward; backward: prep, dBias, dQ/dK/dV, dQ conversion
            "graph_replay": bool(args.graph),
            "roofline": roofline,
        }
        if multi_gpu_check is not None:
            out["multi_gpu_check"] = multi_gpu_check
        if strong is not None:
            out["strong_cfg4"] = strong
        if cpu is not None:
            out["cpu_baseline"] = cpu
        print(json.dumps(out), flush=True)
    if args.graph:
        # a graph that holds collective kernels must be gone before its communicator is
        headline = None
        del graph
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_reference_sweep(args):
    """The reference's own benchmark shapes (evo_h100/benchmark.py:38-46 with the batch of its README
    table, evo_h100/README.md:779-812): B=4, H=16, D=64, N_SEQ=1, N_CTX swept, forward / backward /
    full through the Python operator, wrapper included, `.grad = None` before every backward, an L2
    flush before every timed call, median of the per-call CUDA-event times.  One JSON line."""
    from tk_evo_attention_layer import TKEvoAttention
    import _evoattn
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, H, D, S = 4, 16, 64, 1
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev).manual_seed(1234)

    def bench(fn, iters=60, warm=15):
        for _ in range(warm):
            fn()
        ts = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)

    rows = []
    for N in (128, 256, 384, 512, 640, 768, 1024):
        mk = lambda *shape: torch.randn(shape, device=dev, generator=g).to(torch.bfloat16)
        q, k, v = (mk(B, S, N, H, D) for _ in range(3))
        bias = mk(B, 1, H, N, N)
        # additive mask: 0 valid / -1e9 padded, residue 0 valid (the reference benchmark passes a bool
        # tensor that its layer turns into +0/+1; the contract of the operator is the additive mask)
        keep = torch.rand((B, S, 1, 1, N), device=dev, generator=g) < 0.5
        keep[..., 0] = True
        mask = torch.where(keep, 0.0, -1e9).to(torch.bfloat16)
        d_o = mk(B, S, N, H, D)
        with torch.no_grad():
            ms_f = bench(lambda: TKEvoAttention.apply(q, k, v, mask, bias))
        leaves = [t.clone().requires_grad_(True) for t in (q, k, v, bias)]
        o = TKEvoAttention.apply(leaves[0], leaves[1], leaves[2], mask, leaves[3])

        def bwd_only():
            for t in leaves:
                t.grad = None
            o.backward(d_o, retain_graph=True)

        def full():
            for t in leaves:
                t.grad = None
            TKEvoAttention.apply(leaves[0], leaves[1], leaves[2], mask, leaves[3]).backward(d_o)

        ms_b, ms_a = bench(bwd_only), bench(full)
        # the same full step captured once in a CUDA graph and replayed: what the kernels take without
        # the Python wrapper and the launch latency (the reference's numbers have no such column)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            # leaves of their own, first used on this stream: autograd accumulates a leaf's gradient
            # on the stream of its first use, which must not be the default stream during capture
            gl = [t.detach().clone().requires_grad_(True) for t in leaves]

            def full_g():
                for t in gl:
                    t.grad = None
                TKEvoAttention.apply(gl[0], gl[1], gl[2], mask, gl[3]).backward(d_o)

            for _ in range(3):
                full_g()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            full_g()
        ms_g = bench(graph.replay)
        del graph, gl
        unit = B * S * H * N * N * D / 1e12
        rows.append({"N_CTX": N, "fwd_ms": ms_f, "bwd_ms": ms_b, "full_ms": ms_a, "full_graph_ms": ms_g,
                     "fwd_tflops": 4 * unit / (ms_f * 1e-3), "bwd_tflops": 10 * unit / (ms_b * 1e-3),
                     "full_tflops": 14 * unit / (ms_a * 1e-3), "full_graph_tflops": 14 * unit / (ms_g * 1e-3)})
    _evoattn.device_status()
    print(json.dumps({"sweep": "reference benchmark shapes", "B": B, "H": H, "D": D, "N_SEQ": S, "dtype": "bf16",
                      "timing": "median of 60 per-call CUDA-event times, L2 flushed before each, Python wrapper included "
                                "(full_graph_*: the full step replayed from a CUDA graph)",
                      "rows": rows}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sweep-reference-shapes", action="store_true",
                    help="time the reference benchmark's own shapes (B=4,H=16,D=64,N_SEQ=1) instead of the bench line")
    ap.add_argument("--e2e-chunk-rows", type=int, default=64, help="S rows per chunk of the host-streamed e2e path")
    ap.add_argument("--workload", default="cfg2_msa_row", choices=sorted(wl.WORKLOADS))
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--cpu-rows", type=int, default=64, help="S rows per CPU pass (bounded sample)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--graph", action="store_true",
                    help="capture the step in a CUDA graph and time its replay (launch-bound workloads)")
    ap.add_argument("--no-strong-cfg4", action="store_true",
                    help="N > 1: skip the strong-scaling record of config 4 that the default line carries")
    ap.add_argument("--rows", type=int, default=0,
                    help="override the workload's S (small captures under a profiler)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.sweep_reference_shapes:
        run_reference_sweep(args)
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
