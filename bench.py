#!/usr/bin/env python
"""Benchmark of the scan path: fwd+bwd elements/s and fraction of the HBM roofline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward + one backward pass of the scan over the workload
(B, D, T) = (16, 2048, 8192), bf16 storage / fp32 accumulation, long-memory gates
a = 1 - 10^U(-4,-1), tokens and upstream gradient ~ N(0, 1), generated on the device from a
seed (synthetic data).  The six tensors of a step are at least three times the L2 at every N, so
no flush is needed between iterations.

For N > 1 launch under torchrun (one rank per GPU).  Rows are independent, so they are sharded
with no data-path collective.  The default is STRONG scaling -- the fixed 32768 rows of the
workload are split over the ranks (32768 / N rows each) -- which is the curve the workload
statement asks for; the weak figure (every rank a full 32768-row shard) rides along in the same
line as `weak_scaling`, and `--scaling weak` makes it the headline instead.

Rank 0 prints ONE JSON line.  `value` is device-timed whole-job throughput with inputs resident
in HBM; `e2e` is the same metric through the host-buffer entry of the C ABI (pinned host
inputs -> device -> pinned host outputs inside the timed region) with the copy-only time of the
same pipeline beside it; `roofline` describes the dominant kernel (backward); `cpu_baseline` is
the CPU port timed on this box's host cores; `time_split` is the long-sequence problem
(1, 4096, 262144) fp32 split along T over the N ranks, timed and checked against the oracle on a
row subset; `reference_cuda` is the reference's own CUDA operator timed on the same GPU (a stated
comparison, never the target).

`--impl reference` times the CPU implementation of the path (the pinned C port of the
reference loop, OpenMP over rows, all host threads) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

WORKLOAD = {"name": "scan fwd+bwd (B,D,T)=(16,2048,8192) bf16 storage / fp32 accumulate",
            "B": 16, "D": 2048, "T": 8192, "storage": "bf16"}
METRIC = "scan fwd+bwd elements/s"
UNIT = "elements/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
CPU_SAMPLE_ROWS = 4096
# DRAM traffic of the backward kernel per algorithmic byte, from an ncu capture of the same kernel
# on 4096 rows x T=8192 bf16 (traffic is proportional to rows): reads 201.35 MB against 201.33 MB
# algorithmic, writes algorithmic.
NCU_BWD_READ_RATIO = 201.35 / 201.33


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


# ------------------------------------------------------------------------- clocks sampler ---
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int, period_s: float = 0.005):
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                    "samples": 0}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:
            return local_index
    return local_index


# ------------------------------------------------------------------------- CPU baseline -----
def cpu_port_throughput(rows: int, T: int, repeats: int, warmup: int = 1):
    """fwd+bwd elements/s of the C port (OpenMP over rows) on `rows` x T of the workload."""
    from oracle import c_oracle as oc
    from tests.helpers import make_inputs

    # torchrun exports OMP_NUM_THREADS=1; the CPU baseline is entitled to every core it may use
    oc.set_num_threads(len(os.sched_getaffinity(0)))
    a, x, G = make_inputs(rows, T, 1003, "long", "bf16")
    times = []
    for i in range(warmup + repeats):
        t0 = time.perf_counter()
        h = oc.plain_forward(a, x)
        oc.plain_backward(a, h, G)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    return rows * T / min(times), rows * T / statistics.mean(times), oc.num_threads(), times


def torch_loop_throughput(rows: int, T: int):
    """The reference's own CPU form (T dispatch-bound torch steps + autograd) on a small sample."""
    import torch
    from oracle import torch_loop as tl
    from tests.helpers import make_inputs

    torch.set_num_threads(len(os.sched_getaffinity(0)))
    a, x, G = (torch.from_numpy(v).view(1, rows, T) for v in make_inputs(rows, T, 1003, "long", "bf16"))
    t0 = time.perf_counter()
    tl.plain_fwd_bwd(a, x, G)
    return rows * T / (time.perf_counter() - t0)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    T = WORKLOAD["T"]
    rows = CPU_SAMPLE_ROWS
    best, mean, threads, times = cpu_port_throughput(rows, T, repeats=max(1, args.steps),
                                                     warmup=max(1, args.warmup))
    sample = (f"{rows} of {WORKLOAD['B'] * WORKLOAD['D']} rows x T={T} (rows are independent; "
              f"fp32 arithmetic on bf16-rounded inputs), {len(times)} timed passes")
    line = {
        "impl": "reference", "metric": METRIC, "value": mean, "unit": UNIT, "n_gpus": args.gpus,
        "steps": len(times), "warmup": max(1, args.warmup),
        "ms_per_step": 1e3 * statistics.mean(times), "higher_is_better": True,
        "scaling": args.scaling or "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD["name"], "sample": sample},
        "cpu_baseline": {"value": mean, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample, "best": best, "host_cpus": os.cpu_count()},
        "e2e": {"value": mean, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------- GPU arm ----------
def make_device_inputs(rows, T, seed, device):
    import torch
    gen = torch.Generator(device=device).manual_seed(seed)
    u = torch.rand(rows, T, device=device, generator=gen)
    a = (1.0 - torch.pow(10.0, -4.0 + 3.0 * u)).to(torch.bfloat16)
    del u
    x = torch.randn(rows, T, device=device, generator=gen).to(torch.bfloat16)
    G = torch.randn(rows, T, device=device, generator=gen).to(torch.bfloat16)
    return a, x, G


def _cuda_events(n):
    import torch
    return [torch.cuda.Event(enable_timing=True) for _ in range(n)]


def time_rows_workload(rows, T, seed, device, steps, warmup, barrier, use_graph=True):
    """Device-timed fwd+bwd over `rows` x T bf16 on this rank.

    Returns (ms_per_step, fwd_ms, bwd_ms, tensors).  The headline loop holds nothing but the two
    launches per step between one pair of events; the per-kernel split comes from a second, short
    loop with an event after every launch (events between launches cost a few microseconds each,
    which matters at 40-60 us kernels)."""
    import torch

    from fm_b200 import fm_scan_backward_ex, fm_scan_forward

    a, x, G = make_device_inputs(rows, T, seed, device)
    D = WORKLOAD["D"]
    a3, x3, G3 = (t.view(-1, D, T) if rows % D == 0 else t.view(1, rows, T) for t in (a, x, G))
    h, ga, gx = torch.empty_like(a3), torch.empty_like(a3), torch.empty_like(a3)

    def step():
        fm_scan_forward(a3, x3, None, h)
        fm_scan_backward_ex(a3, G3, None, gx, h, ga, None, None)

    for _ in range(max(3, warmup)):
        step()
    barrier()
    # The two launches of a step are captured once into a CUDA graph and replayed: at 30-60 us per
    # kernel (8 GPUs) the launch path is worth a few per cent.  Nothing is allocated inside step().
    # If capture is not possible the same launches are issued one by one.
    launch, how = step, "eager launches"
    if use_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step()
                with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                    step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            for _ in range(3):
                graph.replay()
            launch, how = graph.replay, "one CUDA graph of the two launches, replayed per step"
        except Exception as e:  # keep measuring with plain launches
            torch.cuda.synchronize()
            how = "eager launches (graph capture failed: %s)" % type(e).__name__
    barrier()
    start, end = _cuda_events(2)
    barrier()
    start.record()
    for _ in range(steps):
        launch()
    end.record()
    barrier()
    ms_per_step = start.elapsed_time(end) / steps

    n_split = max(5, min(steps, 50))
    ev = [_cuda_events(3) for _ in range(n_split)]
    for k in range(n_split):
        ev[k][0].record()
        fm_scan_forward(a3, x3, None, h)
        ev[k][1].record()
        fm_scan_backward_ex(a3, G3, None, gx, h, ga, None, None)
        ev[k][2].record()
    torch.cuda.synchronize()
    fwd_ms = statistics.median(e[0].elapsed_time(e[1]) for e in ev)
    bwd_ms = statistics.median(e[1].elapsed_time(e[2]) for e in ev)
    return ms_per_step, fwd_ms, bwd_ms, (a3, x3, G3), how


def run_ours(args):
    import torch
    import torch.distributed as dist

    from fm_b200 import capi

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback of the product path)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    capi.lib()  # fail loudly if the CUDA library is missing

    B, D, T = WORKLOAD["B"], WORKLOAD["D"], WORKLOAD["T"]
    total_rows = args.rows if args.rows > 0 else B * D
    scaling = args.scaling or "strong"  # at N = 1 the two modes are the same run
    rows = total_rows // world if scaling == "strong" else total_rows
    global_rows = rows * world
    n_local = rows * T
    K = args.steps

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(values):
        if world == 1:
            return [float(v) for v in values]
        t = torch.tensor(values, device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        ms_per_step, fwd_ms, bwd_ms, tensors, launch_how = time_rows_workload(
            rows, T, 1003 + rank, device, K, args.warmup, barrier, use_graph=not args.no_graph)

    # end to end through host buffers
    if args.no_e2e:
        e2e = {"ms": float("nan"), "copy_only_ms": float("nan"), "h2d": 0, "d2h": 0, "steps": 0,
               "launches_per_step": 0, "path": "skipped (--no-e2e)"}
    else:
        e2e = run_e2e(args, *tensors, device, barrier)
    del tensors
    ms_per_step, fwd_ms, bwd_ms, e2e_ms, copy_ms = max_over_ranks(
        [ms_per_step, fwd_ms, bwd_ms, e2e["ms"], e2e["copy_only_ms"]])

    # the other scaling mode, as an extra figure of the same line (N > 1 only; identical at N = 1)
    other = None
    if world > 1 and not args.no_extras:
        o_rows = total_rows if scaling == "strong" else total_rows // world
        o_ms, _, _, o_t, _ = time_rows_workload(o_rows, T, 1003 + rank, device, max(5, min(K, 50)), 3, barrier,
                                                use_graph=not args.no_graph)
        del o_t
        (o_ms,) = max_over_ranks([o_ms])
        other = {"rows_per_gpu": o_rows, "ms_per_step": o_ms, "value": o_rows * world * T / (o_ms * 1e-3),
                 "unit": UNIT}
    torch.cuda.empty_cache()

    time_split = None
    if not args.no_extras and args.rows == 0:
        try:
            time_split = measure_time_split(args, world, rank, device, barrier, max_over_ranks)
        except Exception as e:  # the headline figures above stand on their own
            time_split = {"unavailable": "%s: %s" % (type(e).__name__, str(e)[:200])}
        torch.cuda.empty_cache()

    if rank == 0:
        s = 2  # bytes per stored element
        value = global_rows * T / (ms_per_step * 1e-3)
        peak, peak_kind = measured_peak()
        bwd_gbs = 5 * s * n_local / (bwd_ms * 1e-3) / 1e9
        fwd_gbs = 3 * s * n_local / (fwd_ms * 1e-3) / 1e9
        both_gbs = 8 * s * n_local / (ms_per_step * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD["name"], "rows_per_gpu": rows, "global_rows": global_rows, "T": T,
                       "storage": "bf16", "accumulate": "f32",
                       "gates": "a = 1 - 10^U(-4,-1) rounded to bf16; x, G ~ N(0,1)",
                       "l2": "inputs larger than L2 (six tensors of %d MiB per GPU touched per step), no flush" %
                             (n_local * s >> 20),
                       "sharding": ("the fixed %d rows split over the ranks" % total_rows if scaling == "strong"
                                    else "%d rows on every rank" % total_rows) + ", no collective"},
            "gpu_launches": 2 * K, "launch_path": launch_how,
            "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
            "fwd_elements_per_s": global_rows * T / (fwd_ms * 1e-3),
            "roofline": {"bound": "hbm", "kernel": "plain_backward_kernel", "achieved": bwd_gbs,
                         "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": bwd_gbs / peak,
                         "frac_of_nominal_8TBs": bwd_gbs / NOMINAL_HBM_GBS,
                         "traffic": int((3 * NCU_BWD_READ_RATIO + 2) * s * n_local),
                         "traffic_source": "ncu dram__bytes_read.sum+write.sum on a 4096-row case, scaled by rows",
                         "algorithmic_bytes_per_launch": 5 * s * n_local},
            "roofline_forward": {"kernel": "plain_forward_kernel", "achieved": fwd_gbs,
                                 "frac": fwd_gbs / peak, "frac_of_nominal_8TBs": fwd_gbs / NOMINAL_HBM_GBS,
                                 "algorithmic_bytes_per_launch": 3 * s * n_local},
            "roofline_fwd_bwd": {"achieved": both_gbs, "frac": both_gbs / peak,
                                 "frac_of_nominal_8TBs": both_gbs / NOMINAL_HBM_GBS,
                                 "note": "8*s*N per step over ms_per_step (launch gaps included)"},
            "clocks": clocks.summary(),
            "e2e": {"value": global_rows * T / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                    "ms_per_step": e2e_ms, "steps": e2e["steps"], "path": e2e["path"],
                    "copy_only_ms": copy_ms,
                    "frac_of_copy_only": (copy_ms / e2e_ms) if e2e_ms == e2e_ms and e2e_ms > 0 else None,
                    "copy_only": "the same pipeline with the kernels skipped: H2D and D2H of the same bytes "
                                 "overlapped on the same streams, max over ranks"},
        }
        if other is not None:
            line["weak_scaling" if scaling == "strong" else "strong_scaling"] = other
        if time_split is not None:
            line["time_split"] = time_split
        if world == 1 and not args.no_cpu_baseline:
            best, mean, threads, times = cpu_port_throughput(CPU_SAMPLE_ROWS, T, repeats=5)
            line["cpu_baseline"] = {
                "value": mean, "unit": UNIT, "cores": threads, "kind": "port",
                "sample": f"{CPU_SAMPLE_ROWS} of {total_rows} rows x T={T}, 5 timed fwd+bwd passes of "
                          "the C port (OpenMP over rows)",
                "best": best, "host_cpus": os.cpu_count(),
                "torch_loop_elements_per_s": torch_loop_throughput(64, T),
                "torch_loop_sample": f"64 rows x T={T}, one fwd+autograd-bwd pass of the time-step loop"}
        if world == 1 and not args.no_extras and args.rows == 0:
            line["reference_cuda"] = reference_cuda_figures(device, K)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------ long sequence, split along T
C4_ROWS, C4_T = 4096, 262144
C4_CHECK_ROWS = [0, 1, 2, 3, 1023, 1024, 2047, 2048, 2049, 3071, 3072, 4092, 4093, 4094, 4095, 777]


def measure_time_split(args, world, rank, device, barrier, max_over_ranks):
    """(B,D,T) = (1,4096,262144) fp32, gates sigmoid(N(0,1)+3): rank k owns time block k of every row;
    at N = 1 the plain operator scans the whole rows.  Timed (fwd+bwd, CUDA events, max over ranks)
    and checked on 16 rows over the FULL length against the C oracle run in double."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from fm_b200 import fm_scan
    from fm_b200.time_split import fm_scan_time_split

    B, D, T = 1, C4_ROWS, C4_T
    Tk = T // world
    gen = torch.Generator(device=device).manual_seed(1004 + rank)
    a = torch.sigmoid(torch.randn(B, D, Tk, device=device, generator=gen) + 3.0).requires_grad_(True)
    x = torch.randn(B, D, Tk, device=device, generator=gen).requires_grad_(True)
    G = torch.randn(B, D, Tk, device=device, generator=gen)

    exchange, transport = None, "none (one GPU, rows scanned whole)"
    if world > 1:
        transport = "NCCL all-gather of (P,S) fp32 carries, once per direction"
        if args.exchange in ("fused", "peer"):
            try:
                from fm_b200.peer_exchange import FusedTimeSplit, PeerCarryExchange
                # fused where a row's operands stay in L2 between its two passes (8 ranks: 128 KB rows),
                # three launches with peer stores where they cannot (2 and 4 ranks: 512 KB and 256 KB rows)
                if args.exchange == "fused" and FusedTimeSplit.pays(a):
                    exchange = FusedTimeSplit(B * D)
                    transport = ("one kernel per direction: carry pass, peer stores + bounded local polls, scan "
                                 "pass fused row by row (second pass re-reads the row from L2)")
                else:
                    exchange = PeerCarryExchange(B * D)
                    transport = "peer stores + flags in symmetric memory, fold on arrival"
            except Exception as e:  # symmetric memory unavailable: keep the collective
                transport += " (peer exchange unavailable: %s)" % type(e).__name__

    def step():
        h = fm_scan_time_split(a, x, exchange=exchange) if world > 1 else fm_scan(a, x)
        ga, gx = torch.autograd.grad(h, (a, x), G)
        return h, ga, gx

    steps = max(3, min(args.steps, 20))
    for _ in range(3):
        out = step()
    barrier()
    start, end = _cuda_events(2)
    barrier()
    start.record()
    for _ in range(steps):
        out = step()
    end.record()
    barrier()
    (ms,) = max_over_ranks([start.elapsed_time(end) / steps])
    if exchange is not None:
        exchange.check()

    # parity: the check rows of every block travel to rank 0 (full T), oracle in double there
    idx = torch.tensor(C4_CHECK_ROWS, device=device)
    mine = torch.stack([t.detach()[0].index_select(0, idx) for t in (a, x, G, *out)])   # (6, 16, Tk)
    del out
    if world > 1:
        allb = torch.empty((world,) + tuple(mine.shape), device=device, dtype=mine.dtype)
        dist.all_gather_into_tensor(allb, mine.contiguous())
        full = torch.cat([allb[k] for k in range(world)], dim=-1)
    else:
        full = mine
    result = None
    if rank == 0:
        from oracle import c_oracle as oc
        a_, x_, G_, h_, ga_, gx_ = (full[i].cpu().numpy() for i in range(6))
        f64 = np.float64
        h64 = oc.plain_forward(a_.astype(f64), x_.astype(f64), dtype=f64)
        ga64, gx64, _ = oc.plain_backward(a_.astype(f64), h64, G_.astype(f64), dtype=f64)
        h32 = oc.plain_forward(a_, x_)                      # the reference's own fp32 arithmetic
        ga32, gx32, _ = oc.plain_backward(a_, h32, G_)
        rtol, atol = 1e-5, 1e-6
        checks = {}
        worst = 0.0
        for name, got, ref32, ref64 in (("states", h_, h32, h64), ("grad_gates", ga_, ga32, ga64),
                                        ("grad_tokens", gx_, gx32, gx64)):
            scaled = atol * max(1.0, float(np.abs(ref64).max())) + rtol * np.abs(ref64)
            plain = atol + rtol * np.abs(ref64)
            err, err32 = np.abs(got - ref64), np.abs(ref32 - ref64)
            ratio = float((err / scaled).max())
            worst = max(worst, ratio)
            checks[name] = {"max_err_over_tol": ratio, "max_abs_ref": float(np.abs(ref64).max()),
                            "exceed_unscaled_kernel": int((err > plain).sum()),
                            "exceed_unscaled_reference_fp32": int((err32 > plain).sum()),
                            "elements": int(err.size)}
        n = B * D * T
        peak, kind = measured_peak()
        result = {
            "workload": "scan fwd+bwd (B,D,T)=(1,%d,%d) fp32, T split in %d blocks" % (D, T, world),
            "n_gpus": world, "ms_per_step": ms, "steps": steps, "value": n / (ms * 1e-3), "unit": UNIT,
            "transport": transport,
            "algorithmic_GBs_per_gpu": 8 * 4 * n / world / (ms * 1e-3) / 1e9, "peak": peak, "peak_kind": kind,
            "max_err_over_tol": worst,
            "tolerance": "rtol 1e-5, atol 1e-6 * max(1, max|ref|) against the oracle in double; "
                         "exceed_unscaled_* count elements beyond rtol 1e-5 / atol 1e-6 unscaled, for the kernel "
                         "and for the reference's own fp32 arithmetic (sequential loop)",
            "checked": "%d rows incl. first and last, full T=%d (%d elements per tensor)" % (
                len(C4_CHECK_ROWS), T, len(C4_CHECK_ROWS) * T),
            "checks": checks,
        }
    return result


# ------------------------------------------------------------------ the reference's own CUDA op
def load_reference_cuda():
    """Import the reference's fm/scan/fm_scan.py from baseline/_ref (baseline/make_ref.py put it there).

    The module compiles its kernel at import through torch's load_inline.  When baseline/_ref holds
    the extension already built from those same sources (make_ref.py --prebuild), load_inline is
    answered with that build instead of compiling for minutes; everything else -- the kernel, its
    flags, the autograd class, fm_scan() -- is the reference's own, unmodified."""
    import importlib.util

    import torch.utils.cpp_extension as ce

    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "fm" / "scan" / "fm_scan.py").exists():
        raise FileNotFoundError("baseline/_ref is absent (python baseline/make_ref.py --prebuild)")
    prebuilt = ref_root / "torch_extensions" / "fm_scan" / "fm_scan.so"
    real = ce.load_inline
    if prebuilt.exists():
        def load_prebuilt(name, *a, **k):
            spec = importlib.util.spec_from_file_location(name, str(prebuilt))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            return mod
        ce.load_inline = load_prebuilt
    else:
        os.environ.setdefault("TORCH_EXTENSIONS_DIR", str(ref_root / "torch_extensions"))
    try:
        sys.path.insert(0, str(ref_root))
        import fm.scan.fm_scan as ref
    finally:
        ce.load_inline = real
        sys.path.remove(str(ref_root))
    return ref, ("prebuilt extension" if prebuilt.exists() else "JIT build")


def reference_cuda_figures(device, steps):
    """fwd+bwd of the reference's CUDA operator through its public fm_scan() on this GPU: the
    headline workload through the M = D = 1 fold (32768 rows -> B = 32768, bf16) and its own demo
    shape (1, 32, 2048, 8192) bf16.  Any failure is reported as `unavailable`, never retried."""
    import torch
    try:
        ref, how = load_reference_cuda()
    except Exception as e:
        return {"unavailable": "%s: %s" % (type(e).__name__, str(e)[:200])}
    out = {"build": how, "api": "fm.scan.fm_scan.fm_scan + autograd (its two torch sums included)"}
    try:
        steps = max(3, min(steps, 20))

        def timed(g, x, G):
            g.requires_grad_(True)
            x.requires_grad_(True)

            def one():
                h = ref.fm_scan(g, x)
                return torch.autograd.grad(h, (g, x), G)

            for _ in range(3):
                one()
            torch.cuda.synchronize()
            ev = [_cuda_events(2) for _ in range(steps)]
            for e in ev:
                e[0].record()
                one()
                e[1].record()
            torch.cuda.synchronize()
            return statistics.median(e[0].elapsed_time(e[1]) for e in ev)

        T = WORKLOAD["T"]
        rows = WORKLOAD["B"] * WORKLOAD["D"]
        a, x, G = make_device_inputs(rows, T, 1003, device)
        ms = timed(a.view(rows, 1, T), x.view(rows, 1, T), G.view(rows, 1, 1, T))
        out["headline_via_fold"] = {"shape": "(B,M,D,L)=(%d,1,1,%d) bf16" % (rows, T), "ms_per_step": ms,
                                    "elements_per_s": rows * T / (ms * 1e-3)}
        del a, x, G
        torch.cuda.empty_cache()
        B, M, D, L = 1, 32, 2048, 8192
        gen = torch.Generator(device=device).manual_seed(1070)
        g = (0.9 + 0.1 * torch.rand(B, M, L, device=device, generator=gen)).to(torch.bfloat16)
        x = torch.randn(B, D, L, device=device, generator=gen).to(torch.bfloat16)
        G = torch.randn(B, M, D, L, device=device, generator=gen).to(torch.bfloat16)
        ms = timed(g, x, G)
        out["demo_shape"] = {"shape": "(B,M,D,L)=(1,32,2048,8192) bf16", "ms_per_step": ms,
                             "output_elements_per_s": B * M * D * L / (ms * 1e-3)}
    except Exception as e:
        out["unavailable"] = "%s: %s" % (type(e).__name__, str(e)[:200])
    return out


def run_time_split(args):
    """Secondary workload: configuration 4, (B,D,T) = (1,4096,262144) fp32, T split over the ranks.

    Strong scaling of one long-sequence problem: rank k owns time block k of every row and the
    carries cross NVLink once per direction (`fm_b200.time_split`).  At N = 1 it is the plain op.
    Prints its own JSON line; the headline metric of this repository is the default workload.
    """
    import torch
    import torch.distributed as dist

    from fm_b200 import fm_scan
    from fm_b200.time_split import fm_scan_time_split

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    B, D, T = 1, args.rows or 4096, args.seq_len or 262144
    Tk = T // world
    gen = torch.Generator(device=device).manual_seed(1004 + rank)
    a = torch.sigmoid(torch.randn(B, D, Tk, device=device, generator=gen) + 3.0).requires_grad_(True)
    x = torch.randn(B, D, Tk, device=device, generator=gen).requires_grad_(True)
    G = torch.randn(B, D, Tk, device=device, generator=gen)

    exchange = None
    if world > 1 and args.exchange in ("peer", "fused"):
        from fm_b200.peer_exchange import FusedTimeSplit, PeerCarryExchange
        exchange = FusedTimeSplit(B * D) if args.exchange == "fused" else PeerCarryExchange(B * D)

    def step():
        h = fm_scan_time_split(a, x, exchange=exchange) if world > 1 else fm_scan(a, x)
        return torch.autograd.grad(h, (a, x), G)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    K = args.steps
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        barrier()
        start.record()
        for _ in range(K):
            step()
        end.record()
        barrier()
    ms = start.elapsed_time(end) / K
    if world > 1:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if exchange is not None:
        exchange.check()
    if rank == 0:
        n = B * D * T
        peak, kind = measured_peak()
        passes = 8 if world == 1 else 12  # element passes: 3+5 unsplit, (2+3)+(2+5) split
        line = {"metric": "scan fwd+bwd elements/s (split along T)", "value": n / (ms * 1e-3), "unit": UNIT,
                "n_gpus": world, "steps": K, "warmup": max(3, args.warmup), "ms_per_step": ms,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic",
                "config": {"workload": "scan fwd+bwd (B,D,T)=(1,%d,%d) fp32, T split in %d blocks" % (D, T, world),
                           "gates": "a = sigmoid(N(0,1)+3); x, G ~ N(0,1)",
                           "exchange": (type(exchange).__name__ + ": peer stores + flags in symmetric memory"
                                        if exchange is not None else
                                        "NCCL all-gather of (P,S) fp32 carries, once per direction")},
                "gpu_launches": K * (2 if world == 1 else 6),
                "roofline_fwd_bwd": {"algorithmic_GBs_per_gpu": 8 * 4 * n / world / (ms * 1e-3) / 1e9,
                                     "moved_GBs_per_gpu": passes * 4 * n / world / (ms * 1e-3) / 1e9,
                                     "peak": peak, "peak_kind": kind},
                "clocks": clocks.summary()}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_time_split_block(args):
    """Profiler case: ONE rank's block of the long sequence split along T -- (rows, 32768) fp32, the
    per-GPU share of (1,4096,262144) over 8 ranks -- through the fused kernels with a world of 1 (no
    peers, nothing to wait for), beside the three-launch path on the same data.  One GPU."""
    import ctypes

    import torch

    from fm_b200 import capi
    from fm_b200.ops import CudaScanOps as ops
    from fm_b200.peer_exchange import _bind_fused

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    L = _bind_fused()
    R, T = args.rows or 4096, 32768
    gen = torch.Generator(device=dev).manual_seed(1004)
    a = torch.sigmoid(torch.randn(R, T, device=dev, generator=gen) + 3.0)
    x = torch.randn(R, T, device=dev, generator=gen)
    G = torch.randn(R, T, device=dev, generator=gen)
    h, ga, gx = torch.empty_like(a), torch.empty_like(a), torch.empty_like(a)
    hin = torch.empty(R, device=dev)
    buf = torch.zeros(int(L.fms_tsplit_exchange_bytes(R, 1)), dtype=torch.uint8, device=dev)
    ptrs = (ctypes.c_void_p * 1)(buf.data_ptr())
    st = torch.cuda.current_stream().cuda_stream
    count = [0]

    def fused():
        count[0] += 1
        rc = L.fms_tsplit_forward(a.data_ptr(), x.data_ptr(), None, h.data_ptr(), hin.data_ptr(), R, T, capi.FMS_F32,
                                  ptrs, 1, 0, count[0], 1.0, st)
        rc = rc or L.fms_tsplit_backward(a.data_ptr(), h.data_ptr(), G.data_ptr(), hin.data_ptr(), ga.data_ptr(),
                                         gx.data_ptr(), None, R, T, capi.FMS_F32, ptrs, 1, 0, count[0], 1.0, st)
        assert rc == 0, capi.status_string(rc)

    def three_launch():
        P, S = ops.reduce(a, x)
        hh = ops.forward(a, x, torch.zeros_like(S))
        ops.reduce_reverse(a, G)
        ops.backward(a, hh, G, None, None)

    def timed(fn, steps):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        s0, s1 = _cuda_events(2)
        s0.record()
        for _ in range(steps):
            fn()
        s1.record()
        torch.cuda.synchronize()
        return s0.elapsed_time(s1) / steps

    K = args.steps
    fused_ms = timed(fused, K)
    three_ms = timed(three_launch, K)
    n = R * T
    peak, kind = measured_peak()
    line = {"metric": "scan fwd+bwd elements/s (one block of the split along T)", "value": n / (fused_ms * 1e-3),
            "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": max(3, args.warmup), "ms_per_step": fused_ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "one time block (rows,T)=(%d,%d) fp32 of the split along T, world of 1" % (R, T)},
            "gpu_launches": 2 * K,
            "three_launch_ms": three_ms,
            "roofline_fwd_bwd": {"algorithmic_GBs": 8 * 4 * n / (fused_ms * 1e-3) / 1e9,
                                 "three_launch_algorithmic_GBs": 8 * 4 * n / (three_ms * 1e-3) / 1e9,
                                 "peak": peak, "peak_kind": kind}}
    print(json.dumps(line), flush=True)


def run_fm_mode(args):
    """Secondary workload: the reference's own operator and demo shape, gates (1,32,8192),
    tokens (1,D,8192) -> states (1,32,D,8192), bf16 (fm_test.ipynb:29-33 uses D = 2048).

    One GPU.  Prints its own JSON line: forward writes the states once (the gate and token rows are
    re-read from L2); backward reads states and their gradient once and reduces over D and M
    inside the kernel.  `--rows` sets D (a small D is the profiler case).
    """
    import torch

    from fm_b200 import fm_scan_backward_fm, fm_scan_forward

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    B, M, D, L = 1, 32, args.rows or 2048, 8192
    gen = torch.Generator(device=dev).manual_seed(1070)
    g = (0.9 + 0.1 * torch.rand(B, M, L, device=dev, generator=gen)).to(torch.bfloat16)
    x = torch.randn(B, D, L, device=dev, generator=gen).to(torch.bfloat16)
    G = torch.randn(B, M, D, L, device=dev, generator=gen).to(torch.bfloat16)
    h = torch.empty(B, M, D, L, device=dev, dtype=torch.bfloat16)
    dg, dx = torch.empty_like(g), torch.empty_like(x)

    def fwd():
        fm_scan_forward(g, x, None, h)

    def bwd():
        fm_scan_backward_fm(g, G, dx, h, x, dg, None, None)

    for _ in range(max(3, args.warmup)):
        fwd()
        bwd()
    torch.cuda.synchronize()
    K = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
    with ClockSampler(physical_gpu_index(0)) as clocks:
        for k in range(K):
            ev[k][0].record()
            fwd()
            ev[k][1].record()
            bwd()
            ev[k][2].record()
        torch.cuda.synchronize()
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    n = B * M * D * L
    peak, kind = measured_peak()

    # the layer around the scan (inference): with the states materialised, and read out directly
    from fm_b200 import fm_memory
    del G, h
    alpha = torch.softmax(torch.randn(B, L, M, device=dev, generator=gen), dim=-1).to(torch.bfloat16)
    upd = torch.sigmoid(torch.randn(B, L, 1, device=dev, generator=gen)).to(torch.bfloat16)
    outs = torch.sigmoid(torch.randn(B, L, 1, device=dev, generator=gen)).to(torch.bfloat16)
    inp = torch.randn(B, L, D, device=dev, generator=gen).to(torch.bfloat16)

    def layer_ms(need_states, fused):
        with torch.no_grad():
            for _ in range(3):
                fm_memory(alpha, upd, outs, inp, need_states=need_states, fused=fused)
            torch.cuda.synchronize()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for _ in range(max(1, K // 2)):
                fm_memory(alpha, upd, outs, inp, need_states=need_states, fused=fused)
            s1.record()
            torch.cuda.synchronize()
        return s0.elapsed_time(s1) / max(1, K // 2)

    layer_states_ms = layer_ms(True, False)
    layer_fused_states_ms = layer_ms(True, True)
    layer_fused_ms = layer_ms(False, True)

    def train_ms(fused):
        args = [t.clone().requires_grad_(True) for t in (alpha, upd, outs, inp)]
        Wt = torch.randn(B, L, D, device=dev, generator=gen).to(torch.bfloat16)

        def one():
            out, _ = fm_memory(*args, fused=fused)
            torch.autograd.grad((out * Wt).sum(), args)

        for _ in range(2):
            one()
        torch.cuda.synchronize()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(1, K // 4)
        s0.record()
        for _ in range(reps):
            one()
        s1.record()
        torch.cuda.synchronize()
        return s0.elapsed_time(s1) / reps

    train_fused_ms = train_ms(True)
    torch.cuda.empty_cache()
    train_composed_ms = train_ms(False)
    line = {"metric": "FM-mode scan fwd+bwd output elements/s", "value": n / ((fwd_ms + bwd_ms) * 1e-3),
            "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": max(3, args.warmup),
            "ms_per_step": fwd_ms + bwd_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": "FM mode (B,M,D,L)=(%d,%d,%d,%d) bf16 storage / fp32 accumulate" % (B, M, D, L)},
            "gpu_launches": K * 4,  # forward; backward + two fp32->bf16 casts of the reduced gradients
            "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
            "layer_forward_ms": {"states_materialised_torch_epilogue": layer_states_ms,
                                 "fused_with_normalised_states": layer_fused_states_ms,
                                 "read_out_without_states": layer_fused_ms},
            "layer_train_step_ms": {"fused_op": train_fused_ms,
                                    "fm_scan_plus_torch_norm_and_einsum": train_composed_ms},
            "roofline_forward": {"algorithmic_bytes_per_launch": 2 * n + 2 * (M + D) * B * L,
                                 "achieved": (2 * n + 2 * (M + D) * B * L) / (fwd_ms * 1e-3) / 1e9,
                                 "peak": peak, "peak_kind": kind, "unit": "GB/s"},
            "roofline": {"bound": "hbm", "kernel": "fm_backward_ring_kernel",
                         "algorithmic_bytes_per_launch": 4 * n + 4 * (M + D) * B * L,
                         "achieved": (4 * n + 4 * (M + D) * B * L) / (bwd_ms * 1e-3) / 1e9,
                         "peak": peak, "peak_kind": kind, "unit": "GB/s"},
            "clocks": clocks.summary()}
    line["roofline"]["frac"] = line["roofline"]["achieved"] / peak
    line["roofline_forward"]["frac"] = line["roofline_forward"]["achieved"] / peak
    print(json.dumps(line), flush=True)


def run_channel_last(args):
    """Secondary workload: the plain scan on channel-last tensors (B,T,D) = (16,8192,2048) bf16
    (`--rows` sets B; a small B is the profiler case).  One GPU; prints its own JSON line."""
    import torch

    from fm_b200.fm_scan import _load_ext

    ext = _load_ext()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    B, T, D = args.rows or 16, 8192, 2048
    gen = torch.Generator(device=dev).manual_seed(1080)
    a = (1.0 - torch.pow(10.0, -4.0 + 3.0 * torch.rand(B, T, D, device=dev, generator=gen))).to(torch.bfloat16)
    x = torch.randn(B, T, D, device=dev, generator=gen).to(torch.bfloat16)
    G = torch.randn(B, T, D, device=dev, generator=gen).to(torch.bfloat16)
    h, ga, gx = torch.empty_like(a), torch.empty_like(a), torch.empty_like(a)
    for _ in range(max(3, args.warmup)):
        ext.fm_scan_btd_forward(a, x, None, h)
        ext.fm_scan_btd_backward(a, G, gx, h, ga, None, None)
    torch.cuda.synchronize()
    K = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
    with ClockSampler(physical_gpu_index(0)) as clocks:
        for k in range(K):
            ev[k][0].record()
            ext.fm_scan_btd_forward(a, x, None, h)
            ev[k][1].record()
            ext.fm_scan_btd_backward(a, G, gx, h, ga, None, None)
            ev[k][2].record()
        torch.cuda.synchronize()
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    n = B * T * D
    peak, kind = measured_peak()
    line = {"metric": "channel-last scan fwd+bwd elements/s", "value": n / ((fwd_ms + bwd_ms) * 1e-3), "unit": UNIT,
            "n_gpus": 1, "steps": K, "warmup": max(3, args.warmup), "ms_per_step": fwd_ms + bwd_ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "plain scan on (B,T,D)=(%d,%d,%d) bf16 storage / fp32 accumulate" % (B, T, D)},
            "gpu_launches": K * 6, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
            "roofline_fwd_bwd": {"algorithmic_GBs": 16 * n / ((fwd_ms + bwd_ms) * 1e-3) / 1e9,
                                 "moved_GBs": 24 * n / ((fwd_ms + bwd_ms) * 1e-3) / 1e9, "peak": peak,
                                 "peak_kind": kind},
            "clocks": clocks.summary()}
    print(json.dumps(line), flush=True)


def run_e2e(args, a3, x3, G3, device, barrier):
    """Same step with pinned HOST inputs and outputs through the host-buffer entry of the C ABI.

    Per step, inside the timed region: the three inputs go host -> device, forward and backward
    run, the three results come device -> host (all of them: the host caller ends up with what
    the reference's CPU scan would have left in host memory).  `copy_only_ms` is the same
    pipeline with the kernels skipped -- the ceiling the copies alone set on this box.
    """
    import torch

    from fm_b200.host_pipeline import HostPipeline

    steps = max(1, min(args.e2e_steps, args.steps))
    host_in = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in (a3, x3, G3)]
    for hb, t in zip(host_in, (a3, x3, G3)):
        hb.copy_(t)
    host_out = [torch.empty(a3.shape, dtype=a3.dtype, pin_memory=True) for _ in range(3)]
    rows = a3.numel() // a3.shape[-1]
    pipe = HostPipeline(max(1, rows // 32), a3.shape[-1], a3.dtype, device)
    torch.cuda.synchronize()

    def timed(fn):
        fn()
        barrier()
        start, end = _cuda_events(2)
        start.record()
        for _ in range(steps):
            fn()
        end.record()
        barrier()
        return start.elapsed_time(end) / steps

    ms = timed(lambda: pipe.forward_backward(*host_in, *host_out))
    copy_ms = timed(lambda: pipe.copy_only(*host_in, *host_out))
    pipe.close()
    nbytes = a3.numel() * a3.element_size()
    blocks = 32 if rows >= 2048 else (8 if rows >= 8 else 1)
    return {"ms": ms, "copy_only_ms": copy_ms, "h2d": 3 * nbytes, "d2h": 3 * nbytes,
            "steps": steps, "launches_per_step": 2 * blocks,
            "path": "fms_plain_forward_backward_host: pinned host -> H2D | kernels | D2H overlapped in "
                    "%d row blocks -> pinned host" % blocks}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--scaling", choices=["weak", "strong"], default=None,
                    help="N > 1: strong (default) splits the fixed 32768 rows over the ranks; weak gives "
                         "every rank all 32768")
    ap.add_argument("--workload", choices=["c3", "c4", "c4block", "fm", "btd"], default="c3",
                    help="c3: the headline row-sharded workload; c4: the long sequence split along T; "
                         "c4block: one rank's block of c4 through the fused kernels (profiler case); "
                         "fm: the reference's (B,M,L)x(B,D,L)->(B,M,D,L) operator at its demo shape; "
                         "btd: the plain scan on channel-last (B,T,D) tensors")
    ap.add_argument("--exchange", choices=["nccl", "peer", "fused"], default="fused",
                    help="carry transport of the long sequence split along T")
    ap.add_argument("--no-graph", action="store_true", help="issue the timed launches one by one (no CUDA graph)")
    ap.add_argument("--no-extras", action="store_true",
                    help="headline only: skip time_split, the other scaling mode and reference_cuda")
    ap.add_argument("--seq-len", type=int, default=0,
                    help="--workload c4: total sequence length instead of 262144 (tuning aid: 65536 on 2 GPUs "
                         "gives each rank the block it has at 8 GPUs)")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling aid)")
    ap.add_argument("--rows", type=int, default=0,
                    help="rows per GPU instead of B*D (small case for profiler captures only)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "c4":
        run_time_split(args)
    elif args.workload == "c4block":
        run_time_split_block(args)
    elif args.workload == "fm":
        run_fm_mode(args)
    elif args.workload == "btd":
        run_channel_last(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
