#!/usr/bin/env python
"""Benchmark of the hot path: row-parallel bf16 GEMM fused with reduce-scatter.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload ...]

One process per GPU (under torchrun for N > 1). A step is one pass of the operator over one set
of synthetic inputs: tokens M=8192, K=28672 split K/N across the N ranks, N=8192 outputs
(the Llama-70B MLP down-projection shape), output reduce-scattered along M. Total work is fixed
as N grows (strong scaling); at N=1 the operator is the plain GEMM.

Prints ONE JSON line (rank 0). `value` is whole-job TFLOP/s with inputs resident in HBM, timed
with CUDA events, max over ranks. `e2e` is the same metric through the Python entry point
(tk_kernel.gemm_rs) with pinned HOST operands copied in and the result copied out every step.
`cpu_baseline` / `--impl reference` time the reference's torch CPU path
(torch.matmul on the host, distributed-kernels/bf16_gemm/example.py:105) on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "distributed-hipkittens_b200"))

M_TOK, K_FULL, N_OUT = 8192, 28672, 8192
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return d, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi. It is started well before the timed
    region (its start-up is slow on multi-GPU hosts and would disturb the first steps); only
    samples whose arrival time falls inside [t0, t1] are reported."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append((time.time(), ln.strip()))

    def count_in(self, t0, t1):
        return sum(1 for (t, _) in self.lines if t0 <= t <= t1)

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for (t, ln) in self.lines:
            if not (t0 <= t <= t1):
                continue
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_reference_tflops(budget_s: float = 15.0):
    """The reference's torch CPU path on a bounded sample of the workload: the first `rows` token
    rows against the full [N, K] weight, torch.matmul of the bf16-rounded operands in fp32 with all
    host threads. Returns (TFLOP/s, threads, description, seconds)."""
    import torch
    from oracle import dk_oracle as orc
    threads = torch.get_num_threads()
    g = torch.Generator().manual_seed(0)
    Bt = (torch.randn(N_OUT, K_FULL, generator=g) / math.sqrt(K_FULL)).to(torch.bfloat16)
    rows = 128
    A = torch.randn(rows, K_FULL, generator=g).to(torch.bfloat16)
    orc.gemm_ref(A, Bt)                                # warm-up (thread pool, page faults)
    t0 = time.perf_counter()
    orc.gemm_ref(A, Bt)
    dt = time.perf_counter() - t0
    # grow the sample towards the budget, at most the whole workload
    rows = int(max(128, min(M_TOK, rows * budget_s / max(dt, 1e-3))))
    rows = rows // 128 * 128
    A = torch.randn(rows, K_FULL, generator=g).to(torch.bfloat16)
    t0 = time.perf_counter()
    orc.gemm_ref(A, Bt)
    dt = time.perf_counter() - t0
    tf = 2.0 * rows * N_OUT * K_FULL / dt / 1e12
    return tf, threads, f"first {rows} of {M_TOK} token rows x full N={N_OUT}, K={K_FULL} (oracle gemm_ref, torch CPU fp32)", dt


def run_reference(args, rank):
    """--impl reference: the reference's CPU implementation of the path, rank 0 only."""
    if rank != 0:
        return
    import torch
    vals = []
    desc, threads = "", 1
    for i in range(args.warmup + args.steps):
        tf, threads, desc, dt = cpu_reference_tflops(budget_s=4.0)
        if i >= args.warmup:
            vals.append((tf, dt))
    tf = sum(v for v, _ in vals) / len(vals)
    ms = sum(d for _, d in vals) / len(vals) * 1e3
    line = {
        "impl": "reference", "metric": "gemm_rs_tflops", "value": tf, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"gemm_rs M={M_TOK} N={N_OUT} K={K_FULL} (bounded CPU sample per step)"},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--shape", default=None, help="M,N,K override of the workload (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 0)

    global M_TOK, N_OUT, K_FULL
    if args.shape:
        M_TOK, N_OUT, K_FULL = (int(v) for v in args.shape.split(","))
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU fallback)"
    assert world == args.gpus or world == 1, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import iris_py
    import tk_kernel

    P = world
    assert K_FULL % P == 0 and M_TOK % (P * 128) == 0
    Kloc = K_FULL // P
    Mloc = M_TOK // P
    ws_mb = (2 * M_TOK * N_OUT * 2) // (1 << 20) + 64 if P > 1 else 0
    iris = iris_py.Iris(heap_size_mb=ws_mb + Mloc * N_OUT * 2 * 2 // (1 << 20) + 64, verbose=False)
    assert iris.rank() == rank and iris.world_size() == world
    view = iris.get_device_view()

    # synthetic operands, seeded per rank; several sets so that consecutive steps never hit L2
    shard_bytes = (M_TOK + N_OUT) * Kloc * 2
    nsets = max(2, math.ceil(256e6 / shard_bytes))
    g = torch.Generator(device="cuda").manual_seed(1000 + rank)
    sets = []
    for _ in range(nsets):
        A = torch.randn(M_TOK, Kloc, device="cuda", generator=g).to(torch.bfloat16)
        Bt = (torch.randn(N_OUT, Kloc, device="cuda", generator=g) / math.sqrt(K_FULL)).to(torch.bfloat16)
        sets.append((A, Bt))
    out_t = iris.empty([Mloc, N_OUT], "bfloat16")
    out = torch.as_tensor(out_t, device="cuda").view(torch.bfloat16)

    def step(i):
        A, Bt = sets[i % nsets]
        tk_kernel.gemm_rs(A, Bt, out, view)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        t_wait = time.time() + 8.0
        while not sampler.lines and time.time() < t_wait:   # let nvidia-smi finish starting up
            time.sleep(0.05)
    barrier()
    for i in range(args.warmup):
        step(i)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_clock0 = time.time()
    ev0.record()
    for i in range(args.steps):
        step(i)
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    clocks_extended = False
    if sampler and sampler.count_in(t_clock0, time.time()) < 4:
        # the timed region was shorter than a few sampling periods: keep the same load running,
        # untimed, until the sampler has seen it
        clocks_extended = True
        t_end = time.time() + 1.0
    else:
        t_end = 0.0
    extra = 0
    while True:
        go = torch.tensor([1.0 if time.time() < t_end else 0.0], device="cuda")
        if world > 1:
            dist.broadcast(go, 0)
        if go.item() == 0.0:
            break
        for i in range(10):
            step(i)
        extra += 10
        torch.cuda.synchronize()
    barrier()
    clocks = sampler.stop(t_clock0, time.time()) if sampler else None
    if clocks is not None:
        clocks["extended_by_untimed_steps"] = extra if clocks_extended else 0
    status = tk_kernel.device_status()
    assert status[0] == 0, f"device-side wait timed out: {status}"
    t = torch.tensor([ms_total], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = t.item() / args.steps
    flop_total = 2.0 * M_TOK * N_OUT * K_FULL
    value = flop_total / (ms_step * 1e-3) / 1e12

    e2e_value = e2e_ms = None
    h2d = d2h = 0
    if not args.no_e2e:
        # ---- end to end through the Python entry point with host operands
        hA = torch.empty(M_TOK, Kloc, dtype=torch.bfloat16).pin_memory()
        hB = torch.empty(N_OUT, Kloc, dtype=torch.bfloat16).pin_memory()
        hA.copy_(sets[0][0])
        hB.copy_(sets[0][1])
        hO = torch.empty(Mloc, N_OUT, dtype=torch.bfloat16).pin_memory()
        dA, dB = torch.empty_like(sets[0][0]), torch.empty_like(sets[0][1])

        def e2e_step():
            dA.copy_(hA, non_blocking=True)
            dB.copy_(hB, non_blocking=True)
            tk_kernel.gemm_rs(dA, dB, out, view)
            hO.copy_(out, non_blocking=True)

        e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.e2e_steps):
            e2e_step()
        e1.record()
        barrier()
        te = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_ms = te.item() / args.e2e_steps
        e2e_value = flop_total / (e2e_ms * 1e-3) / 1e12
        h2d = (hA.numel() + hB.numel()) * 2
        d2h = hO.numel() * 2

    if rank == 0:
        peaks, peak_src = load_peaks()
        timed_s = ms_step * args.steps * 1e-3
        sustained = timed_s >= 1.0
        peak = peaks.get("bf16_tflops_sustained" if sustained else "bf16_tflops")
        achieved = (flop_total / P) / (ms_step * 1e-3) / 1e12     # per GPU, per launch
        traffic = None
        prof = ROOT / "profiles" / "traffic.json"
        if prof.exists():
            try:
                traffic = json.loads(prof.read_text()).get(f"gemm_rs_p{P}")
            except Exception:
                traffic = None
        line = {
            "metric": "gemm_rs_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": P,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": f"gemm_rs M={M_TOK} N={N_OUT} K={K_FULL} K-sharded over {P} GPU(s), "
                                   f"out rows reduce-scattered (Llama-70B MLP down-proj shape)",
                       "l2": f"{nsets} operand sets of {shard_bytes / 1e6:.0f} MB rotated: "
                             f"{(nsets - 1) * shard_bytes / 1e6:.0f} MB of other operands pass between two "
                             f"uses of a set (L2 is 126 MB)",
                       "per_gpu_tflops": value / P},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak if peak else None, "traffic": traffic,
                         "peak_source": f"{peak_src} ({'sustained' if sustained else 'burst'} cuBLAS bf16)"},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": args.e2e_steps},
            "gpu_launches": args.steps,
            "clocks": clocks,
        }
        if P == 1 and not args.no_cpu_baseline:
            tf, threads, desc, dt = cpu_reference_tflops()
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                    "sample": desc, "seconds": dt}
        print(json.dumps(line), flush=True)
    barrier()
    del out, out_t, view, iris
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
