#!/usr/bin/env python
"""Benchmark of the hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload gemm_rs|allreduce|moe_mixtral|moe_dsv3]

One process per GPU (under torchrun for N > 1). The default workload, the one the headline metric
is quoted on, is the row-parallel bf16 GEMM fused with reduce-scatter: tokens M=8192, K=28672 split
K/N across the N ranks, N=8192 outputs (the Llama-70B MLP down-projection shape), output
reduce-scattered along M. Total work is fixed as N grows (strong scaling); at N=1 the operator is
the plain GEMM. The other workloads measure the remaining operators of the path (TP all-reduce of
1 MiB / 128 MiB; Mixtral- and DeepSeek-V3-shaped fp8 MoE layers, expert-parallel when N > 1); the
default run appends them to the same JSON line as `secondary`.

Prints ONE JSON line (rank 0). `value` is whole-job throughput with inputs resident in HBM, timed
with CUDA events, max over ranks. `e2e` is the same metric through the Python entry points with
pinned HOST operands copied in and the result copied out every step. `cpu_baseline` /
`--impl reference` time the reference's torch CPU path (torch.matmul on the host,
distributed-kernels/bf16_gemm/example.py:105) on a bounded sample.
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
NVLINK_GBS = 770.0   # measured peer copy per direction over NVLink 5 / NVSwitch (nominal 900)


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return json.loads(p.read_text()), "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def load_traffic(key):
    prof = ROOT / "profiles" / "traffic.json"
    if prof.exists():
        try:
            return json.loads(prof.read_text()).get(key)
        except Exception:
            return None
    return None


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
    """The reference's torch CPU path on a bounded sample of the GEMM workload: the first `rows`
    token rows against the full [N, K] weight, torch.matmul of the bf16-rounded operands in fp32
    with all host threads. Returns (TFLOP/s, threads, description, seconds)."""
    import torch
    from oracle import dk_oracle as orc
    # all the host threads this process may use: torchrun exports OMP_NUM_THREADS=1 to every rank,
    # which would time a one-thread baseline when the reference arm runs under it
    try:
        avail = len(os.sched_getaffinity(0))
    except AttributeError:
        avail = os.cpu_count() or 1
    if torch.get_num_threads() < avail:
        torch.set_num_threads(avail)
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
    return tf, threads, (f"first {rows} of {M_TOK} token rows x full N={N_OUT}, K={K_FULL} "
                         f"(oracle gemm_ref, torch CPU fp32)"), dt


def gemm_rs_workload_name(P):
    return (f"gemm_rs M={M_TOK} N={N_OUT} K={K_FULL} K-sharded over {P} GPU(s), "
            f"out rows reduce-scattered (Llama-70B MLP down-proj shape)")


def run_reference(args, rank, out):
    """--impl reference: the reference's CPU implementation of the path, rank 0 only."""
    if rank != 0:
        return
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
        # the same workload string as the GPU arm prints for this N; what a step sampled is in cpu_baseline
        "config": {"workload": gemm_rs_workload_name(args.gpus)},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    out.write(json.dumps(line) + "\n")
    out.flush()


# ------------------------------------------------------------------------------------ workloads
class GemmRs:
    """Row-parallel GEMM + reduce-scatter (the headline workload)."""
    metric, unit, dtype, scaling = "gemm_rs_tflops", "TFLOP/s", "bf16", "strong"
    launches_per_step = 1

    @staticmethod
    def heap_mb(P):
        ws_mb = (2 * M_TOK * ((N_OUT + 255) // 256 * 256) * 2) // (1 << 20) + 64 if P > 1 else 0
        return ws_mb + (M_TOK // P) * N_OUT * 2 * 2 // (1 << 20) + 64

    def __init__(self, ctx):
        import torch
        self.ctx = ctx
        P, rank = ctx.world, ctx.rank
        assert K_FULL % P == 0 and M_TOK % (P * 128) == 0
        self.Kloc, self.Mloc = K_FULL // P, M_TOK // P
        ctx.make_heap(self.heap_mb(P))
        self.shard_bytes = (M_TOK + N_OUT) * self.Kloc * 2
        self.nsets = max(2, math.ceil(256e6 / self.shard_bytes))
        g = torch.Generator(device="cuda").manual_seed(1000 + rank)
        self.sets = []
        for _ in range(self.nsets):
            A = torch.randn(M_TOK, self.Kloc, device="cuda", generator=g).to(torch.bfloat16)
            Bt = (torch.randn(N_OUT, self.Kloc, device="cuda", generator=g) / math.sqrt(K_FULL)).to(torch.bfloat16)
            self.sets.append((A, Bt))
        self.out_t = ctx.iris.empty([self.Mloc, N_OUT], "bfloat16")
        self.out = torch.as_tensor(self.out_t, device="cuda").view(torch.bfloat16)
        self.work = 2.0 * M_TOK * N_OUT * K_FULL          # FLOP per step, whole job
        self.scale = 1e12

    def step(self, i):
        A, Bt = self.sets[i % self.nsets]
        self.ctx.tk.gemm_rs(A, Bt, self.out, self.ctx.view)

    def check(self):
        """Relative Frobenius error of the first 64 rows this rank owns against a NCCL sum of the
        ranks' fp32 partial products (a checker outside the timed region, not part of the path)."""
        import torch
        ctx = self.ctx
        A, Bt = self.sets[0]
        self.ctx.tk.gemm_rs(A, Bt, self.out, ctx.view)
        torch.cuda.synchronize()
        err = 0.0
        for r in range(ctx.world):
            rows = slice(r * self.Mloc, r * self.Mloc + 64)
            p = A[rows].float() @ Bt.float().T
            if ctx.world > 1:
                ctx.dist.all_reduce(p)
            if r == ctx.rank:
                err = ((self.out[:64].float() - p).norm() / p.norm()).item()
        return ctx.max_over_ranks(err)

    def e2e_setup(self):
        import torch
        A, Bt = self.sets[0]
        self.hA = torch.empty(M_TOK, self.Kloc, dtype=torch.bfloat16).pin_memory()
        self.hB = torch.empty(N_OUT, self.Kloc, dtype=torch.bfloat16).pin_memory()
        self.hA.copy_(A)
        self.hB.copy_(Bt)
        self.hO = torch.empty(self.Mloc, N_OUT, dtype=torch.bfloat16).pin_memory()
        self.dA, self.dB = torch.empty_like(A), torch.empty_like(Bt)
        return (self.hA.numel() + self.hB.numel()) * 2, self.hO.numel() * 2

    E2E_CHUNKS = 8

    def e2e_step(self):
        import torch
        if self.ctx.world > 1:
            self.dA.copy_(self.hA, non_blocking=True)
            self.dB.copy_(self.hB, non_blocking=True)
            self.ctx.tk.gemm_rs(self.dA, self.dB, self.out, self.ctx.view)
            self.hO.copy_(self.out, non_blocking=True)
            return
        # One GPU: the step is bound by the host link, so the calls are pipelined the way a user
        # with host-resident operands would: Bt goes in first, then A in row chunks on a copy
        # stream; each chunk's GEMM starts when its rows have landed, and its rows of the result go
        # back on a third stream while the next chunk is still coming in.
        if not hasattr(self, "s_in"):
            self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
            n = self.E2E_CHUNKS
            self.ev_in = [torch.cuda.Event() for _ in range(n)]
            self.ev_mm = [torch.cuda.Event() for _ in range(n)]
        cur = torch.cuda.current_stream()
        n = self.E2E_CHUNKS
        rows = M_TOK // n
        self.s_in.wait_stream(cur)        # the previous step's GEMMs are done with dA / dB
        self.s_out.wait_stream(cur)
        with torch.cuda.stream(self.s_in):
            self.dB.copy_(self.hB, non_blocking=True)
            for c in range(n):
                sl = slice(c * rows, (c + 1) * rows)
                self.dA[sl].copy_(self.hA[sl], non_blocking=True)
                self.ev_in[c].record(self.s_in)
        for c in range(n):
            sl = slice(c * rows, (c + 1) * rows)
            cur.wait_event(self.ev_in[c])
            self.ctx.tk.gemm_rs(self.dA[sl], self.dB, self.out[sl], self.ctx.view)
            self.ev_mm[c].record(cur)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_mm[c])
                self.hO[sl].copy_(self.out[sl], non_blocking=True)
        cur.wait_stream(self.s_out)       # the step ends when the last rows are back on the host

    def config(self, value):
        P = self.ctx.world
        return {"workload": gemm_rs_workload_name(P),
                "l2": f"{self.nsets} operand sets of {self.shard_bytes / 1e6:.0f} MB rotated: "
                      f"{(self.nsets - 1) * self.shard_bytes / 1e6:.0f} MB of other operands pass between two "
                      f"uses of a set (L2 is 126 MB)",
                "per_gpu_tflops": value / P}

    def roofline(self, ms_step, sustained, peaks, peak_src):
        P = self.ctx.world
        peak = peaks.get("bf16_tflops_sustained" if sustained else "bf16_tflops")
        achieved = (self.work / P) / (ms_step * 1e-3) / 1e12
        r = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
             "frac": achieved / peak if peak else None, "traffic": load_traffic(f"gemm_rs_p{P}"),
             "peak_source": f"{peak_src} ({'sustained' if sustained else 'burst'} cuBLAS bf16)"}
        if P > 1:
            egress = 2.0 * M_TOK * N_OUT * (P - 1) / P          # bf16 partials leaving this GPU
            r["nvlink"] = {"egress_bytes_per_step": egress,
                           "achieved_gbs": egress / (ms_step * 1e-3) / 1e9, "peak_gbs": NVLINK_GBS,
                           "floor_ms": egress / (NVLINK_GBS * 1e9) * 1e3}
        return r


class AgGemm:
    """Column-parallel GEMM fused with the all-gather of its activations: the Llama-70B MLP
    up-projection, tokens M=8192 row-sharded over the ranks, K=8192, N=28672 split N/P per rank."""
    metric, unit, dtype, scaling = "ag_gemm_tflops", "TFLOP/s", "bf16", "strong"
    launches_per_step = 1
    M, K, N = 8192, 8192, 28672

    @classmethod
    def heap_mb(cls, P):
        return (2 * cls.M * cls.K * 2) // (1 << 20) + 64 if P > 1 else 64

    def __init__(self, ctx):
        import torch
        self.ctx = ctx
        P, rank = ctx.world, ctx.rank
        ctx.make_heap(self.heap_mb(P))
        self.Nloc, self.shard = self.N // P, self.M // P
        g = torch.Generator(device="cuda").manual_seed(2000 + rank)
        set_bytes = (self.shard + self.Nloc) * self.K * 2
        self.nsets = max(2, math.ceil(256e6 / set_bytes))
        self.sets = []
        for _ in range(self.nsets):
            A = torch.randn(self.shard, self.K, device="cuda", generator=g).to(torch.bfloat16)
            Bt = (torch.randn(self.Nloc, self.K, device="cuda", generator=g) / math.sqrt(self.K)).to(torch.bfloat16)
            self.sets.append((A, Bt))
        self.out = torch.empty(self.M, self.Nloc, dtype=torch.bfloat16, device="cuda")
        self.work = 2.0 * self.M * self.N * self.K
        self.scale = 1e12

    def step(self, i):
        A, Bt = self.sets[i % self.nsets]
        self.ctx.tk.ag_gemm(A, Bt, self.out, self.ctx.view)

    def check(self):
        """64 rows of every source shard against torch on a NCCL all-gather of the shards."""
        import torch
        ctx = self.ctx
        A, Bt = self.sets[0]
        ctx.tk.ag_gemm(A, Bt, self.out, ctx.view)
        torch.cuda.synchronize()
        parts = [torch.empty(64, self.K, dtype=torch.bfloat16, device="cuda") for _ in range(ctx.world)]
        if ctx.world > 1:
            ctx.dist.all_gather(parts, A[:64].contiguous())
        else:
            parts = [A[:64]]
        err = 0.0
        for r, p in enumerate(parts):
            ref = p.float() @ Bt.float().T
            got = self.out[r * self.shard:r * self.shard + 64].float()
            err = max(err, ((got - ref).norm() / ref.norm()).item())
        return ctx.max_over_ranks(err)

    def e2e_setup(self):
        return None

    def config(self, value):
        P = self.ctx.world
        return {"workload": f"ag_gemm M={self.M} K={self.K} N={self.N}: activations row-sharded over {P} GPU(s), "
                            f"weight columns split N/{P} (Llama-70B MLP up-proj shape), all-gather fused into the GEMM",
                "l2": f"{self.nsets} operand sets rotated", "per_gpu_tflops": value / P}

    def roofline(self, ms_step, sustained, peaks, peak_src):
        P = self.ctx.world
        peak = peaks.get("bf16_tflops_sustained" if sustained else "bf16_tflops")
        achieved = (self.work / P) / (ms_step * 1e-3) / 1e12
        r = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
             "frac": achieved / peak if peak else None, "traffic": None,
             "peak_source": f"{peak_src} ({'sustained' if sustained else 'burst'} cuBLAS bf16)"}
        if P > 1:
            ingress = 2.0 * self.M * self.K * (P - 1) / P
            r["nvlink"] = {"ingress_bytes_per_step": ingress, "achieved_gbs": ingress / (ms_step * 1e-3) / 1e9,
                           "peak_gbs": NVLINK_GBS, "floor_ms": ingress / (NVLINK_GBS * 1e9) * 1e3}
        return r


class MxGemm:
    """MXFP8 GEMM 8192^3 (e4m3 with one e8m0 scale per 1x32 block, scales applied by the tensor core):
    the shape the reference's GEMM benchmarks use (kernels/cdna4/gemm/mxfp8, analysis/fp8_gemm)."""
    metric, unit, dtype, scaling = "gemm_mxfp8_tflops", "TFLOP/s", "fp8_e4m3", "weak"
    launches_per_step = 1
    M = N = K = 8192

    def __init__(self, ctx):
        import torch
        self.ctx = ctx
        g = torch.Generator(device="cuda").manual_seed(3000 + ctx.rank)
        self.sets = []
        for _ in range(3):          # 3 x 134 MB of operands rotated: more than L2 between two uses
            a = torch.randn(self.M, self.K, device="cuda", generator=g).to(torch.bfloat16)
            b = (torch.randn(self.N, self.K, device="cuda", generator=g) / math.sqrt(self.K)).to(torch.bfloat16)
            aq, sa, asf = ctx.capi.mx_quant(a)
            bq, sb, bsf = ctx.capi.mx_quant(b)
            self.sets.append((aq, asf, bq, bsf))
            self.rowmajor = (sa, sb)          # scales of the last set, row-major, for check()
        self.a_bf16 = a
        self.work = 2.0 * self.M * self.N * self.K * ctx.world
        self.scale = 1e12

    def step(self, i):
        aq, asf, bq, bsf = self.sets[i % 3]
        self.out = self.ctx.tk.gemm_mxfp8(aq, asf, bq, bsf)

    def quant_gbs(self):
        """The quantiser alone: 2 bytes read + 1 written per element (+ scales)."""
        import torch
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            self.ctx.capi.mx_quant(self.a_bf16)
        e0.record()
        for _ in range(10):
            self.ctx.capi.mx_quant(self.a_bf16)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 10
        return self.M * self.K * (3 + 1.0 / 32 + 4.0 / 128) / (ms * 1e-3) / 1e9

    def check(self):
        """64 rows of the fp32-output GEMM against torch on the dequantised operands."""
        import torch
        aq, asf, bq, bsf = self.sets[2]
        sa, sb = self.rowmajor
        out = self.ctx.tk.gemm_mxfp8(aq, asf, bq, bsf, True)
        torch.cuda.synchronize()

        def deq(q, sc):
            f = torch.ldexp(torch.ones_like(sc, dtype=torch.float32), sc.to(torch.int32) - 127)
            return q.view(torch.float8_e4m3fn).float() * f.repeat_interleave(32, dim=1)
        ref = deq(aq[:64], sa[:64]) @ deq(bq, sb).T
        return self.ctx.max_over_ranks(((out[:64] - ref).norm() / ref.norm()).item())

    def e2e_setup(self):
        return None

    def config(self, value):
        return {"workload": f"MXFP8 GEMM {self.M}x{self.N}x{self.K} per GPU (e4m3, 1x32 e8m0 scales applied by the "
                            f"block-scaled MMA), bf16 out", "l2": "3 operand sets of 134 MB rotated",
                "per_gpu_tflops": value / self.ctx.world}

    def roofline(self, ms_step, sustained, peaks, peak_src):
        bf16 = peaks.get("bf16_tflops_sustained" if sustained else "bf16_tflops")
        ach = 2.0 * self.M * self.N * self.K / (ms_step * 1e-3) / 1e12
        return {"bound": "tensor", "achieved": ach, "peak": 2.0 * bf16 if bf16 else None, "unit": "TFLOP/s",
                "frac": ach / (2.0 * bf16) if bf16 else None, "frac_of_nominal_4500": ach / 4500.0, "traffic": None,
                "peak_source": f"2 x {peak_src} cuBLAS bf16 ({'sustained' if sustained else 'burst'}) taken as the fp8 dense peak"}


class AllReduce:
    """TP all-reduce of bf16 activations: decode [64 x 8192] (1 MiB) and prefill [8192 x 8192]
    (128 MiB); a step is one all-reduce of each."""
    metric, unit, dtype, scaling = "allreduce_busbw", "GB/s", "bf16", "weak"
    launches_per_step = 2
    HEAP_MB = 3 * 129 + 3 * 2 + 64

    def __init__(self, ctx):
        import torch
        self.ctx = ctx
        ctx.make_heap(self.HEAP_MB)
        # NVLS (in-switch reduction) when the system has NVLink multicast: a collective opt-in
        self.nvls = ctx.world > 1 and os.environ.get("DK_BENCH_NVLS", "1") != "0" and ctx.enable_multicast()
        g = torch.Generator(device="cuda").manual_seed(100 + ctx.rank)
        self.bufs = {}
        for name, shape in (("decode", (64, 8192)), ("prefill", (8192, 8192))):
            xs = []
            for _ in range(2):      # two input buffers, alternated
                t = torch.as_tensor(ctx.iris.empty(list(shape)), device="cuda").view(torch.bfloat16)
                t.copy_(torch.randn(*shape, device="cuda", generator=g).to(torch.bfloat16))
                xs.append(t)
            o = torch.as_tensor(ctx.iris.empty(list(shape)), device="cuda").view(torch.bfloat16)
            self.bufs[name] = (xs, o)
        P = ctx.world
        S = (64 * 8192 + 8192 * 8192) * 2
        self.work = S * (2.0 * (P - 1) / P if P > 1 else 1.0)     # bus bytes per step
        self.scale = 1e9
        self.detail = {}

    def step(self, i):
        for name in ("decode", "prefill"):
            xs, o = self.bufs[name]
            self.ctx.tk.allreduce(xs[i % 2], o, self.ctx.view, -1)

    def check(self):
        import torch
        ctx = self.ctx
        worst = 0.0
        for name in ("decode", "prefill"):
            xs, o = self.bufs[name]
            for algo in (((0, 1, 2) if self.nvls else (0, 1)) if ctx.world > 1 else (0,)):
                o.zero_()
                ctx.barrier()
                ctx.tk.allreduce(xs[0], o, ctx.view, algo)
                torch.cuda.synchronize()
                ref = xs[0].float().clone()
                if ctx.world > 1:
                    ctx.dist.all_reduce(ref)
                worst = max(worst, ((o.float() - ref).norm() / ref.norm()).item())
                ctx.barrier()
        return ctx.max_over_ranks(worst)

    def time_each(self):
        """Separate timings of the two messages and of both algorithms (reported in config)."""
        import torch
        out = {}
        for name in ("decode", "prefill"):
            xs, o = self.bufs[name]
            for algo, an in ((0, "oneshot"), (1, "twoshot"), (2, "nvls")):
                if (self.ctx.world == 1 and algo >= 1) or (algo == 2 and not self.nvls):
                    continue
                # called through the C ABI with prebuilt arguments: the Python entry point costs
                # more host time per call than the 1 MiB kernel runs
                import ctypes as C
                L = self.ctx.capi.lib()
                st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
                px = [C.c_void_p(t.data_ptr()) for t in xs]
                po, n_el, vw = C.c_void_p(o.data_ptr()), o.numel(), C.byref(self.ctx.dkview)
                for _ in range(3):
                    self.ctx.capi.check(L.dk_allreduce(px[0], po, n_el, algo, vw, st))
                self.ctx.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                n = 50
                e0.record()
                for j in range(n):
                    L.dk_allreduce(px[j % 2], po, n_el, algo, vw, st)
                e1.record()
                self.ctx.barrier()
                out[f"{name}_{an}_us"] = self.ctx.max_over_ranks(e0.elapsed_time(e1) / n) * 1e3
        self.detail = out

    def e2e_setup(self):
        return None

    def config(self, value):
        c = {"workload": f"TP all-reduce bf16, 1 MiB [64x8192] + 128 MiB [8192x8192] per step, "
                         f"{self.ctx.world} GPU(s), algorithm picked by size",
             "l2": "two input buffers alternated; the 128 MiB message exceeds L2",
             "nvls": bool(self.nvls)}
        c.update(self.detail)
        return c

    def roofline(self, ms_step, sustained, peaks, peak_src):
        ach = self.work / (ms_step * 1e-3) / 1e9
        return {"bound": "nvlink", "achieved": ach, "peak": NVLINK_GBS, "unit": "GB/s",
                "frac": ach / NVLINK_GBS, "traffic": None,
                "peak_source": "measured peer copy per direction, 770 GB/s (nominal 900)"}


class Moe:
    """fp8 block-scaled MoE layer through ONE call per step (tk_kernel.moe_layer_ep): route ->
    exchange of the routing table -> permutation -> dispatch (once per token and GPU) -> quantise ->
    gate/up grouped GEMM + SiLU*mul + requantise -> down grouped GEMM -> expert-side combine -> final
    sum at home. Expert-parallel when N > 1."""
    unit, dtype, scaling = "TFLOP/s", "fp8_e4m3", "strong"

    SHAPES = {"moe_mixtral": dict(T=16384, H=4096, F=14336, E=8, k=2, zipf=0.0,
                                  name="Mixtral-8x7B-shaped: 16384 tokens, hidden 4096, ffn 14336, E=8 top-2"),
              "moe_dsv3": dict(T=32768, H=7168, F=2048, E=256, k=8, zipf=1.1,
                               name="DeepSeek-V3-shaped: 32768 tokens, hidden 7168, expert inter 2048, "
                                    "E=256 top-8, Zipf(1.1)")}

    @classmethod
    def heap_mb(cls, ctx, which, tokens=0):
        s = cls.SHAPES[which]
        T = tokens or s["T"]
        n = ctx.tk.moe_ep_workspace_bytes(T // ctx.world, s["k"], s["E"], s["H"], s["F"], ctx.world)
        return n // (1 << 20) + 64

    def __init__(self, ctx, which, scales="fp32"):
        """scales: "fp32" = 128x128 blocks with fp32 scales, promoted in software every 128 of K (the
        format the configurations name); "pow2" = the same blocks with power-of-two scales, applied
        by the tensor core (tcgen05 block-scaled MMA); "pow2_fp8" = as "pow2", and every token is
        quantised per 128 channels on its home rank and crosses NVLink as fp8 (1x128 activation scales)."""
        import torch
        self.ctx = ctx
        self.pow2 = scales != "fp32"
        self.mode = {"fp32": 0, "pow2": 1, "pow2_fp8": 2}[scales]
        s = self.SHAPES[which]
        self.which = which
        self.metric = which + "_tflops"
        self.scales = scales
        self.s = s
        P, rank = ctx.world, ctx.rank
        T, H, F, E, k = s["T"], s["H"], s["F"], s["E"], s["k"]
        assert E % P == 0 and T % P == 0
        self.epr, self.Tl = E // P, T // P
        capi = ctx.capi
        ctx.make_heap(self.heap_mb(ctx, which))
        g = torch.Generator(device="cuda").manual_seed(7 + rank)
        self.x = torch.randn(self.Tl, H, device="cuda", generator=g).to(torch.bfloat16)
        logits = torch.randn(self.Tl, E, device="cuda", generator=g)
        if s["zipf"] > 0:
            pi = torch.randperm(E, generator=torch.Generator().manual_seed(1)).float()
            p = (pi + 1.0) ** (-s["zipf"])
            logits = logits + torch.log(p / p.sum()).cuda()[None, :]
        self.logits = logits.contiguous()
        # this rank's experts, quantised with the library's own block quantisers
        w13q, w13s, w2q, w2s = [], [], [], []

        def quant_w(w):
            if self.pow2:
                q, _, _, atoms = capi.quant_block128_pow2(w)
                return q, atoms
            return capi.quant_block128(w)
        for _ in range(self.epr):
            w = (torch.randn(2 * F, H, device="cuda", generator=g) / math.sqrt(H)).to(torch.bfloat16)
            q, sc = quant_w(w)
            w13q.append(q)
            w13s.append(sc)
            w = (torch.randn(H, F, device="cuda", generator=g) / math.sqrt(F)).to(torch.bfloat16)
            q, sc = quant_w(w)
            w2q.append(q)
            w2s.append(sc)
            del w
        self.w13q, self.w13s = torch.stack(w13q), torch.stack(w13s)
        self.w2q, self.w2s = torch.stack(w2q), torch.stack(w2s)
        if self.pow2:             # block atoms of all experts, one row block after the other
            self.w13s = self.w13s.reshape(-1, self.w13s.shape[-2], 512)
            self.w2s = self.w2s.reshape(-1, self.w2s.shape[-2], 512)
        del w13q, w2q
        nbytes = ctx.tk.moe_ep_workspace_bytes(self.Tl, k, E, H, F, P)
        self.ws_t = ctx.iris.empty([nbytes], "uint8")           # the layer's workspace, inside the heap
        self.ws = torch.as_tensor(self.ws_t, device="cuda")
        self.out = torch.empty(self.Tl, H, dtype=torch.bfloat16, device="cuda")
        self.counts = torch.zeros(self.epr, dtype=torch.int32, device="cuda")
        self.work = float(T) * k * (2.0 * H * 2 * F + 2.0 * F * H)      # useful FLOP per step, whole job
        self.per_pair = 2.0 * H * 2 * F + 2.0 * F * H
        self.scale = 1e12
        # route, memset, hist, scan, place, 2 slot kernels, (dispatch), quantise, 2 grouped GEMMs,
        # combine push, final sum
        # (one rank without the fp8 dispatch: no dispatch kernel, the quantiser gathers straight from x)
        self.launches_per_step = 12 if (P == 1 and self.mode != 2) else 13
        self.gemm_ms = None
        ctx.barrier()

    def step(self, i):
        ctx = self.ctx
        return ctx.tk.moe_layer_ep(self.x, self.logits, self.s["k"], self.w13q, self.w13s, self.w2q, self.w2s,
                                   self.out, self.ws, ctx.view, self.mode, self.counts)

    def time_gemm(self):
        """The two grouped GEMMs timed inside the layer (events recorded by the call itself), median of
        five steps; pair counts of this rank and of the most loaded rank."""
        import torch
        ctx = self.ctx
        e = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        for ev in e:
            ev.record()
        torch.cuda.synchronize()
        ts = []
        for i in range(5):
            ctx.capi.moe_ep_layer(self.x, self.logits, self.w13q, self.w13s, self.w2q, self.w2s, self.out,
                                  self.ws.data_ptr(), ctx.dkview, self.s["k"],
                                  scale_mode=self.mode, counts_out=self.counts, gemm_events=e)
            ctx.barrier()
            ts.append(e[0].elapsed_time(e[1]))
        ts.sort()
        self.gemm_ms = ts[len(ts) // 2]
        self.pairs_rank = int(self.counts.sum().item())
        # the step is timed as the max over ranks: say what the most loaded rank carried
        self.pairs_max = int(ctx.max_over_ranks(float(self.pairs_rank)))
        self.gemm_ms_max = ctx.max_over_ranks(self.gemm_ms)
        self.gemm_tflops_min = -ctx.max_over_ranks(-self.pairs_rank * self.per_pair / (self.gemm_ms * 1e-3) / 1e12)

    def check(self):
        """The layer's output against the same arithmetic with NCCL as the exchange: tokens and logits
        are all-gathered, every rank runs its own experts on ALL tokens routed to them through the
        single-purpose entry points (route, permute, quantise, grouped GEMMs), scatters w * y into a
        dense fp32 [T, H] buffer, and a NCCL all-reduce forms the reference. Outside the timed region;
        relative Frobenius error of this rank's tokens, max over ranks."""
        import torch
        ctx, s = self.ctx, self.s
        capi, dist = ctx.capi, ctx.dist
        P, r, k, E, H = ctx.world, ctx.rank, s["k"], s["E"], s["H"]
        out = self.step(0).clone()
        torch.cuda.synchronize()
        if P > 1:
            xs = [torch.empty_like(self.x) for _ in range(P)]
            ls = [torch.empty_like(self.logits) for _ in range(P)]
            dist.all_gather(xs, self.x)
            dist.all_gather(ls, self.logits)
            x_all, lg_all = torch.cat(xs), torch.cat(ls)
            del xs, ls
        else:
            x_all, lg_all = self.x, self.logits
        idx, w = capi.moe_route(lg_all, k)
        # what this rank's tokens send: one vector per (token, other GPU) after per-GPU dedup,
        # against one per (token, expert on another GPU) without it
        dests = (idx[r * self.Tl:(r + 1) * self.Tl] // self.epr).long()
        onehot = torch.zeros(self.Tl, P, dtype=torch.bool, device="cuda")
        onehot.scatter_(1, dests, True)
        onehot[:, r] = False
        self._vectors = int(onehot.sum().item())
        self._remote_pairs = int((dests != r).sum().item())
        rop, por, offs, _ = capi.moe_permute(idx, E, 128, experts_per_segment=self.epr)
        por_me, offs_me = (por, offs) if P == 1 else (por[r].contiguous(), offs[r].contiguous())
        cap = por_me.shape[0]
        if self.mode == 2:
            q, atoms = self._rows128_pow2(x_all, por_me, k)
            y = capi.moe_ffn_mxfp8(q, atoms, self.w13q, self.w13s, self.w2q, self.w2s, offs_me)
            del atoms
        elif self.pow2:
            q, _, _, atoms = capi.quant_block128_pow2(x_all, rows=cap, row_map=por_me, map_mode=1, k=k)
            y = capi.moe_ffn_mxfp8(q, atoms, self.w13q, self.w13s, self.w2q, self.w2s, offs_me)
        else:
            q, sc = capi.quant_block128(x_all, rows=cap, row_map=por_me, map_mode=1, k=k)
            y = capi.moe_ffn_fp8(q, sc, self.w13q, self.w13s, self.w2q, self.w2s, offs_me)
        del q
        T = x_all.shape[0]
        contrib = torch.zeros(T, H, dtype=torch.float32, device="cuda")
        mine = (idx // self.epr) == r
        tok = torch.arange(T, device="cuda")[:, None].expand(T, k)[mine]
        rows, wts = rop[mine].long(), w[mine]
        for c0 in range(0, tok.numel(), 16384):
            sl = slice(c0, c0 + 16384)
            contrib.index_add_(0, tok[sl], wts[sl, None] * y[rows[sl]].float())
        del y
        if P > 1:
            dist.all_reduce(contrib)
        ref = contrib[r * self.Tl:(r + 1) * self.Tl]
        err = ((out.float() - ref).norm() / ref.norm()).item()
        del contrib
        return ctx.max_over_ranks(err)

    @staticmethod
    def _rows128_pow2(x_all, por, k):
        """The check's own statement of the fp8 dispatch, in torch on the GPU: expert rows gathered
        from the tokens, every 1x128 group of a row scaled by s = 2^ceil(log2(amax/448)) (1 for
        zeros) and rounded to e4m3; the scale bytes as the atoms the grouped GEMM reads (row slot
        i = 32*i1 + i0 of a 128-row block owns bytes i0*16 + i1*4 .. +3 of each atom of four column
        blocks). Returns (q uint8 [cap, H], atoms uint8 [cap/128, ceil(H/512), 512])."""
        import torch
        cap, H = por.shape[0], x_all.shape[1]
        nb = H // 128
        nj = (nb + 3) // 4
        q = torch.zeros(cap, H, dtype=torch.uint8, device="cuda")
        e8 = torch.full((cap, 4 * nj), 127, dtype=torch.uint8, device="cuda")
        for r0 in range(0, cap, 8192):
            pr = por[r0:r0 + 8192].long()
            live = pr >= 0
            xf = x_all[(pr.clamp(min=0) // k)].float() * live[:, None]
            g = xf.reshape(-1, nb, 128)
            amax = g.abs().amax(dim=2)
            m, e = torch.frexp(amax / 448.0)
            e = torch.where(m == 0.5, e - 1, e).to(torch.int32)
            e = torch.where(amax > 0, e, torch.zeros_like(e)).clamp(-127, 127)
            sc = torch.ldexp(torch.ones_like(amax), e)
            q[r0:r0 + 8192] = (g / sc[:, :, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).reshape(-1, H).view(torch.uint8)
            e8[r0:r0 + 8192, :nb] = (e + 127).to(torch.uint8)
        atoms = e8.reshape(cap // 128, 4, 32, nj, 4).permute(0, 3, 2, 1, 4).contiguous().reshape(cap // 128, nj, 512)
        return q, atoms

    def exchange_volume(self):
        """NVLink bytes this rank's tokens cause (after check() has counted them): dispatch sends one
        vector per (token, other GPU), bf16 or (fp8 dispatch) e4m3 + one scale byte per 128 channels
        padded to 16 bytes; combine returns one bf16 vector per (token, other GPU)."""
        vb = self.s["H"] * 2
        if self.mode == 2:
            return {"dispatch_egress_bytes_rank0": self._vectors * (self.s["H"] + (self.s["H"] // 128 + 15) // 16 * 16),
                    "combine_ingress_bytes_rank0": self._vectors * vb,
                    "vectors_per_direction_rank0": self._vectors, "pairs_on_other_gpus_rank0": self._remote_pairs}
        return {"dispatch_egress_bytes_rank0": self._vectors * vb, "combine_ingress_bytes_rank0": self._vectors * vb,
                "vectors_per_direction_rank0": self._vectors, "pairs_on_other_gpus_rank0": self._remote_pairs}

    def e2e_setup(self):
        import torch
        self.hx = torch.empty(self.x.shape, dtype=self.x.dtype).pin_memory()
        self.hx.copy_(self.x)
        self.hl = torch.empty(self.logits.shape, dtype=self.logits.dtype).pin_memory()
        self.hl.copy_(self.logits)
        self.ho = torch.empty(self.Tl, self.s["H"], dtype=torch.bfloat16).pin_memory()
        return self.hx.numel() * 2 + self.hl.numel() * 4, self.ho.numel() * 2

    def e2e_step(self):
        self.x.copy_(self.hx, non_blocking=True)
        self.logits.copy_(self.hl, non_blocking=True)
        out = self.step(0)
        self.ho.copy_(out, non_blocking=True)

    def config(self, value):
        s, P = self.s, self.ctx.world
        c = {"workload": f"fp8 MoE layer, {s['name']}, 128x128 block scales "
                         f"({'power-of-two, applied by the tensor core' if self.pow2 else 'fp32, promoted in software'})"
                         f"{', tokens dispatched as fp8 with 1x128 scales' if self.mode == 2 else ''}, EP={P}",
             "l2": f"expert weights ({(self.w13q.numel() + self.w2q.numel()) / 1e6:.0f} MB fp8 on this GPU) exceed L2",
             "per_gpu_tflops": value / P}
        if self.gemm_ms:
            c["grouped_gemm_ms_rank0"] = self.gemm_ms
            c["grouped_gemm_tflops_rank0"] = self.pairs_rank * self.per_pair / (self.gemm_ms * 1e-3) / 1e12
            c["pairs_rank0"] = self.pairs_rank
            c["pairs_max_rank"] = self.pairs_max
            c["grouped_gemm_ms_max_rank"] = self.gemm_ms_max
        return c

    def roofline(self, ms_step, sustained, peaks, peak_src):
        bf16 = peaks.get("bf16_tflops_sustained" if sustained else "bf16_tflops")
        peak = 2.0 * bf16 if bf16 else None          # no measured fp8 figure: twice the measured bf16 GEMM
        if self.gemm_ms:
            ach = self.pairs_rank * self.per_pair / (self.gemm_ms * 1e-3) / 1e12
            what = "grouped GEMM kernels alone (rank 0)"
        else:
            ach = (self.work / self.ctx.world) / (ms_step * 1e-3) / 1e12
            what = "whole step"
        return {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                "frac": ach / peak if peak else None,
                "frac_of_nominal_4500": ach / 4500.0,
                "traffic": load_traffic(self.metric + ("_pow2" if self.pow2 else "")), "of": what,
                "peak_source": f"2 x {peak_src} cuBLAS bf16 ({'sustained' if sustained else 'burst'}) "
                               f"taken as the fp8 dense peak"}


class Ctx:
    def __init__(self, rank, world, local_rank):
        import torch
        import torch.distributed as dist
        import iris_py
        import tk_kernel
        from __graft_entry__ import load_package
        self.rank, self.world, self.local_rank = rank, world, local_rank
        self.torch, self.dist, self.iris_py, self.tk = torch, dist, iris_py, tk_kernel
        self.capi = load_package().capi
        self.iris = None

    def make_heap(self, mb):
        """The symmetric heap of this process, created on the first call (later calls reuse it: blocks
        return to it when the tensors that own them die)."""
        if self.iris is not None:
            return
        self.iris = self.iris_py.Iris(heap_size_mb=int(mb), verbose=False)
        assert self.iris.rank() == self.rank and self.iris.world_size() == self.world
        self.view = self.iris.get_device_view()
        self.dkview = self.capi.DkView.from_address(self.view._addr())

    def enable_multicast(self):
        """Collective: map the NVLink multicast object over the heaps; the view is refreshed."""
        ok = bool(self.iris.enable_multicast())
        if ok:
            self.view = self.iris.get_device_view()
            self.dkview = self.capi.DkView.from_address(self.view._addr())
        return ok

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v):
        t = self.torch.tensor([v], device="cuda", dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.item()


def _claim_stdout():
    """Keep the real stdout for the one JSON line; whatever libraries print (NCCL's version banner
    goes to stdout) is sent to stderr instead."""
    real = os.fdopen(os.dup(1), "w")
    sys.stdout.flush()
    os.dup2(2, 1)
    return real


def time_steps(ctx, wl, steps, warmup):
    """W untimed steps, then K steps between CUDA events, barrier + synchronize on both sides.
    Returns (milliseconds per step as the max over ranks, wall-clock interval of the timed region)."""
    import torch
    ctx.barrier()
    for i in range(warmup):
        wl.step(i)
    ctx.barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    ev0.record()
    for i in range(steps):
        wl.step(i)
    ev1.record()
    ctx.barrier()
    return ctx.max_over_ranks(ev0.elapsed_time(ev1)) / steps, (t0, time.time())


def moe_secondary(ctx, which, scales, peaks, tokens=0):
    """One MoE configuration at the launched number of GPUs: step time, the grouped GEMMs timed inside
    the step, the share of the step that is not GEMM, the exchange volume, and a parity check."""
    if tokens:
        Moe.SHAPES[which] = dict(Moe.SHAPES[which], T=tokens)
    wl = Moe(ctx, which, scales)
    ms, _ = time_steps(ctx, wl, steps=10, warmup=3)
    wl.time_gemm()
    err = wl.check()
    P = ctx.world
    tf_job = wl.work / (ms * 1e-3) / 1e12
    gemm_tf = wl.pairs_rank * wl.per_pair / (wl.gemm_ms * 1e-3) / 1e12
    burst, sust = peaks.get("bf16_tflops"), peaks.get("bf16_tflops_sustained")
    e = {"workload": wl.config(tf_job)["workload"], "step_ms": ms, "tflops_whole_job": tf_job,
         "tflops_per_gpu": tf_job / P,
         "grouped_gemm_tflops_per_gpu_rank0": gemm_tf,
         "grouped_gemm_tflops_per_gpu_slowest_rank": wl.gemm_tflops_min,
         "grouped_gemm_ms_rank0": wl.gemm_ms, "grouped_gemm_ms_max_rank": wl.gemm_ms_max,
         "roofline_frac_of_2x_measured_bf16_burst": gemm_tf / (2 * burst) if burst else None,
         "roofline_frac_of_2x_measured_bf16_sustained": gemm_tf / (2 * sust) if sust else None,
         "roofline_frac_of_nominal_4500": gemm_tf / 4500.0,
         "non_gemm_share_of_step": max(0.0, 1.0 - wl.gemm_ms_max / ms),
         "pairs_rank0": wl.pairs_rank, "pairs_max_rank": wl.pairs_max,
         "traffic": load_traffic(wl.metric + ("_pow2" if scales != "fp32" else "")),
         "check_rel_fro": err}
    e.update(wl.exchange_volume())
    assert err <= 2e-2, f"{which} ({scales}): layer differs from the NCCL-exchanged reference by {err}"
    del wl
    import gc
    import torch
    gc.collect()
    torch.cuda.empty_cache()
    return e


def ag_gemm_secondary(ctx, peaks, peak_src):
    wl = AgGemm(ctx)
    ms, _ = time_steps(ctx, wl, steps=20, warmup=5)
    err = wl.check()
    value = wl.work / (ms * 1e-3) / 1e12
    e = {"workload": wl.config(value)["workload"], "step_ms": ms, "tflops_whole_job": value,
         "tflops_per_gpu": value / ctx.world, "check_rel_fro": err, "roofline": wl.roofline(ms, False, peaks, peak_src)}
    assert err <= 1e-2, f"all-gather + GEMM differs from the NCCL-gathered reference by {err}"
    del wl
    return e


def mx_gemm_secondary(ctx, peaks, peak_src):
    wl = MxGemm(ctx)
    ms, _ = time_steps(ctx, wl, steps=20, warmup=5)
    err = wl.check()
    r = wl.roofline(ms, False, peaks, peak_src)
    e = {"workload": wl.config(0.0)["workload"], "step_ms": ms, "tflops_per_gpu": r["achieved"], "roofline": r,
         "quantiser_hbm_gbs": wl.quant_gbs(), "quantiser_frac_of_measured_hbm": None, "check_rel_fro": err}
    if peaks.get("hbm_gbs"):
        e["quantiser_frac_of_measured_hbm"] = e["quantiser_hbm_gbs"] / peaks["hbm_gbs"]
    assert err <= 1e-3, f"MXFP8 GEMM differs from the dequantised torch reference by {err}"
    del wl
    return e


def allreduce_secondary(ctx):
    wl = AllReduce(ctx)
    ms, _ = time_steps(ctx, wl, steps=10, warmup=3)
    wl.time_each()
    err = wl.check()
    P = ctx.world
    e = {"nvls": bool(wl.nvls), "check_rel_fro": err, "step_busbw_gbs": wl.work / (ms * 1e-3) / 1e9}
    for name, nbytes in (("decode", 64 * 8192 * 2), ("prefill", 8192 * 8192 * 2)):
        for an in ("oneshot", "twoshot", "nvls"):
            us = wl.detail.get(f"{name}_{an}_us")
            if us is not None:
                e[f"{name}_{an}_us"] = us
                e[f"{name}_{an}_busbw_gbs"] = nbytes * 2.0 * (P - 1) / P / (us * 1e-6) / 1e9
    assert err <= 1e-2, f"all-reduce differs from the NCCL sum by {err}"
    del wl
    return e


def run_emulated(args, out):
    """--emulate-ranks P: the multi-rank kernels with all P ranks on ONE GPU (every rank's heap is a
    region of one buffer; phases run rank after rank, the all-reduce as one cooperative launch), for
    profiling them where only one GPU can be profiled. Not a benchmark of the metric: NVLink is not
    involved, the figures are HBM-side. Prints one JSON line with the per-phase times."""
    import torch
    from __graft_entry__ import load_package
    capi = load_package().capi
    P, steps, warm = args.emulate_ranks, args.steps, max(args.warmup, 3)
    torch.cuda.set_device(0)

    def job(ws_bytes):
        region = capi.CTRL_BYTES + (ws_bytes + 4095) // 4096 * 4096
        buf = torch.zeros(P * region + 4096, dtype=torch.uint8, device="cuda")
        base0 = (buf.data_ptr() + 1023) // 1024 * 1024
        bases = [base0 + r * region for r in range(P)]
        return buf, [capi.make_view(r, P, bases, region) for r in range(P)], [b + capi.CTRL_BYTES for b in bases]

    def timed(fn, first_seq=1):
        seq = first_seq
        for _ in range(warm):
            fn(seq)
            seq += 1
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn(seq)
            seq += 1
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps, seq

    g = torch.Generator(device="cuda").manual_seed(0)
    res = {"emulated_ranks": P, "workload": args.workload, "steps": steps}
    if args.workload == "allreduce":
        n = (args.tokens or 4096) * 4096                      # bf16 elements per rank (32 MiB by default)
        buf, views, ws = job(2 * n * 2 + 8192)
        xs = [capi.tensor_from_ptr(w, (n,), torch.bfloat16) for w in ws]
        outs = [capi.tensor_from_ptr(w + n * 2 + 4096, (n,), torch.bfloat16) for w in ws]
        for x in xs:
            x.copy_(torch.randn(n, device="cuda", generator=g).to(torch.bfloat16))
        seq = 1
        for algo, name in ((0, "oneshot"), (1, "twoshot")):
            ms, seq = timed(lambda s_, a=algo: capi.allreduce_all_ranks(views, xs, outs, a, s_), seq)
            res[f"{name}_ms"] = ms
            # every rank reads P inputs and writes one output (one-shot) / reads P slices, writes P slices
            res[f"{name}_hbm_gbs"] = (P * (P + 1) * n * 2 if algo == 0 else P * 2 * n * 2) / (ms * 1e-3) / 1e9
        res["bytes_per_rank"] = n * 2
    elif args.workload in ("gemm_rs", "ag_gemm"):
        M, N, K = (M_TOK, N_OUT, K_FULL) if args.shape else ((8192, 8192, 28672) if args.workload == "gemm_rs"
                                                             else (8192, 28672, 8192))
        if args.workload == "gemm_rs":
            Kl = K // P
            buf, views, ws = job(capi.gemm_rs_workspace_bytes(M, N, P))
            A = [torch.randn(M, Kl, device="cuda", generator=g).to(torch.bfloat16) for _ in range(P)]
            B = [(torch.randn(N, Kl, device="cuda", generator=g) / math.sqrt(K)).to(torch.bfloat16) for _ in range(P)]
            O = [torch.empty(M // P, N, dtype=torch.bfloat16, device="cuda") for _ in range(P)]
            call = lambda r, s_, ph: capi.gemm_rs_phase(A[r], B[r], O[r], ws[r], views[r], s_, ph)
            names = ("produce", "reduce")
        else:
            Nl = N // P
            buf, views, ws = job(capi.ag_gemm_workspace_bytes(M, K, P))
            A = [torch.randn(M // P, K, device="cuda", generator=g).to(torch.bfloat16) for _ in range(P)]
            B = [(torch.randn(Nl, K, device="cuda", generator=g) / math.sqrt(K)).to(torch.bfloat16) for _ in range(P)]
            O = [torch.empty(M, Nl, dtype=torch.bfloat16, device="cuda") for _ in range(P)]
            call = lambda r, s_, ph: capi.ag_gemm_phase(A[r], B[r], O[r], ws[r], views[r], s_, ph)
            names = ("push", "gemm")
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        acc = [0.0, 0.0]
        for it in range(warm + steps):
            seq = it + 1
            ev[0].record()
            for r in range(P):
                call(r, seq, 1)
            ev[1].record()
            for r in range(P):
                call(r, seq, 2)
            ev[2].record()
            torch.cuda.synchronize()
            if it >= warm:
                acc[0] += ev[0].elapsed_time(ev[1]) / steps
                acc[1] += ev[1].elapsed_time(ev[2]) / steps
        res.update({f"{names[0]}_ms_all_ranks": acc[0], f"{names[1]}_ms_all_ranks": acc[1], "shape": [M, N, K]})
    else:
        sh = dict(Moe.SHAPES[args.workload])
        T, H, F, k = args.tokens or 4096, sh["H"], sh["F"], sh["k"]
        E = args.experts or sh["E"]
        epr, Tl = E // P, T // P
        pow2 = args.scales != "fp32"
        mode = {"fp32": 0, "pow2": 1, "pow2_fp8": 2}[args.scales]
        buf, views, ws = job(capi.moe_ep_workspace_bytes(Tl, k, E, H, F, P))
        ranks = []
        for r in range(P):
            w13 = [(capi.quant_block128_pow2 if pow2 else capi.quant_block128)(
                (torch.randn(2 * F, H, device="cuda", generator=g) / math.sqrt(H)).to(torch.bfloat16)) for _ in range(epr)]
            w2 = [(capi.quant_block128_pow2 if pow2 else capi.quant_block128)(
                (torch.randn(H, F, device="cuda", generator=g) / math.sqrt(F)).to(torch.bfloat16)) for _ in range(epr)]
            si = 3 if pow2 else 1
            s13, s2 = torch.stack([w[si] for w in w13]), torch.stack([w[si] for w in w2])
            if pow2:
                s13, s2 = s13.reshape(-1, s13.shape[-2], 512), s2.reshape(-1, s2.shape[-2], 512)
            ranks.append(dict(x=torch.randn(Tl, H, device="cuda", generator=g).to(torch.bfloat16),
                              logits=torch.randn(Tl, E, device="cuda", generator=g),
                              w13q=torch.stack([w[0] for w in w13]), w13s=s13,
                              w2q=torch.stack([w[0] for w in w2]), w2s=s2,
                              out=torch.empty(Tl, H, dtype=torch.bfloat16, device="cuda")))

        def layer(seq):
            for ph in (1, 2, 4, 8):
                for r, d in enumerate(ranks):
                    capi.moe_ep_layer(d["x"], d["logits"], d["w13q"], d["w13s"], d["w2q"], d["w2s"], d["out"], ws[r],
                                      views[r], k, scale_mode=mode, epoch=seq, phases=ph)
        ms, _ = timed(layer)
        res.update({"layer_ms_all_ranks": ms, "tokens": T, "experts": E, "H": H, "F": F, "k": k, "scales": args.scales})
    st = capi.device_status()
    assert st[0] == 0, f"device-side error record: {st}"
    out.write(json.dumps(res) + "\n")
    out.flush()


def main():
    out = _claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemm_rs",
                    choices=["gemm_rs", "ag_gemm", "gemm_mxfp8", "allreduce", "moe_mixtral", "moe_dsv3"])
    ap.add_argument("--scales", default="fp32", choices=["fp32", "pow2", "pow2_fp8"],
                    help="MoE workloads: fp32 128x128 block scales (software promotion) or power-of-two "
                         "block scales applied by the block-scaled MMA; pow2_fp8: the latter with every token "
                         "quantised per 128 channels at home and dispatched as fp8")
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-secondary", action="store_true",
                    help="skip the other operators of the metric (MoE layers, all-reduce, sustained GEMM)")
    ap.add_argument("--shape", default=None, help="M,N,K override of the GEMM workload (profiling runs)")
    ap.add_argument("--check", action="store_true",
                    help="compare one result with a NCCL/torch reference outside the timed region "
                         "(always done when more than one GPU is used)")
    ap.add_argument("--tokens", type=int, default=0, help="token-count override of a MoE workload (profiling runs)")
    ap.add_argument("--experts", type=int, default=0, help="expert-count override with --emulate-ranks (profiling runs)")
    ap.add_argument("--emulate-ranks", type=int, default=0,
                    help="profiling runs: all ranks of a P-rank job on one GPU, phase by phase (see run_emulated)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 0)

    global M_TOK, N_OUT, K_FULL
    if args.shape:
        M_TOK, N_OUT, K_FULL = (int(v) for v in args.shape.split(","))
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if args.impl == "reference":
        run_reference(args, rank, out)
        return
    if args.emulate_ranks:
        assert world == 1, "--emulate-ranks runs on one GPU"
        run_emulated(args, out)
        return

    import torch
    import torch.distributed as dist
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU fallback)"
    assert world == args.gpus or world == 1, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"           # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    ctx = Ctx(rank, world, local_rank)
    secondary_on = args.workload == "gemm_rs" and not args.no_secondary and not args.shape
    # one symmetric heap for everything this run will do
    need = {"gemm_rs": GemmRs.heap_mb(world), "ag_gemm": AgGemm.heap_mb(world), "allreduce": AllReduce.HEAP_MB,
            "gemm_mxfp8": 64}
    for wname in ("moe_mixtral", "moe_dsv3"):
        need[wname] = Moe.heap_mb(ctx, wname, args.tokens if args.workload == wname else 0)
    heap_mb = need[args.workload] + (sum(v for k_, v in need.items() if k_ != args.workload) if secondary_on else 0)
    ctx.make_heap(heap_mb)

    if args.workload == "gemm_rs":
        wl = GemmRs(ctx)
    elif args.workload == "ag_gemm":
        wl = AgGemm(ctx)
    elif args.workload == "gemm_mxfp8":
        wl = MxGemm(ctx)
    elif args.workload == "allreduce":
        wl = AllReduce(ctx)
    else:
        if args.tokens:
            Moe.SHAPES[args.workload]["T"] = args.tokens
        wl = Moe(ctx, args.workload, args.scales)
    barrier = ctx.barrier

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        t_wait = time.time() + 8.0
        while not sampler.lines and time.time() < t_wait:   # let nvidia-smi finish starting up
            time.sleep(0.05)
    ms_step, (t_clock0, _) = time_steps(ctx, wl, args.steps, args.warmup)
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
            wl.step(i)
        extra += 10
        torch.cuda.synchronize()
    barrier()
    clocks = sampler.stop(t_clock0, time.time()) if sampler else None
    if clocks is not None:
        clocks["extended_by_untimed_steps"] = extra if clocks_extended else 0
    status = ctx.tk.device_status()
    assert status[0] == 0, f"device-side error record: {status}"
    value = wl.work / (ms_step * 1e-3) / wl.scale

    # parity outside the timed region: always when peers are involved
    check_err = None
    if args.check or world > 1:
        check_err = wl.check()
    if isinstance(wl, AllReduce):
        wl.time_each()
    if isinstance(wl, Moe):
        wl.time_gemm()

    # the same step back to back for at least two seconds: the figure a long-running job sees under
    # the power cap, against the sustained peak
    sustained_ms = None
    if isinstance(wl, GemmRs) and secondary_on:
        n = max(args.steps, int(math.ceil(2000.0 / ms_step)))
        sustained_ms, _ = time_steps(ctx, wl, n, 0)

    e2e_value = e2e_ms = None
    h2d = d2h = 0
    if not args.no_e2e:
        sizes = wl.e2e_setup()
        if sizes is not None:
            h2d, d2h = sizes
            barrier()
            wl.e2e_step()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.e2e_steps):
                wl.e2e_step()
            e1.record()
            barrier()
            e2e_ms = ctx.max_over_ranks(e0.elapsed_time(e1)) / args.e2e_steps
            e2e_value = wl.work / (e2e_ms * 1e-3) / wl.scale
    status = ctx.tk.device_status()
    assert status[0] == 0, f"device-side error record: {status}"

    peaks, peak_src = load_peaks()
    line = None
    if rank == 0:
        sustained = ms_step * args.steps * 1e-3 >= 1.0
        line = {
            "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": wl.scaling, "vs_baseline": None, "dtype": wl.dtype,
            "data": "synthetic",
            "config": wl.config(value),
            "roofline": wl.roofline(ms_step, sustained, peaks, peak_src),
            "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": args.e2e_steps},
            "gpu_launches": args.steps * wl.launches_per_step,
            "clocks": clocks,
        }
        if check_err is not None:
            line["check_rel_fro"] = check_err
        if sustained_ms is not None:
            r = wl.roofline(sustained_ms, True, peaks, peak_src)
            line["roofline"]["sustained"] = {"ms_per_step": sustained_ms, "achieved": r["achieved"], "peak": r["peak"],
                                             "frac": r["frac"], "peak_source": r["peak_source"],
                                             "seconds": sustained_ms * max(args.steps, int(math.ceil(2000.0 / ms_step))) * 1e-3}
        if world == 1 and not args.no_cpu_baseline and isinstance(wl, GemmRs):
            tf, threads, desc, dt = cpu_reference_tflops()
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                    "sample": desc, "seconds": dt}
    if check_err is not None and isinstance(wl, GemmRs):
        assert check_err <= 1e-2, f"GEMM + reduce-scatter differs from the NCCL sum by {check_err}"

    # the other operators the metric names, at the same number of GPUs
    if secondary_on:
        del wl
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        sec = {}
        sec["ag_gemm"] = ag_gemm_secondary(ctx, peaks, peak_src)
        sec["gemm_mxfp8"] = mx_gemm_secondary(ctx, peaks, peak_src)
        if world > 1:
            sec["allreduce"] = allreduce_secondary(ctx)
        for which in ("moe_mixtral", "moe_dsv3"):
            for scales in ("fp32", "pow2", "pow2_fp8"):
                sec[f"{which}_{scales}"] = moe_secondary(ctx, which, scales, peaks)
        if world == 1:
            sys.path.insert(0, str(ROOT / "examples"))
            import bench_gemm
            sec["gemm_reference_bench_shapes"] = bench_gemm.run(iters=20)
        status = ctx.tk.device_status()
        assert status[0] == 0, f"device-side error record: {status}"
        if line is not None:
            line["secondary"] = sec
    else:
        del wl
    if rank == 0:
        out.write(json.dumps(line) + "\n")
        out.flush()
    barrier()
    ctx.view = ctx.dkview = None
    ctx.iris = None
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
