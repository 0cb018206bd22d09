#!/usr/bin/env python
"""Single-GPU timing of tk_kernel.dispatch_micro(A, Bt, C) on the shapes of the reference's GEMM
benchmark script (kernels/cdna4/gemm/bf16fp32/bench.py:10-19), next to torch.matmul on the same
shapes. Prints one line per shape: milliseconds and TFLOP/s of both.

    python examples/bench_gemm.py [--iters 50]
"""
import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "distributed-hipkittens_b200"))
import tk_kernel    # noqa: E402

# (m, n, k)
SHAPES = [(8192, 8192, 8192), (4096, 8192, 2048), (8192, 4096, 2048), (8192, 2048, 4096),
          (4096, 4096, 4096), (2048, 4096, 4096), (2048, 2048, 4096), (2048, 2048, 2048)]


def time_ms(fn, iters, flush):
    for _ in range(5):
        fn()
    e0 = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    e1 = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    for i in range(iters):
        flush.zero_()                     # a buffer larger than L2 between timed launches
        e0[i].record()
        fn()
        e1[i].record()
    torch.cuda.synchronize()
    t = sorted(a.elapsed_time(b) for a, b in zip(e0, e1))
    return t[len(t) // 2]


def run(iters=50):
    torch.manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    rows = []
    for m, n, k in SHAPES:
        A = torch.randn(m, k, device="cuda").to(torch.bfloat16)
        Bt = torch.randn(n, k, device="cuda").to(torch.bfloat16)
        C = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        ours = time_ms(lambda: tk_kernel.dispatch_micro(A, Bt, C), iters, flush)
        ref = time_ms(lambda: torch.matmul(A, Bt.t(), out=C), iters, flush)
        fl = 2.0 * m * n * k
        rows.append({"shape": [m, n, k], "ms": ours, "tflops": fl / ours / 1e9, "torch_ms": ref,
                     "torch_tflops": fl / ref / 1e9})
    return rows


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=50)
    for r in run(ap.parse_args().iters):
        m, n, k = r["shape"]
        print(f"{m:5d} x {n:5d} x {k:5d}: dispatch_micro {r['ms']:.3f} ms {r['tflops']:7.0f} TFLOP/s | "
              f"torch.matmul {r['torch_ms']:.3f} ms {r['torch_tflops']:7.0f} TFLOP/s")
