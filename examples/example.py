#!/usr/bin/env python
"""The reference's distributed GEMM example, runnable against this build.

It makes the calls of distributed-kernels/bf16_gemm/example.py:60-122 in the same order with the same
numbers: operands allocated from the symmetric heap (`iris.empty`), M = 7680 rows split over the
ranks, K = N = 8192, A drawn with seed 1234 + rank and B with seed 0 on the GPU as bf16 randn / 10,
`tk_kernel.dispatch_micro(A, B, C, view, M_local, N, K, row_offset)`, then max |C - A B^T| < 0.1.

    python examples/example.py                                   # one GPU
    torchrun --nproc-per-node 8 examples/example.py              # one process per GPU
    python examples/example.py --as-rank 3 --of 8                # the 960-row shard of rank 3, on one GPU

Differences from the reference script: ranks come from RANK / WORLD_SIZE / LOCAL_RANK (or Open MPI's
variables) instead of MPI, `mpi4py` is used for the final MPI.Finalize only when it is installed, and
the process exits with status 1 when the check fails.
"""
import argparse
import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "distributed-hipkittens_b200"))
import iris_py      # noqa: E402
import tk_kernel    # noqa: E402


def heap_tensor(iris, shape):
    """bf16 torch view of a fresh heap block. `iris_py.Tensor` carries __cuda_array_interface__, so
    torch.as_tensor wraps the block without copying and keeps it alive."""
    return torch.as_tensor(iris.empty(list(shape), dtype="bfloat16"), device="cuda").view(torch.bfloat16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=192 * 40)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--scale", type=float, default=10.0)
    ap.add_argument("--heap-mb", type=int, default=512)
    ap.add_argument("--as-rank", type=int, default=None, help="run this rank's shard alone on one GPU")
    ap.add_argument("--of", type=int, default=1, help="world size the shard of --as-rank belongs to")
    args = ap.parse_args()

    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", os.environ.get("OMPI_COMM_WORLD_LOCAL_RANK", "0"))))
    iris = iris_py.Iris(heap_size_mb=args.heap_mb, verbose=False)
    rank, world = iris.rank(), iris.world_size()
    shard_rank, shard_world = (args.as_rank, args.of) if args.as_rank is not None else (rank, world)
    M, N, K = args.m, args.n, args.k
    M_local = M // shard_world
    say = print if rank == 0 else (lambda *a, **k: None)
    say(f"distributed GEMM {M}x{K} @ {K}x{N}: {shard_world} shard(s) of {M_local} rows, {world} process(es)")

    A, B, C = heap_tensor(iris, (M_local, K)), heap_tensor(iris, (N, K)), heap_tensor(iris, (M_local, N))
    torch.manual_seed(1234 + shard_rank)
    A.copy_(torch.randn(M_local, K, dtype=torch.bfloat16, device="cuda") / args.scale)
    torch.manual_seed(0)
    B.copy_(torch.randn(N, K, dtype=torch.bfloat16, device="cuda") / args.scale)
    C.zero_()
    iris.barrier()

    C_ref = torch.matmul(A, B.t())
    view = iris.get_device_view()
    tk_kernel.dispatch_micro(A, B, C, view, M_local, N, K, shard_rank * M_local)
    torch.cuda.synchronize()
    iris.barrier()

    status = tk_kernel.device_status()
    max_error = (C.float() - C_ref.float()).abs().max().item()
    ok = max_error < 0.1 and status[0] == 0
    print(f"Rank {shard_rank}: Max error: {max_error:.6f}, {'PASSED' if ok else 'FAILED'}", flush=True)

    del A, B, C, C_ref, view
    iris.barrier()
    del iris
    try:
        from mpi4py import MPI
        if MPI.Is_initialized() and not MPI.Is_finalized():
            MPI.Finalize()
    except ImportError:
        pass
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
