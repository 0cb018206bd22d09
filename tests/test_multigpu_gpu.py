"""The multi-process path over real peer memory: one process per GPU, the symmetric heap mapped
across processes, GEMM + reduce-scatter and all-reduce checked against the oracle on every rank.
Needs at least two GPUs; skipped otherwise (the single-GPU tests drive the same kernels with all
ranks on one device)."""
import os
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _worker(rank, world, job, q):
    try:
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), DK_JOB_ID=job,
                          NCCL_NVLS_ENABLE="0")
        sys.path.insert(0, str(ROOT))
        sys.path.insert(0, str(ROOT / "distributed-hipkittens_b200"))
        import iris_py
        import tk_kernel
        from oracle import dk_oracle as orc
        torch.cuda.set_device(rank)
        iris = iris_py.Iris(heap_size_mb=192)
        assert iris.rank() == rank and iris.world_size() == world
        view = iris.get_device_view()
        res = {}

        # ---- GEMM + reduce-scatter, three calls on one workspace (both parities, flag reuse)
        M, N, K = 256 * world, 520, 512 * world
        A, Bt = orc.make_gemm_inputs(M, N, K, seed=0)
        As, Bs = orc.shard_k(A, Bt, world)
        want = orc.gemm_rs_ref(As, Bs)[rank]
        dA, dB = As[rank].cuda(), Bs[rank].cuda()
        out = torch.as_tensor(iris.empty([M // world, N]), device="cuda").view(torch.bfloat16)
        errs = []
        for _ in range(3):
            out.fill_(float("nan"))
            iris.barrier()
            tk_kernel.gemm_rs(dA, dB, out, view)
            torch.cuda.synchronize()
            errs.append(orc.rel_fro(out.float().cpu(), want))
        res["gemm_rs"] = errs

        # ---- all-reduce, one-shot and two-shot
        shape = (64, 8192)
        xs = orc.make_allreduce_inputs(shape, world)
        ref = orc.allreduce_ref(xs)
        x = torch.as_tensor(iris.empty(list(shape)), device="cuda").view(torch.bfloat16)
        o = torch.as_tensor(iris.empty(list(shape)), device="cuda").view(torch.bfloat16)
        for algo in (0, 1, -1):
            x.copy_(xs[rank])
            o.fill_(float("nan"))
            iris.barrier()
            tk_kernel.allreduce(x, o, view, algo)
            torch.cuda.synchronize()
            res[f"allreduce{algo}"] = orc.rel_fro(o.float().cpu(), ref)
            res[f"allreduce{algo}_sum"] = int(o.view(torch.int16).to(torch.int64).sum().item())
        res["status"] = tk_kernel.device_status()
        iris.barrier()
        q.put((rank, res))
        del out, x, o, view
        del iris
    except Exception as e:  # report instead of hanging the parent
        import traceback
        q.put((rank, {"error": traceback.format_exc()}))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_memory_path(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    job = f"pytest{os.getpid()}w{world}"
    ps = [ctx.Process(target=_worker, args=(r, world, job, q)) for r in range(world)]
    for p in ps:
        p.start()
    results = dict(q.get(timeout=240) for _ in ps)
    for p in ps:
        p.join(60)
    for r in range(world):
        assert "error" not in results[r], results[r].get("error")
        assert results[r]["status"][0] == 0
        assert all(e <= 1e-2 for e in results[r]["gemm_rs"]), results[r]["gemm_rs"]
        for algo in (0, 1, -1):
            assert results[r][f"allreduce{algo}"] <= 1e-2
            # every rank holds the same bits
            assert results[r][f"allreduce{algo}_sum"] == results[0][f"allreduce{algo}_sum"]
