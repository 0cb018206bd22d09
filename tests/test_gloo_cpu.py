"""Two CPU ranks under torch.distributed (gloo): the host-side logic of the multi-rank path.

What is exercised: K-sharding of the row-parallel GEMM against a real reduce-scatter, the
expert-parallel layout computed independently on every rank from an all-gathered routing table
(every rank must derive the same global permutation), the symmetric-heap bootstrap (dk_comm) running
next to a gloo process group, and host-side failure detection (a peer that leaves before the
barrier is reported, not waited for forever)."""
import ctypes as C
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _worker(rank, world, port, q):
    try:
        sys.path.insert(0, str(ROOT))
        from __graft_entry__ import load_package
        from oracle import dk_oracle as orc
        capi = load_package().capi
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        res = {}

        # ---- row-parallel GEMM + reduce-scatter: sharded partials, summed by gloo, vs the oracle
        M, N, K = 256, 128, 512
        A, Bt = orc.make_gemm_inputs(M, N, K, seed=0)          # same seed on every rank
        As, Bs = orc.shard_k(A, Bt, world)
        partial = orc.gemm_ref(As[rank], Bs[rank])
        mine = torch.empty(M // world, N)
        dist.reduce_scatter(mine, list(partial.chunk(world, 0)))
        res["gemm_rs"] = orc.rel_fro(mine, orc.gemm_rs_ref(As, Bs)[rank])
        res["gemm_full"] = orc.rel_fro(mine, orc.gemm_ref(A, Bt)[rank * (M // world):(rank + 1) * (M // world)])

        # ---- expert-parallel layout from an all-gathered routing table
        T, E, k = 64 * world, 4 * world, 2
        g = torch.Generator().manual_seed(3)
        logits = torch.randn(T, E, generator=g)
        Tl = T // world
        my_idx, _ = orc.moe_route(logits[rank * Tl:(rank + 1) * Tl].contiguous(), k)
        gathered = [torch.empty_like(my_idx) for _ in range(world)]
        dist.all_gather(gathered, my_idx)
        all_idx = torch.cat(gathered, 0)
        recv_pair, recv_offs, rop, dest = orc.ep_layout(all_idx, E, world)
        full_idx, _ = orc.moe_route(logits, k)
        res["route_consistent"] = bool(torch.equal(all_idx, full_idx))
        # rows this rank will receive, and a checksum of the global permutation every rank computed
        res["recv_rows"] = int((recv_pair[rank] >= 0).sum())
        res["perm_checksum"] = int((rop.long() * (torch.arange(T * k).reshape(T, k) + 1)).sum())
        res["pairs_to_me"] = int((dest == rank).sum())

        # ---- the heap's own bootstrap between the same two processes
        L = capi.lib()
        c = C.c_void_p()
        rc = L.dk_comm_create(rank, world, f"gloo.{port}".encode(), 20000, C.byref(c))
        blob = (C.c_int * world)()
        mine_i = C.c_int(1000 + rank)
        rc2 = L.dk_comm_allgather(c, C.byref(mine_i), 4, blob)
        rc3 = L.dk_comm_barrier(c)
        res["comm"] = (rc, rc2, rc3, list(blob))
        # failure detection: rank 1 leaves; rank 0's next barrier must return an error, quickly
        dist.barrier()
        if rank == 1:
            L.dk_comm_destroy(c)
            res["after_leave"] = None
        else:
            import time
            time.sleep(0.5)
            t0 = time.time()
            rc4 = L.dk_comm_barrier(c)
            res["after_leave"] = (rc4, time.time() - t0, L.dk_last_error_string().decode())
            L.dk_comm_destroy(c)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, res))
    except Exception:
        import traceback
        q.put((rank, {"error": traceback.format_exc()}))


def test_two_ranks_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 300
    ps = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in ps:
        p.start()
    out = dict(q.get(timeout=120) for _ in ps)
    for p in ps:
        p.join(30)
    for r in range(world):
        assert "error" not in out[r], out[r].get("error")
        assert out[r]["gemm_rs"] < 1e-5 and out[r]["gemm_full"] < 1e-5
        assert out[r]["route_consistent"]
        assert out[r]["recv_rows"] == out[r]["pairs_to_me"]
        assert out[r]["comm"] == (0, 0, 0, [1000, 1001])
    assert out[0]["perm_checksum"] == out[1]["perm_checksum"]
    assert out[0]["recv_rows"] + out[1]["recv_rows"] == 64 * world * 2
    rc4, dt, msg = out[0]["after_leave"]
    assert rc4 == 4 and dt < 5.0 and "barrier" in msg     # DK_ERR_BOOTSTRAP, not a hang


def test_reference_arm_under_torchrun_prints_one_line_from_rank0():
    """bench.py --impl reference launched like the GPU arm (torchrun, 2 ranks): rank 0 alone times
    the CPU path, with all the host threads it may use although torchrun exports OMP_NUM_THREADS=1,
    and prints ONE JSON line; the other rank exits 0 without work."""
    import json
    import subprocess
    port = 29900 + os.getpid() % 90
    env = dict(os.environ)
    env.pop("OMP_NUM_THREADS", None)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(ROOT / "bench.py"),
                        "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, r.stdout
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 2 and d["metric"] == "gemm_rs_tflops"
    assert d["cpu_baseline"]["kind"] == "port" and d["gpu_launches"] == 0
    assert d["e2e"]["value"] == d["value"] and d["e2e"]["h2d_bytes_per_step"] == 0
    try:
        avail = len(os.sched_getaffinity(0))
    except AttributeError:
        avail = os.cpu_count() or 1
    assert d["cpu_baseline"]["cores"] == avail
    assert "K-sharded over 2 GPU(s)" in d["config"]["workload"]
