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

        # ---- all-gather + GEMM: every rank's row shard against this rank's own weight columns
        Ma, Na, Ka = 256 * world, 264, 512
        Afull, _ = orc.make_gemm_inputs(Ma, 8, Ka, seed=40)
        Bcol = orc.make_gemm_inputs(8, Na, Ka, seed=41 + rank)[1]
        want_ag = orc.gemm_ref(Afull, Bcol)
        sh = Ma // world
        dAs, dBc = Afull[rank * sh:(rank + 1) * sh].contiguous().cuda(), Bcol.cuda()
        out_ag = torch.empty(Ma, Na, dtype=torch.bfloat16, device="cuda")
        errs = []
        for _ in range(3):
            out_ag.fill_(float("nan"))
            iris.barrier()
            tk_kernel.ag_gemm(dAs, dBc, out_ag, view)
            torch.cuda.synchronize()
            errs.append(orc.rel_fro(out_ag.float().cpu(), want_ag))
        res["ag_gemm"] = errs

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
        # ---- expert-parallel MoE layer: all-gather of the routing table, dispatch, FFN, combine
        from __graft_entry__ import load_package
        capi = load_package().capi
        v = capi.DkView.from_address(view._addr())
        T, H, F, E, k = 128 * world, 256, 128, 4 * world, 2
        epr, Tl = E // world, T // world
        x, logits, w13q, w13s, w2q, w2s = orc.make_moe_inputs(T, H, F, E, k, seed=5, zipf_s=1.1)
        idx_c, w_c = orc.moe_route(logits, k)
        rop_c, por_c, offs_c, _ = orc.moe_permute(idx_c, E)
        xq_c, xs_c = orc.quant_block128(orc.moe_gather_rows(x, por_c, k))
        y_c, _, _ = orc.moe_ffn_ref(xq_c, xs_c, w13q, w13s, w2q, w2s, offs_c)
        want_moe = orc.moe_combine_ref(y_c, rop_c, w_c)[rank * Tl:(rank + 1) * Tl]
        sl = slice(rank * Tl, (rank + 1) * Tl)
        my_idx, my_w = capi.moe_route(logits[sl].contiguous().cuda(), k)
        all_idx = torch.as_tensor(iris.empty([T, k], "int32"), device="cuda")
        cap = capi.lib().dk_moe_rows_capacity(T, k, epr, 128)
        xrecv = torch.as_tensor(iris.empty([cap, H]), device="cuda").view(torch.bfloat16)
        ybuf = torch.as_tensor(iris.empty([cap, H]), device="cuda").view(torch.bfloat16)
        moe_errs = []
        for _ in range(2):
            xrecv.fill_(33.0)
            capi.allgather(my_idx, all_idx, v)
            rop, por, offs, counts = capi.moe_permute(all_idx, E, 128, experts_per_segment=epr)
            my_rop = rop[sl].contiguous()
            capi.moe_dispatch(x[sl].contiguous().cuda(), my_idx, my_rop, epr, xrecv, v, sync=True)
            xq, xs = capi.quant_block128(xrecv, row_map=por[rank].contiguous(), map_mode=2)
            es = slice(rank * epr, (rank + 1) * epr)
            y = capi.moe_ffn_fp8(xq, xs, w13q[es].cuda(), w13s[es].cuda(), w2q[es].cuda(), w2s[es].cuda(),
                                 offs[rank].contiguous())
            ybuf.copy_(y)
            out_moe = capi.moe_combine_ep(ybuf, my_idx, my_rop, my_w, epr, v, sync=True)
            torch.cuda.synchronize()
            moe_errs.append(orc.rel_fro(out_moe.float().cpu(), want_moe))
        res["moe_ep"] = moe_errs
        res["moe_idx_ok"] = bool(torch.equal(all_idx.cpu(), idx_c))

        # ---- the same layer as ONE call (dedup dispatch, expert-side combine, flags instead of
        # barriers), fp32 scales, power-of-two scales, then the latter with the fp8 dispatch; two calls each on one
        # workspace
        nbytes = tk_kernel.moe_ep_workspace_bytes(Tl, k, E, H, F, world)
        ws = torch.as_tensor(iris.empty([nbytes], "uint8"), device="cuda")
        ws.fill_(0xFF)                       # its contents need no initialisation
        counts = torch.empty(epr, dtype=torch.int32, device="cuda")
        out_l = torch.empty(Tl, H, dtype=torch.bfloat16, device="cuda")
        layer_errs = []
        torch.cuda.synchronize()
        iris.barrier()
        for scale_mode in (0, 1, 2):     # 2: tokens cross as fp8 with 1x128 scales (weights as in mode 1)
            if scale_mode == 0:
                a13, a2 = w13s[es].contiguous().cuda(), w2s[es].contiguous().cuda()
                q13, q2 = w13q[es].contiguous().cuda(), w2q[es].contiguous().cuda()
                want_l = want_moe
            elif scale_mode == 2:
                xq_r, xs_r, _ = orc.quant_rows128_pow2(orc.moe_gather_rows(x, por_c, k))
                y_r = orc.moe_ffn_rows_pow2_ref(xq_r, xs_r, st(p13, 0), st(p13, 1), st(p2, 0), st(p2, 1), offs_c)[0]
                want_l = orc.moe_combine_ref(y_r, rop_c, w_c)[sl]
            else:
                import math
                g = torch.Generator().manual_seed(99)
                p13 = [orc.quant_block128_pow2((torch.randn(2 * F, H, generator=g) / math.sqrt(H)).to(torch.bfloat16))
                       for _ in range(E)]
                p2 = [orc.quant_block128_pow2((torch.randn(H, F, generator=g) / math.sqrt(F)).to(torch.bfloat16))
                      for _ in range(E)]
                st = lambda parts, i: torch.stack([t[i] for t in parts])
                xq_p, xs_p, _ = orc.quant_block128_pow2(orc.moe_gather_rows(x, por_c, k))
                y_p = orc.moe_ffn_pow2_ref(xq_p, xs_p, st(p13, 0), st(p13, 1), st(p2, 0), st(p2, 1), offs_c)[0]
                want_l = orc.moe_combine_ref(y_p, rop_c, w_c)[sl]
                q13, q2 = st(p13, 0)[es].contiguous().cuda(), st(p2, 0)[es].contiguous().cuda()
                e13, e2 = st(p13, 2)[es], st(p2, 2)[es]
                a13 = orc.block128_scales_to_block_atoms(e13.reshape(-1, e13.shape[-1])).cuda()
                a2 = orc.block128_scales_to_block_atoms(e2.reshape(-1, e2.shape[-1])).cuda()
            for _ in range(2):
                out_l.fill_(float("nan"))
                tk_kernel.moe_layer_ep(x[sl].contiguous().cuda(), logits[sl].contiguous().cuda(), k, q13, a13, q2, a2,
                                       out_l, ws, view, scale_mode, counts)
                torch.cuda.synchronize()
                layer_errs.append(orc.rel_fro(out_l.float().cpu(), want_l))
        # the same call with its number kept on the device, captured into a CUDA graph after one eager
        # call and replayed on new tokens (weights and scale mode of the last round above)
        xs_g, ls_g = x[sl].contiguous().cuda(), logits[sl].contiguous().cuda()
        counts_g = torch.empty_like(counts)
        call = lambda: tk_kernel.moe_layer_ep(xs_g, ls_g, k, q13, a13, q2, a2, out_l, ws, view, 2, counts_g, True)
        call()
        torch.cuda.synchronize()
        iris.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            call()
        for seed in (71, 72):
            gg = torch.Generator().manual_seed(seed)
            x_g = torch.randn(T, H, generator=gg).to(torch.bfloat16)
            lg_g = torch.randn(T, E, generator=gg)
            idx_g, w_g = orc.moe_route(lg_g, k)
            rop_g, por_g, offs_g, _ = orc.moe_permute(idx_g, E)
            xq_r, xs_r, _ = orc.quant_rows128_pow2(orc.moe_gather_rows(x_g, por_g, k))
            y_r = orc.moe_ffn_rows_pow2_ref(xq_r, xs_r, st(p13, 0), st(p13, 1), st(p2, 0), st(p2, 1), offs_g)[0]
            want_g = orc.moe_combine_ref(y_r, rop_g, w_g)[sl]
            xs_g.copy_(x_g[sl])
            ls_g.copy_(lg_g[sl])
            out_l.fill_(float("nan"))
            torch.cuda.synchronize()
            graph.replay()
            torch.cuda.synchronize()
            layer_errs.append(orc.rel_fro(out_l.float().cpu(), want_g))
        del graph
        res["moe_layer"] = layer_errs
        want_counts = torch.bincount(idx_c.reshape(-1).long(), minlength=E)[es]
        res["moe_layer_counts_ok"] = bool(torch.equal(counts.cpu().long(), want_counts))
        iris.barrier()
        del ws
        res["status"] = tk_kernel.device_status()
        iris.barrier()
        del out, x, o, view, all_idx, xrecv, ybuf
        del iris
        # ---- a second heap in the same process: its reduce-scatter workspace is its own (the first
        # heap's workspaces went away with it)
        iris = iris_py.Iris(heap_size_mb=192)
        view = iris.get_device_view()
        out = torch.as_tensor(iris.empty([M // world, N]), device="cuda").view(torch.bfloat16)
        out.fill_(float("nan"))
        iris.barrier()
        tk_kernel.gemm_rs(dA, dB, out, view)
        torch.cuda.synchronize()
        res["gemm_rs_second_heap"] = orc.rel_fro(out.float().cpu(), want)
        res["status2"] = tk_kernel.device_status()
        iris.barrier()
        q.put((rank, res))
        del out, view
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
        assert all(e <= 1e-2 for e in results[r]["ag_gemm"]), results[r]["ag_gemm"]
        assert results[r]["moe_idx_ok"]
        assert all(e <= 2e-2 for e in results[r]["moe_ep"]), results[r]["moe_ep"]
        assert all(e <= 2e-2 for e in results[r]["moe_layer"]), results[r]["moe_layer"]
        assert results[r]["moe_layer_counts_ok"]
        assert results[r]["gemm_rs_second_heap"] <= 1e-2 and results[r]["status2"][0] == 0
        for algo in (0, 1, -1):
            assert results[r][f"allreduce{algo}"] <= 1e-2
            # every rank holds the same bits
            assert results[r][f"allreduce{algo}_sum"] == results[0][f"allreduce{algo}_sum"]


def _nvls_worker(rank, world, job, q):
    """NVLS all-reduce (multimem.ld_reduce + multimem.st through the NVSwitch). The heap leaves
    through its destructor on every path, so the multicast binding is always undone in order."""
    iris = None
    res = {}
    try:
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), DK_JOB_ID=job)
        sys.path.insert(0, str(ROOT))
        sys.path.insert(0, str(ROOT / "distributed-hipkittens_b200"))
        import iris_py
        import tk_kernel
        from oracle import dk_oracle as orc
        torch.cuda.set_device(rank)
        iris = iris_py.Iris(heap_size_mb=96)
        res["nvls"] = bool(iris.enable_multicast())
        if res["nvls"]:
            view = iris.get_device_view()
            for name, shape in (("small", (64, 8192)), ("large", (2048, 8192))):
                xs = orc.make_allreduce_inputs(shape, world)
                ref = orc.allreduce_ref(xs)
                x = torch.as_tensor(iris.empty(list(shape)), device="cuda").view(torch.bfloat16)
                o = torch.as_tensor(iris.empty(list(shape)), device="cuda").view(torch.bfloat16)
                for it, algo in enumerate((2, 2, -1)):
                    x.copy_(xs[rank])
                    o.fill_(float("nan"))
                    iris.barrier()
                    tk_kernel.allreduce(x, o, view, algo)
                    torch.cuda.synchronize()
                    res[f"{name}{it}"] = orc.rel_fro(o.float().cpu(), ref)
                    res[f"{name}{it}_sum"] = int(o.view(torch.int16).to(torch.int64).sum().item())
                # in place
                x.copy_(xs[rank])
                iris.barrier()
                tk_kernel.allreduce(x, x, view, 2)
                torch.cuda.synchronize()
                res[f"{name}_inplace"] = orc.rel_fro(x.float().cpu(), ref)
                del x, o
            res["status"] = tk_kernel.device_status()
            del view
        iris.barrier()
    except Exception:
        import traceback
        res["error"] = traceback.format_exc()
    finally:
        q.put((rank, res))
        del iris


@pytest.mark.parametrize("world", [2, 4, 8])
def test_nvls_allreduce(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    job = f"pytestnvls{os.getpid()}w{world}"
    ps = [ctx.Process(target=_nvls_worker, args=(r, world, job, q)) for r in range(world)]
    for p in ps:
        p.start()
    results = dict(q.get(timeout=240) for _ in ps)
    for p in ps:
        p.join(60)
    for r in range(world):
        assert "error" not in results[r], results[r].get("error")
    if not results[0]["nvls"]:
        assert not any(results[r]["nvls"] for r in range(world))   # the ranks agree
        pytest.skip("no NVLink multicast support on this system")
    for r in range(world):
        assert results[r]["status"][0] == 0
        for name in ("small", "large"):
            for it in range(3):
                assert results[r][f"{name}{it}"] <= 1e-2
                assert results[r][f"{name}{it}_sum"] == results[0][f"{name}{it}_sum"]
            assert results[r][f"{name}_inplace"] <= 1e-2
