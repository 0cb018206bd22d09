"""dk_moe_ep_layer: the expert-parallel fp8 MoE layer as one call, with all ranks of a job on ONE
GPU. Every rank's heap is a region of one buffer; the layer is run phase by phase over the ranks
(routing + exchange, permutation + dispatch, experts + combine push, final sum), so that no launch
waits for a later one. The multi-process form over real peer memory is in tests/test_multigpu_gpu.py.

Checked against the oracle's single-rank layer (the per-expert 128-row blocks hold the same rows in
both layouts, so the quantisation is the same): per-expert pair counts bit-exact, output within 2e-2
relative Frobenius error. With the fp8 dispatch (scale_mode 2) the oracle quantises every token per
1x128 group before the experts see it. Two calls in a row with different tokens on the same workspace, whose
bytes are poisoned before the first call: nothing may depend on its old contents."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 2e-2


def _inputs(orc, T, H, F, E, k, zipf, seed, pow2):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    if zipf > 0:
        pi = torch.randperm(E, generator=torch.Generator().manual_seed(1)).float()
        p = (pi + 1.0) ** (-zipf)
        logits = logits + torch.log(p / p.sum())[None, :]
    gw = torch.Generator().manual_seed(99)          # the same weights for every call
    quant = orc.quant_block128_pow2 if pow2 else orc.quant_block128
    w13 = [quant((torch.randn(2 * F, H, generator=gw) / math.sqrt(H)).to(torch.bfloat16)) for _ in range(E)]
    w2 = [quant((torch.randn(H, F, generator=gw) / math.sqrt(F)).to(torch.bfloat16)) for _ in range(E)]
    st = lambda parts, i: torch.stack([p[i] for p in parts])
    return x, logits.contiguous(), [st(w13, i) for i in range(len(w13[0]))], [st(w2, i) for i in range(len(w2[0]))]


def _oracle(orc, x, logits, w13, w2, E, k, pow2, fp8_dispatch=False):
    idx, w = orc.moe_route(logits, k)
    rop, por, offs, counts = orc.moe_permute(idx, E)
    rows = orc.moe_gather_rows(x, por, k)
    if fp8_dispatch:          # tokens quantised per 1x128 group where they live; rows carry their own scales
        xq, xs, _ = orc.quant_rows128_pow2(rows)
        y = orc.moe_ffn_rows_pow2_ref(xq, xs, w13[0], w13[1], w2[0], w2[1], offs)[0]
    elif pow2:
        xq, xs, _ = orc.quant_block128_pow2(rows)
        y = orc.moe_ffn_pow2_ref(xq, xs, w13[0], w13[1], w2[0], w2[1], offs)[0]
    else:
        xq, xs = orc.quant_block128(rows)
        y = orc.moe_ffn_ref(xq, xs, w13[0], w13[1], w2[0], w2[1], offs)[0]
    return orc.moe_combine_ref(y, rop, w), counts


@pytest.mark.parametrize("mode", [0, 1, 2], ids=["fp32_scales", "pow2_scales", "pow2_scales_fp8_dispatch"])
@pytest.mark.parametrize("P,T,H,F,E,k,zipf", [(1, 256, 256, 128, 4, 2, 0.0), (2, 256, 256, 128, 4, 2, 0.0),
                                              (2, 384, 256, 256, 16, 8, 1.1), (4, 512, 512, 256, 16, 4, 1.1),
                                              (8, 1024, 256, 128, 32, 8, 1.1), (8, 512, 256, 128, 8, 2, 0.0),
                                              (8, 2048, 256, 128, 256, 8, 1.1)])   # 32 experts per rank, some empty
def test_ep_layer_call_all_ranks_on_one_gpu(capi, orc, P, T, H, F, E, k, zipf, mode):
    _run_layer(capi, orc, P, T, H, F, E, k, zipf, mode, epochs=(1, 2))


DEVICE = 0xFFFFFFFF      # DK_EPOCH_DEVICE: the call number lives in device memory


@pytest.mark.parametrize("mode", [0, 2], ids=["fp32_scales", "pow2_scales_fp8_dispatch"])
def test_ep_layer_device_numbered_calls(capi, orc, mode):
    """Calls numbered on the device (what makes the layer replayable from a CUDA graph), mixed with a
    host-numbered call on the same heap regions: each kind has its own flags and counter."""
    _run_layer(capi, orc, 4, 512, 256, 128, 16, 4, 1.1, mode, epochs=(DEVICE, DEVICE, 1, DEVICE))


def _run_layer(capi, orc, P, T, H, F, E, k, zipf, mode, epochs):
    pow2 = mode != 0
    epr, Tl = E // P, T // P
    ws_bytes = capi.moe_ep_workspace_bytes(Tl, k, E, H, F, P)
    assert ws_bytes > 0
    region = capi.CTRL_BYTES + (ws_bytes + 4095) // 4096 * 4096
    buf = torch.zeros(P * region + 4096, dtype=torch.uint8, device="cuda")
    base0 = (buf.data_ptr() + 1023) // 1024 * 1024
    bases = [base0 + r * region for r in range(P)]
    views = [capi.make_view(r, P, bases, region) for r in range(P)]
    ws = [b + capi.CTRL_BYTES for b in bases]
    for r in range(P):      # the workspace needs no initialisation: poison it (the flags stay zero)
        capi.tensor_from_ptr(ws[r], (ws_bytes,), torch.uint8).fill_(0xFF)
    capi.device_status()
    for call, epoch in enumerate(epochs, 1):
        x, logits, w13, w2 = _inputs(orc, T, H, F, E, k, zipf, seed=20 + call, pow2=pow2)
        want, want_counts = _oracle(orc, x, logits, w13, w2, E, k, pow2, fp8_dispatch=mode == 2)
        dev = []
        for r in range(P):
            es, sl = slice(r * epr, (r + 1) * epr), slice(r * Tl, (r + 1) * Tl)
            if pow2:
                s13 = orc.block128_scales_to_block_atoms(w13[2][es].reshape(-1, w13[2].shape[-1])).cuda()
                s2 = orc.block128_scales_to_block_atoms(w2[2][es].reshape(-1, w2[2].shape[-1])).cuda()
            else:
                s13, s2 = w13[1][es].contiguous().cuda(), w2[1][es].contiguous().cuda()
            dev.append(dict(x=x[sl].contiguous().cuda(), logits=logits[sl].contiguous().cuda(),
                            w13q=w13[0][es].contiguous().cuda(), w13s=s13, w2q=w2[0][es].contiguous().cuda(), w2s=s2,
                            out=torch.full((Tl, H), float("nan"), dtype=torch.bfloat16, device="cuda"),
                            counts=torch.full((epr,), -1, dtype=torch.int32, device="cuda")))
        for phase in (1, 2, 4, 8):
            for r in range(P):
                d = dev[r]
                capi.moe_ep_layer(d["x"], d["logits"], d["w13q"], d["w13s"], d["w2q"], d["w2s"], d["out"], ws[r],
                                  views[r] if P > 1 else None, k, scale_mode=mode, epoch=epoch,
                                  phases=phase, counts_out=d["counts"])
            torch.cuda.synchronize()
        assert capi.device_status()[0] == 0
        counts = torch.cat([d["counts"].cpu() for d in dev])
        assert torch.equal(counts, want_counts)                    # bit-exact
        got = torch.cat([d["out"].float().cpu() for d in dev], 0)
        assert not torch.isnan(got).any()
        assert orc.rel_fro(got, want) <= TOL
        # every rank's tokens by themselves (one rank's error must not hide in the global norm)
        for r in range(P):
            sl = slice(r * Tl, (r + 1) * Tl)
            assert orc.rel_fro(got[sl], want[sl]) <= TOL


def test_ep_layer_python_entry_point_one_rank(orc):
    """tk_kernel.moe_layer_ep on one rank, workspace from the symmetric heap."""
    import iris_py
    import tk_kernel
    T, H, F, E, k = 256, 256, 128, 8, 2
    x, logits, w13, w2 = _inputs(orc, T, H, F, E, k, 0.0, seed=5, pow2=False)
    want, want_counts = _oracle(orc, x, logits, w13, w2, E, k, False)
    nbytes = tk_kernel.moe_ep_workspace_bytes(T, k, E, H, F, 1)
    iris = iris_py.Iris(heap_size_mb=nbytes // (1 << 20) + 64)
    ws = torch.as_tensor(iris.empty([nbytes], "uint8"), device="cuda")
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    counts = torch.empty(E, dtype=torch.int32, device="cuda")
    tk_kernel.moe_layer_ep(x.cuda(), logits.cuda(), k, w13[0].cuda(), w13[1].cuda(), w2[0].cuda(), w2[1].cuda(), out, ws,
                           iris.get_device_view(), 0, counts)
    torch.cuda.synchronize()
    assert tk_kernel.device_status()[0] == 0
    assert torch.equal(counts.cpu(), want_counts)
    assert orc.rel_fro(out.float().cpu(), want) <= TOL


@pytest.mark.parametrize("mode", [1, 2], ids=["pow2_scales", "pow2_scales_fp8_dispatch"])
def test_ep_layer_replayed_from_a_cuda_graph(orc, mode):
    """The whole layer (route .. final sum, 12 launches) captured once into a CUDA graph after one
    eager call and replayed on new tokens written into the captured buffers. One rank; the ranks of
    a real job do the same with device-numbered calls (tests/test_multigpu_gpu.py)."""
    import tk_kernel
    T, H, F, E, k = 512, 256, 256, 8, 2
    nbytes = tk_kernel.moe_ep_workspace_bytes(T, k, E, H, F, 1)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    xs = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")
    ls = torch.zeros(T, E, dtype=torch.float32, device="cuda")
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    counts = torch.empty(E, dtype=torch.int32, device="cuda")
    x, logits, w13, w2 = _inputs(orc, T, H, F, E, k, 1.1, seed=40, pow2=True)
    dw = [w13[0].cuda(), orc.block128_scales_to_block_atoms(w13[2].reshape(-1, w13[2].shape[-1])).cuda(),
          w2[0].cuda(), orc.block128_scales_to_block_atoms(w2[2].reshape(-1, w2[2].shape[-1])).cuda()]
    call = lambda: tk_kernel.moe_layer_ep(xs, ls, k, dw[0], dw[1], dw[2], dw[3], out, ws, None, mode, counts, True)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        call()                       # eager once: everything the library sets up lazily exists afterwards
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        call()
    for seed in (41, 42, 43):
        x, logits, _, _ = _inputs(orc, T, H, F, E, k, 1.1, seed=seed, pow2=True)
        want, want_counts = _oracle(orc, x, logits, w13, w2, E, k, True, fp8_dispatch=mode == 2)
        xs.copy_(x)
        ls.copy_(logits)
        out.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert tk_kernel.device_status()[0] == 0
        assert torch.equal(counts.cpu(), want_counts)
        assert orc.rel_fro(out.float().cpu(), want) <= TOL
