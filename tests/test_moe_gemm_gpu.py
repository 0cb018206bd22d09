"""fp8 grouped GEMM (128x128 block scales) and the fused FFN against the oracle's block-dequantised
fp32 reference. Tolerance: relative Frobenius error <= 2e-2."""
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 2e-2


def _case(orc, T, H, F, E, k, seed=0, zipf=0.0):
    x, logits, w13q, w13s, w2q, w2s = orc.make_moe_inputs(T, H, F, E, k, seed=seed, zipf_s=zipf)
    idx, w = orc.moe_route(logits, k)
    rop, por, offs, counts = orc.moe_permute(idx, E)
    xq, xs = orc.quant_block128(orc.moe_gather_rows(x, por, k))
    return dict(x=x, idx=idx, w=w, rop=rop, por=por, offs=offs, xq=xq, xs=xs, w13q=w13q, w13s=w13s,
                w2q=w2q, w2s=w2s)


@pytest.mark.parametrize("T,H,F,E,k", [(64, 128, 128, 1, 1), (256, 256, 256, 4, 2), (512, 512, 384, 8, 2),
                                       (300, 1024, 256, 16, 4)])
def test_plain_grouped_gemm(capi, orc, T, H, F, E, k):
    c = _case(orc, T, H, F, E, k)
    # X [R,H] times W2-shaped weights is not meaningful; use the down weights on a fresh fp8 input
    R = c["xq"].shape[0]
    g = torch.Generator().manual_seed(9)
    hq, hs = orc.quant_block128(torch.randn(R, F, generator=g))
    want = orc.grouped_gemm_ref(hq, hs, c["w2q"], c["w2s"], c["offs"])
    if H % 256 != 0:
        pytest.skip("plain mode needs N % 256 == 0")
    y = capi.moe_grouped_gemm_fp8(hq.cuda(), hs.cuda(), c["w2q"].cuda(), c["w2s"].cuda(), c["offs"].cuda(), False)
    torch.cuda.synchronize()
    assert capi.device_status()[0] == 0
    valid = c["por"] >= 0
    assert orc.rel_fro(y.float().cpu()[valid], want[valid]) <= TOL
    assert orc.rel_fro(y.float().cpu(), want) <= TOL


@pytest.mark.parametrize("T,H,F,E,k", [(64, 128, 128, 1, 1), (256, 256, 256, 4, 2), (512, 512, 384, 8, 2),
                                       (300, 1024, 256, 16, 4), (1024, 256, 512, 64, 8)])
def test_gated_grouped_gemm_and_ffn(capi, orc, T, H, F, E, k):
    c = _case(orc, T, H, F, E, k, zipf=1.1 if E >= 16 else 0.0)
    want_y, want_hq, want_hs = orc.moe_ffn_ref(c["xq"], c["xs"], c["w13q"], c["w13s"], c["w2q"], c["w2s"], c["offs"])
    d = {n: c[n].cuda() for n in ("xq", "xs", "w13q", "w13s", "w2q", "w2s", "offs")}
    hq, hs = capi.moe_grouped_gemm_fp8(d["xq"], d["xs"], d["w13q"], d["w13s"], d["offs"], True)
    torch.cuda.synchronize()
    assert capi.device_status()[0] == 0
    got_h = orc.dequant_block128(hq.cpu(), hs.cpu())
    ref_h = orc.dequant_block128(want_hq, want_hs)
    assert orc.rel_fro(got_h, ref_h) <= TOL
    # scales agree closely (they come from fp32 maxima of nearly identical values)
    Rb = int(c["offs"][-1]) // 128
    assert torch.allclose(hs.cpu()[:Rb], want_hs[:Rb], rtol=1e-3)
    if H % 256 == 0:
        y = capi.moe_ffn_fp8(d["xq"], d["xs"], d["w13q"], d["w13s"], d["w2q"], d["w2s"], d["offs"])
        torch.cuda.synchronize()
        assert capi.device_status()[0] == 0
        assert orc.rel_fro(y.float().cpu(), want_y) <= TOL
        # through combine: the full single-GPU MoE layer
        out = capi.moe_combine(y, c["rop"].cuda(), c["w"].cuda())
        want_out = orc.moe_combine_ref(want_y, c["rop"], c["w"])
        assert orc.rel_fro(out.float().cpu(), want_out) <= TOL


def test_ffn_with_banded_tile_walk(capi, orc):
    """Experts with more row tiles than a band holds (the band shrunk to three row tiles; bands of
    3, 3 and a rest): the tile order changes, the result does not."""
    T, H, F, E, k = 2048, 256, 256, 4, 2
    c = _case(orc, T, H, F, E, k, zipf=1.1)
    assert int((c["offs"][1:] - c["offs"][:-1]).max()) // 128 > 3
    want_y = orc.moe_ffn_ref(c["xq"], c["xs"], c["w13q"], c["w13s"], c["w2q"], c["w2s"], c["offs"])[0]
    d = {n: c[n].cuda() for n in ("xq", "xs", "w13q", "w13s", "w2q", "w2s", "offs")}
    capi.check(capi.lib().dk_set_walk_band_bytes(3 * 128 * H))
    try:
        y = capi.moe_ffn_fp8(d["xq"], d["xs"], d["w13q"], d["w13s"], d["w2q"], d["w2s"], d["offs"])
        torch.cuda.synchronize()
    finally:
        capi.check(capi.lib().dk_set_walk_band_bytes(32 << 20))
    assert capi.device_status()[0] == 0
    assert orc.rel_fro(y.float().cpu(), want_y) <= TOL


def test_grouped_gemm_empty_experts_and_errors(capi, orc):
    T, H, F, E, k = 128, 256, 128, 8, 1
    c = _case(orc, T, H, F, E, k)
    # route everything to expert 3
    idx = torch.full((T, 1), 3, dtype=torch.int32)
    rop, por, offs, counts = orc.moe_permute(idx, E)
    xq, xs = orc.quant_block128(orc.moe_gather_rows(c["x"], por, k))
    want_y, _, _ = orc.moe_ffn_ref(xq, xs, c["w13q"], c["w13s"], c["w2q"], c["w2s"], offs)
    y = capi.moe_ffn_fp8(xq.cuda(), xs.cuda(), c["w13q"].cuda(), c["w13s"].cuda(), c["w2q"].cuda(),
                         c["w2s"].cuda(), offs.cuda())
    torch.cuda.synchronize()
    assert orc.rel_fro(y.float().cpu(), want_y) <= TOL
    with pytest.raises(capi.DkError):
        capi.moe_grouped_gemm_fp8(xq.cuda()[:, :64].contiguous(), xs.cuda(), c["w13q"].cuda(), c["w13s"].cuda(),
                                  offs.cuda(), True)      # K % 128 != 0


def test_tk_kernel_moe_layer_single_gpu(orc):
    """The whole MoE layer through the Python entry points of tk_kernel on one GPU."""
    import iris_py
    import tk_kernel
    T, H, F, E, k = 384, 256, 256, 8, 2
    x, logits, w13q, w13s, w2q, w2s = orc.make_moe_inputs(T, H, F, E, k, seed=8)
    idx_c, w_c = orc.moe_route(logits, k)
    rop_c, por_c, offs_c, _ = orc.moe_permute(idx_c, E)
    xq_c, xs_c = orc.quant_block128(orc.moe_gather_rows(x, por_c, k))
    y_c, _, _ = orc.moe_ffn_ref(xq_c, xs_c, w13q, w13s, w2q, w2s, offs_c)
    want = orc.moe_combine_ref(y_c, rop_c, w_c)

    iris = iris_py.Iris(heap_size_mb=64)
    view = iris.get_device_view()
    idx, w = tk_kernel.moe_route(logits.cuda(), k)
    rop, por, offs, counts = tk_kernel.moe_permute(idx, E)
    assert torch.equal(idx.cpu(), idx_c) and torch.equal(rop.cpu(), rop_c) and torch.equal(offs.cpu(), offs_c)
    R = int(offs_c[-1])
    assert torch.equal(por.cpu()[:R], por_c)
    xq, xs = tk_kernel.moe_quant(x.cuda(), por, 1, k)
    assert torch.equal(xq.cpu()[:R], xq_c) and torch.equal(xs.cpu()[:R // 128], xs_c)
    y = tk_kernel.moe_ffn_fp8(xq, xs, w13q.cuda(), w13s.cuda(), w2q.cuda(), w2s.cuda(), offs)
    out = tk_kernel.moe_combine(y, idx, rop, w, E, view)
    torch.cuda.synchronize()
    assert tk_kernel.device_status()[0] == 0
    assert orc.rel_fro(out.float().cpu(), want) <= TOL
