"""Expert-parallel MoE layer with all ranks on one GPU: every rank's heap is a region of one
buffer; dispatch pushes into the destination rank's receive rows, each rank runs its experts,
combine pulls from the ranks that computed them. Ordering comes from stream order here (sync=0);
the barrier-bracketed form runs in tests/test_multigpu_gpu.py on real peers. Row maps bit-exact,
values within 2e-2 of the oracle's single-rank result (the per-expert 128-row blocks are the same
rows in both layouts, so quantisation is identical)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.mark.parametrize("P,T,H,F,E,k,zipf", [(2, 256, 256, 128, 4, 2, 0.0), (4, 512, 512, 256, 16, 4, 1.1),
                                              (8, 512, 256, 128, 32, 8, 1.1)])
def test_ep_layer_all_ranks_on_one_gpu(capi, orc, P, T, H, F, E, k, zipf):
    x, logits, w13q, w13s, w2q, w2s = orc.make_moe_inputs(T, H, F, E, k, seed=3, zipf_s=zipf)
    epr, Tl = E // P, T // P
    # ---- oracle, single rank
    idx_c, w_c = orc.moe_route(logits, k)
    rop_c, por_c, offs_c, _ = orc.moe_permute(idx_c, E)
    xq_c, xs_c = orc.quant_block128(orc.moe_gather_rows(x, por_c, k))
    y_c, _, _ = orc.moe_ffn_ref(xq_c, xs_c, w13q, w13s, w2q, w2s, offs_c)
    want = orc.moe_combine_ref(y_c, rop_c, w_c)

    # ---- device: route + segmented permutation of the global routing table
    idx, w = capi.moe_route(logits.cuda(), k)
    assert torch.equal(idx.cpu(), idx_c)
    rop, por, offs, counts = capi.moe_permute(idx, E, 128, experts_per_segment=epr)
    recv_pair, recv_offs, rop_ref, _ = orc.ep_layout(idx_c, E, P)
    assert torch.equal(rop.cpu(), rop_ref)
    cap = por.shape[1]

    row_bytes = cap * H * 2
    region = capi.CTRL_BYTES + 2 * ((row_bytes + 4095) // 4096 * 4096)
    buf = torch.zeros(P * region + 4096, dtype=torch.uint8, device="cuda")
    base0 = (buf.data_ptr() + 1023) // 1024 * 1024
    bases = [base0 + r * region for r in range(P)]
    views = [capi.make_view(r, P, bases, region) for r in range(P)]
    off_y = capi.CTRL_BYTES + (row_bytes + 4095) // 4096 * 4096
    xrecv = [capi.tensor_from_ptr(b + capi.CTRL_BYTES, (cap, H), torch.bfloat16) for b in bases]
    ybuf = [capi.tensor_from_ptr(b + off_y, (cap, H), torch.bfloat16) for b in bases]
    for t in xrecv:
        t.fill_(55.0)          # garbage in the padding rows must not matter

    dx = x.cuda()
    for r in range(P):
        sl = slice(r * Tl, (r + 1) * Tl)
        capi.moe_dispatch(dx[sl].contiguous(), idx[sl].contiguous(), rop[sl].contiguous(), epr, xrecv[r],
                          views[r], sync=False)
    for d in range(P):
        R = int(recv_offs[d][-1])
        valid = recv_pair[d] >= 0
        got_rows = xrecv[d].cpu()[:R][valid]
        want_rows = x[(recv_pair[d][valid].long() // k)]
        assert torch.equal(got_rows.view(torch.int16), want_rows.view(torch.int16))    # bit-exact move
        xq, xs = capi.quant_block128(xrecv[d], row_map=por[d].contiguous(), map_mode=2)
        es = slice(d * epr, (d + 1) * epr)
        y = capi.moe_ffn_fp8(xq, xs, w13q[es].cuda(), w13s[es].cuda(), w2q[es].cuda(), w2s[es].cuda(),
                             offs[d].contiguous())
        ybuf[d].copy_(y)
    outs = []
    for r in range(P):
        sl = slice(r * Tl, (r + 1) * Tl)
        outs.append(capi.moe_combine_ep(ybuf[r], idx[sl].contiguous(), rop[sl].contiguous(),
                                        w[sl].contiguous(), epr, views[r], sync=False))
    torch.cuda.synchronize()
    assert capi.device_status()[0] == 0
    got = torch.cat(outs, 0).float().cpu()
    assert orc.rel_fro(got, want) <= TOL


def test_peer_wait_runs_out_and_is_reported(capi):
    """Failure detection on the device without faulting it: a barrier with a peer that never
    signals (a flag nothing sets) gives up after the configured limit, records where, and returns;
    the context stays usable."""
    import ctypes as C
    region = capi.CTRL_BYTES + 4096
    buf = torch.zeros(2 * region + 4096, dtype=torch.uint8, device="cuda")
    base0 = (buf.data_ptr() + 1023) // 1024 * 1024
    views = [capi.make_view(r, 2, [base0, base0 + region], region) for r in range(2)]
    L = capi.lib()
    capi.device_status()
    capi.check(L.dk_set_peer_wait_ms(200))
    try:
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        capi.check(L.dk_peer_barrier_epoch(C.byref(views[0]), 1, stream))    # rank 1 never arrives
        torch.cuda.synchronize()
        code, block, site, detail = capi.device_status()
        assert code == 2 and site == 48 and detail == 1
        # both ranks arrive (one after the other: the first leaves its flag, the second finds it)
        capi.check(L.dk_peer_barrier_epoch(C.byref(views[1]), 1, stream))
        torch.cuda.synchronize()
        assert capi.device_status()[0] == 0
    finally:
        capi.check(L.dk_set_peer_wait_ms(20000))
    a = torch.ones(128, 64, dtype=torch.bfloat16, device="cuda")
    c = capi.gemm_bf16(a, a)
    torch.cuda.synchronize()
    assert float(c[0, 0]) == 64.0
