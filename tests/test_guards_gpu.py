"""Indices that come from device memory are not trusted: a kernel that meets one pointing outside
its buffers skips the access and leaves a record (code 3, site, detail) instead of writing out of
bounds. And while any record is unread, collective entry points refuse to launch. Nothing here
faults the GPU: the guarded path is the one that runs, and guard words around the buffers show it."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
GUARD = 0x5A


def _guarded(n, dtype):
    """n elements with 256 guard elements on either side, all set to the guard pattern."""
    whole = torch.full((n + 512,), GUARD, dtype=dtype, device="cuda")
    return whole, whole[256:256 + n]


def _intact(whole, n):
    return bool((whole[:256] == GUARD).all() and (whole[256 + n:] == GUARD).all())


def _permute(capi, idx, E, cap, pad=128):
    T, k = idx.shape
    L = capi.lib()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rop_w, rop = _guarded(T * k, torch.int32)
    por_w, por = _guarded(cap, torch.int32)
    offs = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    counts = torch.empty(E, dtype=torch.int32, device="cuda")
    sb = L.dk_moe_permute_scratch_bytes(T, k, E)
    scratch = torch.empty(sb, dtype=torch.uint8, device="cuda")
    P = lambda t: C.c_void_p(t.data_ptr())
    capi.check(L.dk_moe_permute(P(idx), T, k, E, pad, E, P(rop), P(por), cap, P(offs), P(counts), P(scratch), sb, st))
    torch.cuda.synchronize()
    return (rop_w, rop), (por_w, por), offs, counts


def test_expert_id_outside_range_is_skipped_and_recorded(capi, orc):
    capi.device_status()
    g = torch.Generator().manual_seed(0)
    T, E, k = 300, 8, 2
    idx = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32)
    idx[17, 1] = -1          # a dropped token
    idx[200, 0] = E          # an id past the last expert
    cap = capi.lib().dk_moe_rows_capacity(T, k, E, 128)
    (rop_w, rop), (por_w, por), offs, counts = _permute(capi, idx.cuda(), E, cap)
    code, _, site, detail = capi.device_status()
    assert code == 3 and site == 80 and detail in (17 * k + 1, 200 * k)
    assert _intact(rop_w, T * k) and _intact(por_w, cap)
    rop = rop.cpu().reshape(T, k)
    assert rop[17, 1] == -1 and rop[200, 0] == -1
    # every other pair sits where the oracle puts it once the two bad pairs are taken out
    keep = torch.ones(T * k, dtype=torch.bool)
    keep[17 * k + 1] = keep[200 * k] = False
    flat = idx.reshape(-1)[keep].reshape(-1, 1)
    want_rop, _, want_offs, want_counts = orc.moe_permute(flat, E)
    assert torch.equal(rop.reshape(-1)[keep], want_rop.reshape(-1))
    assert torch.equal(offs.cpu(), want_offs) and torch.equal(counts.cpu(), want_counts)
    # combine treats a pair without a row as absent
    y = torch.randn(cap, 64, generator=g).to(torch.bfloat16)
    w = torch.rand(T, k, generator=g)
    out = capi.moe_combine(y.cuda(), rop.cuda(), w.cuda())
    torch.cuda.synchronize()
    w0 = w.clone()
    w0[rop < 0] = 0
    want = orc.moe_combine_ref(y.float(), rop.clamp(min=0), w0)
    assert orc.rel_fro(out.float().cpu(), want) <= 1e-2


def test_undersized_capacity_is_skipped_and_recorded(capi):
    capi.device_status()
    T, E, k = 512, 4, 2
    idx = (torch.arange(T * k, dtype=torch.int32) % E).reshape(T, k)
    cap = 512                 # 1024 pairs need 1024 rows
    (rop_w, rop), (por_w, por), offs, counts = _permute(capi, idx.cuda(), E, cap)
    code, _, site, _ = capi.device_status()
    assert code == 3 and site == 81
    assert _intact(rop_w, T * k) and _intact(por_w, cap)
    rop = rop.cpu()
    assert int((rop >= cap).sum()) == 0 and int((rop < 0).sum()) == T * k - cap


@pytest.mark.parametrize("path", ["fp32_scales", "pow2_scales"])
def test_offsets_beyond_the_output_are_skipped_and_recorded(capi, path):
    capi.device_status()
    R, H, F, E = 256, 256, 128, 2
    offs = torch.tensor([0, 128, 384], dtype=torch.int32).cuda()    # expert 1 claims rows up to 384 > R
    xq = torch.full((R, H), 0x38, dtype=torch.uint8, device="cuda")
    wq = torch.full((E, 2 * F, H), 0x38, dtype=torch.uint8, device="cuda")
    L = capi.lib()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    P = lambda t: C.c_void_p(t.data_ptr())
    out_w, out = _guarded(R * F, torch.uint8)
    if path == "fp32_scales":
        xs = torch.ones(R // 128, H // 128, device="cuda")
        ws = torch.ones(E, 2 * F // 128, H // 128, device="cuda")
        hs = torch.ones(R // 128, F // 128, device="cuda")
        capi.check(L.dk_moe_grouped_gemm_fp8(P(xq), P(xs), P(wq), P(ws), P(offs), E, R, F, H, 1, P(out), P(hs), st))
        site = 37
    else:
        xa = torch.full((R // 128, 1, 512), 127, dtype=torch.uint8, device="cuda")
        wa = torch.full((E * 2 * F // 128, 1, 512), 127, dtype=torch.uint8, device="cuda")
        he = torch.empty(R // 128, F // 128, dtype=torch.uint8, device="cuda")
        ha = torch.empty(R // 128, 1, 512, dtype=torch.uint8, device="cuda")
        capi.check(L.dk_moe_grouped_gemm_mxfp8(P(xq), P(xa), P(wq), P(wa), P(offs), E, R, F, H, 1, P(out), P(he),
                                               P(ha), st))
        site = 69
    torch.cuda.synchronize()
    code, _, got_site, detail = capi.device_status()
    assert code == 3 and got_site == site and detail == 1
    assert _intact(out_w, R * F)
    out = out.reshape(R, F)
    assert bool((out[:128] != GUARD).any())        # expert 0 was computed
    assert bool((out[128:] == GUARD).all())        # expert 1 was left alone


def test_collectives_refuse_to_launch_while_a_record_is_unread(capi):
    """After a peer wait has run out the ranks are out of step: the next collective returns
    DK_ERR_DEVICE (and launches nothing) until the host has read the record."""
    region = capi.CTRL_BYTES + (1 << 20)
    buf = torch.zeros(2 * region + 4096, dtype=torch.uint8, device="cuda")
    base0 = (buf.data_ptr() + 1023) // 1024 * 1024
    views = [capi.make_view(r, 2, [base0, base0 + region], region) for r in range(2)]
    L = capi.lib()
    capi.device_status()
    capi.check(L.dk_set_peer_wait_ms(200))
    try:
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        capi.check(L.dk_peer_barrier_epoch(C.byref(views[0]), 1, st))      # rank 1 never arrives
        torch.cuda.synchronize()
        # unread: a barrier and a reduce-scatter phase are both refused, the record stays
        assert L.dk_peer_barrier_epoch(C.byref(views[0]), 2, st) == capi.ERR_DEVICE
        assert b"has not been read" in L.dk_last_error_string()
        a = torch.zeros(256, 64, dtype=torch.bfloat16, device="cuda")
        o = torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda")
        with pytest.raises(capi.DkError) as e:
            capi.gemm_rs_phase(a, a, o, base0 + capi.CTRL_BYTES, views[0], 1, 1)
        assert e.value.code == capi.ERR_DEVICE
        code, _, site, detail = capi.device_status()                       # read: clears
        assert code == 2 and site == 48 and detail == 1
        # read: both ranks' barriers launch again
        capi.check(L.dk_peer_barrier_epoch(C.byref(views[1]), 1, st))
        capi.check(L.dk_peer_barrier_epoch(C.byref(views[0]), 1, st))
        torch.cuda.synchronize()
        assert capi.device_status()[0] == 0
    finally:
        capi.check(L.dk_set_peer_wait_ms(20000))
