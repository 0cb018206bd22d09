"""The oracle against the golden vectors and against itself (CPU only)."""
from pathlib import Path

import numpy as np
import torch

GOLD = Path(__file__).resolve().parent / "golden"


def _bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def test_example_inputs_match_golden(orc):
    fx = np.load(GOLD / "gemm_example.npz")
    for rank in (0, 1):
        A, B = orc.example_inputs(128, 256, 128, rank=rank)
        assert torch.equal(A, _bf16(fx[f"A{rank}"]))
        assert torch.equal(B, _bf16(fx["B"]))
        C_ref = _bf16(fx[f"C{rank}"])
        # the oracle's fp32 product passes the example's own acceptance test on the golden output
        ok, err = orc.example_check(orc.gemm_ref(A, B).to(torch.bfloat16), A, B)
        assert ok and err < 0.02
        assert orc.rel_fro(C_ref.float(), orc.gemm_ref(A, B)) < 1e-2


def test_sharded_equals_unsharded(orc):
    A, Bt = orc.make_gemm_inputs(256, 128, 512, seed=3)
    full = orc.gemm_ref(A, Bt)
    for world in (1, 2, 4, 8):
        As, Bs = orc.shard_k(A, Bt, world)
        outs = orc.gemm_rs_ref(As, Bs)
        got = torch.cat(outs, 0)
        assert orc.rel_fro(got, full) < 1e-6
        bf = torch.cat(orc.gemm_rs_bf16_partials_ref(As, Bs), 0)
        assert orc.rel_fro(bf, full) < 5e-3   # what bf16 partials cost


def test_allreduce_ref(orc):
    xs = orc.make_allreduce_inputs((16, 64), 4)
    s = orc.allreduce_ref(xs)
    assert torch.allclose(s, sum(x.double() for x in xs).float(), atol=1e-6)


def test_route_permute_golden(orc):
    fx = np.load(GOLD / "moe_small.npz")
    logits = torch.from_numpy(fx["logits"])
    idx, w = orc.moe_route(logits, 2)
    assert np.array_equal(idx.numpy(), fx["topk_idx"])
    assert np.allclose(w.numpy(), fx["topk_w"], rtol=1e-6)
    assert idx[3, 0].item() == 1 or idx[3, 1].item() == 1 or logits[3, 1] < logits[3].topk(2).values[1]
    rop, por, offs, counts = orc.moe_permute(idx, 8, 128)
    assert np.array_equal(rop.numpy(), fx["row_of_pair"])
    assert np.array_equal(por.numpy(), fx["pair_of_row"])
    assert np.array_equal(offs.numpy(), fx["offsets"])
    assert np.array_equal(counts.numpy(), fx["counts"])


def test_route_tie_break_lower_index(orc):
    logits = torch.zeros(4, 8)
    idx, w = orc.moe_route(logits, 3)
    assert idx.tolist() == [[0, 1, 2]] * 4
    assert torch.allclose(w, torch.full((4, 3), 1 / 3))


def test_permute_properties(orc):
    g = torch.Generator().manual_seed(0)
    T, E, k = 300, 16, 4
    idx, _ = orc.moe_route(torch.randn(T, E, generator=g), k)
    rop, por, offs, counts = orc.moe_permute(idx, E, 128)
    assert int(counts.sum()) == T * k
    assert all(int(o) % 128 == 0 for o in offs)
    # inverse maps
    flat = rop.reshape(-1).long()
    assert torch.equal(por[flat].long(), torch.arange(T * k))
    assert int((por >= 0).sum()) == T * k
    # rows of one expert are sorted by (token, slot)
    for e in range(E):
        rows = por[int(offs[e]):int(offs[e]) + int(counts[e])].long()
        assert torch.equal(rows, rows.sort().values)
        assert (idx.reshape(-1)[rows] == e).all()
    # empty input
    rop0, por0, offs0, c0 = orc.moe_permute(torch.zeros(0, k, dtype=torch.int32), E, 128)
    assert por0.numel() == 0 and int(offs0[-1]) == 0


def test_quant_golden_and_roundtrip(orc):
    fx = np.load(GOLD / "moe_small.npz")
    x = _bf16(fx["x"])
    q, s = orc.quant_block128(x)
    assert np.array_equal(q.numpy(), fx["q"])
    assert np.array_equal(s.numpy(), fx["s"])
    assert s[0, 0].item() == 1.0 and int(q[:128, :128].max()) == 0   # all-zero block
    back = orc.dequant_block128(q, s)
    assert orc.rel_fro(back, x.float()) < 0.04   # e4m3 has 3 mantissa bits
    # the block maximum maps to +-448 exactly
    blk = q[128:, 128:].view(torch.float8_e4m3fn).float().abs().max().item()
    assert blk == 448.0


def test_ffn_and_combine_shapes(orc):
    T, H, F, E, k = 64, 128, 128, 4, 2
    x, logits, w13q, w13s, w2q, w2s = orc.make_moe_inputs(T, H, F, E, k, seed=1)
    idx, w = orc.moe_route(logits, k)
    rop, por, offs, counts = orc.moe_permute(idx, E)
    xp = orc.moe_gather_rows(x, por, k)
    xq, xs = orc.quant_block128(xp)
    y, hq, hs = orc.moe_ffn_ref(xq, xs, w13q, w13s, w2q, w2s, offs)
    assert y.shape == (int(offs[-1]), H) and hq.shape == (int(offs[-1]), F)
    out = orc.moe_combine_ref(y, rop, w)
    assert out.shape == (T, H) and torch.isfinite(out).all()
    # padding rows stay zero through the FFN
    pad = por < 0
    assert float(y[pad].abs().max()) == 0.0 if pad.any() else True


def test_ep_layout_consistent_with_single_rank(orc):
    g = torch.Generator().manual_seed(2)
    T, E, k, P = 128, 16, 4, 4
    idx, _ = orc.moe_route(torch.randn(T, E, generator=g), k)
    recv_pair, recv_offs, rop, dest = orc.ep_layout(idx, E, P)
    assert sum(int((rp >= 0).sum()) for rp in recv_pair) == T * k
    for d in range(P):
        rp = recv_pair[d]
        valid = rp[rp >= 0].long()
        assert (dest.reshape(-1)[valid] == d).all()
        assert torch.equal(rop.reshape(-1)[valid].long(), (rp >= 0).nonzero().flatten())
    # with one rank the layout is moe_permute
    rp1, ro1, rop1, _ = orc.ep_layout(idx, E, 1)
    rop_s, por_s, offs_s, _ = orc.moe_permute(idx, E)
    assert torch.equal(rp1[0], por_s) and torch.equal(ro1[0], offs_s) and torch.equal(rop1, rop_s)


# ---- the plain-C restatement and the Python oracle pin each other ------------------------------
def _c_oracle():
    import ctypes as C
    import subprocess
    root = Path(__file__).resolve().parents[1] / "oracle"
    lib = root / "libdk_oracle_c.so"
    if not lib.exists():
        subprocess.run(["make", "-C", str(root), "-s"], check=True)
    return C.CDLL(str(lib))


def test_c_oracle_matches_python_oracle(orc):
    import ctypes as C
    L = _c_oracle()
    g = torch.Generator().manual_seed(21)
    T, E, k = 500, 64, 6
    logits = torch.randn(T, E, generator=g)
    logits[7] = 0.25                                   # all equal: lowest indices win
    logits[9, 3] = logits[9, 40] = 9.0                 # tie at the top
    idx_c = torch.empty(T, k, dtype=torch.int32)
    w_c = torch.empty(T, k)
    L.dk_c_route(C.c_void_p(logits.data_ptr()), T, E, k, C.c_void_p(idx_c.data_ptr()), C.c_void_p(w_c.data_ptr()))
    idx_p, w_p = orc.moe_route(logits, k)
    assert torch.equal(idx_c, idx_p)
    assert torch.allclose(w_c, w_p, rtol=1e-5)

    for seg in (E, E // 4):
        nseg = E // seg
        cap = T * k + seg * 127
        cap = (cap + 127) // 128 * 128
        rop = torch.empty(T, k, dtype=torch.int32)
        por = torch.empty(nseg, cap, dtype=torch.int32)
        offs = torch.empty(nseg, seg + 1, dtype=torch.int32)
        cnt = torch.empty(E, dtype=torch.int32)
        L.dk_c_permute(C.c_void_p(idx_p.data_ptr()), T, k, E, 128, seg, cap, C.c_void_p(rop.data_ptr()),
                       C.c_void_p(por.data_ptr()), C.c_void_p(offs.data_ptr()), C.c_void_p(cnt.data_ptr()))
        if seg == E:
            r_rop, r_por, r_offs, r_cnt = orc.moe_permute(idx_p, E, 128)
            assert torch.equal(rop, r_rop) and torch.equal(offs[0], r_offs) and torch.equal(cnt, r_cnt)
            assert torch.equal(por[0, :r_por.numel()], r_por)
        else:
            recv_pair, recv_offs, r_rop, _ = orc.ep_layout(idx_p, E, nseg)
            assert torch.equal(rop, r_rop)
            for d in range(nseg):
                assert torch.equal(offs[d], recv_offs[d])
                assert torch.equal(por[d, :recv_pair[d].numel()], recv_pair[d])

    for scale in (1.0, 3e-4, 500.0):
        x = (torch.randn(256, 384, generator=g) * scale).to(torch.bfloat16)
        x[:128, :128] = 0
        q = torch.empty(256, 384, dtype=torch.uint8)
        s = torch.empty(2, 3)
        L.dk_c_quant_block128(C.c_void_p(x.view(torch.int16).data_ptr()), 256, 384, C.c_void_p(q.data_ptr()),
                              C.c_void_p(s.data_ptr()))
        q_p, s_p = orc.quant_block128(x)
        assert torch.equal(s, s_p)
        assert torch.equal(q, q_p)


def test_c_e4m3_conversion_exhaustive_against_torch():
    """Every bf16 bit pattern in [-448, 448] through the C quantiser's e4m3 rounding vs torch's."""
    import ctypes as C
    L = _c_oracle()
    bits = torch.arange(0, 65536, dtype=torch.int32).to(torch.int16)
    vals = bits.view(torch.bfloat16).float()
    keep = torch.isfinite(vals) & (vals.abs() <= 448)
    v = vals[keep]
    n = (v.numel() // 128) * 128
    v = v[:n]
    # scale 1: put the block maximum at exactly 448 so that s == 1 and q == e4m3(x)
    x = v.reshape(-1, 128).to(torch.bfloat16)
    pad_rows = (-x.shape[0]) % 128
    x = torch.cat([x, torch.zeros(pad_rows, 128, dtype=torch.bfloat16)], 0)
    x[0, 0] = 448.0
    x[-1 if pad_rows else 0, 1] = 448.0
    for r0 in range(0, x.shape[0], 128):
        x[r0, 2] = 448.0
    q = torch.empty(x.shape, dtype=torch.uint8)
    s = torch.empty(x.shape[0] // 128, 1)
    L.dk_c_quant_block128(C.c_void_p(x.view(torch.int16).data_ptr()), x.shape[0], 128, C.c_void_p(q.data_ptr()),
                          C.c_void_p(s.data_ptr()))
    assert bool((s == 1.0).all())
    want = x.float().to(torch.float8_e4m3fn).view(torch.uint8)
    assert torch.equal(q, want)


# ---- MXFP8 (1x32 e8m0) oracle against the reference's regenerated fixture -----------------------
def test_mx_oracle_matches_reference_fixture(orc):
    """tests/golden/mx_fixture.npz: the reference's mma_scaled fixture (mt19937(123), N(0, 0.5),
    256^3) regenerated by make_mx_golden.cpp. The Python oracle must reproduce its quantisation bit
    for bit and its CPU expectation to fp32 summation-order accuracy; the fixture's own acceptance
    (|err| <= 0.1 % of max|c|, mma_scaled.cu:296-307) is asserted as well."""
    fx = np.load(GOLD / "mx_fixture.npz")
    a, b = torch.from_numpy(fx["a"]), torch.from_numpy(fx["b"])
    aq, sa = orc.mx_quant(a)
    bq, sb = orc.mx_quant(b)
    assert np.array_equal(sa.numpy(), fx["sa"]) and np.array_equal(sb.numpy(), fx["sb"])
    assert np.array_equal(aq.numpy(), fx["aq"]) and np.array_equal(bq.numpy(), fx["bq"])
    # the block maximum lands in [1, 2) before rounding: no element can saturate
    assert float(aq.view(torch.float8_e4m3fn).float().abs().max()) <= 2.0
    c = orc.mx_gemm_ref(aq, sa, bq, sb)
    want = torch.from_numpy(fx["c"])
    c_max = float(want.abs().max())
    assert float((c - want).abs().max()) <= 1e-5 * c_max
    assert float((c - want).abs().max()) <= 1e-3 * c_max          # the fixture's acceptance
    # quantisation error itself, against the unquantised product: a few per cent (3 mantissa bits)
    assert orc.rel_fro(c, a @ b.t()) < 0.06


def test_mx_scale_layouts(orc):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(256, 512, generator=g) * torch.logspace(-6, 6, 512)[None, :]
    x[5, 64:96] = 0                                     # an all-zero block: scale byte 0
    q, s = orc.mx_quant(x)
    assert s.shape == (256, 16) and int(s[5, 2]) == 0
    assert torch.equal(q[5, 64:96], torch.zeros(32, dtype=torch.uint8))
    # dequantised values stay within one e4m3 step (2^-3 relative, 2^-4 after rounding) of x
    d = orc.mx_dequant(q, s)
    blk_max = x.reshape(256, 16, 32).abs().amax(-1, keepdim=True).expand(-1, -1, 32).reshape(256, 512)
    assert bool(((d - x).abs() <= blk_max * 2.0 ** -4 + 1e-30).all())
    # the reference's per-iteration packing: byte j of word [ki, row] is the scale of block 4*ki + j
    w = orc.mx_pack_iter(s)
    assert w.shape == (4, 256)
    for ki, row, j in ((0, 0, 0), (1, 7, 3), (3, 255, 2)):
        assert (int(w[ki, row]) >> (8 * j)) & 0xFF == int(s[row, 4 * ki + j])
    # the tensor-core atom layout: row r0 + 32*r1 of row block rb, group k of K block kb
    t = orc.mx_sf_atoms(s)
    assert t.shape == (2, 4, 32, 4, 4)
    for rb, kb, r0, r1, k in ((0, 0, 0, 0, 0), (1, 3, 31, 3, 3), (0, 2, 17, 1, 2)):
        assert int(t[rb, kb, r0, r1, k]) == int(s[rb * 128 + r1 * 32 + r0, kb * 4 + k])
    assert t.flatten()[((1 * 4 + 3) * 32 + 31) * 16 + 3 * 4 + 3] == s[255, 15]   # byte offset r0*16 + r1*4 + k


def test_pow2_block_quantiser(orc):
    """Power-of-two 128x128 scales: never saturate, give up at most one bit against the fp32
    scale, and are the same numbers whether read as fp32 scales or as e8m0 bytes in 1x32 atoms."""
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(256, 384, generator=g) * torch.logspace(-3, 3, 384)[None, :]).to(torch.bfloat16)
    x[:128, :128] = 0
    x[128:, 128:256] = 448.0 * 2.0 ** -5               # amax/448 an exact power of two
    q, s, e = orc.quant_block128_pow2(x)
    q0, s0 = orc.quant_block128(x)
    assert float(s[0, 0]) == 1.0 and int(e[0, 0]) == 127
    assert float(s[1, 1]) == 2.0 ** -5 and int(e[1, 1]) == 122
    assert bool((s >= s0).all()) and bool((s < 2 * s0 + 1e-30).all())      # rounded up, by less than 2x
    assert torch.equal(torch.ldexp(torch.ones_like(s), e.to(torch.int32) - 127), s)
    qf = q.view(torch.float8_e4m3fn).float()
    assert float(qf.abs().max()) <= 448.0
    blk_max = qf.abs().reshape(2, 128, 3, 128).amax(dim=(1, 3))
    assert bool((blk_max[s0 != 1] > 223.0).all())                            # block maximum in (224, 448]
    # dequantised error: the fp32-scale quantiser's bound doubled at worst
    d, d0 = orc.dequant_block128(q, s), orc.dequant_block128(q0, s0)
    xf = x.float()
    assert orc.rel_fro(d, xf) <= 2.0 * orc.rel_fro(d0, xf) + 1e-6
    # as scale atoms for the tensor core: 16 identical bytes per row group
    atoms = orc.block128_scales_to_sf_atoms(e)
    assert atoms.shape == (2, 3, 32, 4, 4) and bool((atoms[1, 1] == 122).all())
    # and those atoms describe the same dequantisation as the 1x32 format would
    s_rows = e[:, :, None].expand(-1, -1, 4).reshape(2, 12).repeat_interleave(128, dim=0)   # [R, C/32]
    assert torch.allclose(orc.mx_dequant(q, s_rows), d)
    assert torch.equal(orc.mx_sf_atoms(s_rows), atoms)


def test_rows128_quantiser_of_the_fp8_dispatch(orc):
    """1x128 power-of-two row scales: a row's bytes and scales depend on that row alone (so tokens
    can be quantised where they live, before they are permuted into expert order); where all rows of
    a 128-row block are equal they are the 128x128 quantiser's; the atom layout puts row slot
    i = 32*i1 + i0 at bytes i0*16 + i1*4 .. +3 of each atom."""
    g = torch.Generator().manual_seed(12)
    x = (torch.randn(256, 640, generator=g) * torch.logspace(-2, 2, 256)[:, None]).to(torch.bfloat16)
    x[7] = 0
    q, s, e = orc.quant_rows128_pow2(x)
    assert q.shape == (256, 640) and s.shape == (256, 5) and e.shape == (256, 5)
    assert bool((s[7] == 1.0).all()) and bool((e[7] == 127).all()) and bool((q[7] == 0).all())
    perm = torch.randperm(256, generator=g)
    qp, sp, ep = orc.quant_rows128_pow2(x[perm])
    assert torch.equal(qp, q[perm]) and torch.equal(ep, e[perm])
    one = orc.quant_rows128_pow2(x[33:34])
    assert torch.equal(one[0][0], q[33]) and torch.equal(one[2][0], e[33])
    qf = q.view(torch.float8_e4m3fn).float().reshape(256, 5, 128)
    gmax = qf.abs().amax(dim=2)
    live = x.float().reshape(256, 5, 128).abs().amax(dim=2) > 0
    assert bool((gmax[live] > 223.0).all()) and float(gmax.max()) <= 448.0     # group maximum in (224, 448]
    assert orc.rel_fro(orc.dequant_rows128(q, s), x.float()) <= 0.04
    # a block of equal rows: the row scales are the block's scales
    xb = x[40:41].expand(128, -1).contiguous()
    qb, sb, eb = orc.quant_block128_pow2(xb)
    qr, sr, er = orc.quant_rows128_pow2(xb)
    assert torch.equal(qb, qr) and bool((er == eb[0][None, :]).all())
    # atoms
    atoms = orc.rows128_scales_to_block_atoms(e)
    assert atoms.shape == (2, 2, 512)
    for r, kb in ((0, 0), (37, 2), (255, 4), (130, 3)):
        i = r % 128
        assert int(atoms[r // 128, kb // 4, (i % 32) * 16 + (i // 32) * 4 + kb % 4]) == int(e[r, kb])
    assert int(atoms[0, 1, 0 * 16 + 0 * 4 + 1]) == 127        # column block 5 does not exist: scale 1
    # and the uniform form is the special case of equal rows
    assert torch.equal(orc.rows128_scales_to_block_atoms(er), orc.block128_scales_to_block_atoms(eb).reshape(1, 2, 512))


def test_ffn_with_row_scales_reduces_to_block_scales(orc):
    """moe_ffn_rows_pow2_ref with row scales that are constant inside every 128-row block is
    moe_ffn_pow2_ref."""
    x, logits, w13q, w13s, w2q, w2s = orc.make_moe_inputs(256, 256, 128, 4, 2, seed=3)
    idx, w = orc.moe_route(logits, 2)
    rop, por, offs, counts = orc.moe_permute(idx, 4)
    rows = orc.moe_gather_rows(x, por, 2)
    xq, xs, _ = orc.quant_block128_pow2(rows)
    p13 = [orc.quant_block128_pow2(orc.dequant_block128(w13q[e], w13s[e]).to(torch.bfloat16)) for e in range(4)]
    p2 = [orc.quant_block128_pow2(orc.dequant_block128(w2q[e], w2s[e]).to(torch.bfloat16)) for e in range(4)]
    st = lambda parts, i: torch.stack([p[i] for p in parts])
    a = orc.moe_ffn_pow2_ref(xq, xs, st(p13, 0), st(p13, 1), st(p2, 0), st(p2, 1), offs)[0]
    xs_rows = xs.repeat_interleave(128, dim=0)
    b = orc.moe_ffn_rows_pow2_ref(xq, xs_rows, st(p13, 0), st(p13, 1), st(p2, 0), st(p2, 1), offs)[0]
    assert torch.allclose(a, b, rtol=1e-6, atol=1e-6)
