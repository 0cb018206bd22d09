"""Routing, permutation, block quantisation and combine on the GPU against the oracle.
Indices, counts, offsets, both permutation maps and the quantised bytes and scales: bit-exact.
Routing weights and combine: floating point, tolerances written at the assertion."""
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"


def _bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


@pytest.mark.parametrize("T,E,k", [(64, 8, 2), (1000, 8, 2), (513, 256, 8), (7, 5, 3), (4096, 64, 6), (1, 1, 1)])
def test_route_matches_oracle(capi, orc, T, E, k):
    g = torch.Generator().manual_seed(T + E)
    logits = torch.randn(T, E, generator=g)
    if T > 3 and E > 5:
        logits[3, 1] = logits[3, 5] = logits[3].max() + 1    # a tie at the top
        logits[2] = 0.0                                      # all equal
    idx, w = capi.moe_route(logits.cuda(), k)
    ridx, rw = orc.moe_route(logits, k)
    assert torch.equal(idx.cpu(), ridx)                          # bit-exact
    assert torch.allclose(w.cpu(), rw, rtol=1e-5, atol=1e-7)     # expf on GPU vs CPU
    assert torch.allclose(w.sum(1).cpu(), torch.ones(T), atol=1e-5)


def test_route_golden(capi):
    fx = np.load(GOLD / "moe_small.npz")
    idx, w = capi.moe_route(torch.from_numpy(fx["logits"]).cuda(), 2)
    assert np.array_equal(idx.cpu().numpy(), fx["topk_idx"])
    assert np.allclose(w.cpu().numpy(), fx["topk_w"], rtol=1e-5)


@pytest.mark.parametrize("T,E,k", [(64, 8, 2), (1000, 8, 2), (2048, 256, 8), (1, 4, 1), (5000, 16, 4), (0, 8, 2)])
def test_permute_bit_exact(capi, orc, T, E, k):
    g = torch.Generator().manual_seed(T * 7 + E)
    idx, _ = orc.moe_route(torch.randn(T, E, generator=g), k) if T else (torch.zeros(0, k, dtype=torch.int32), None)
    rop, por, offs, counts = capi.moe_permute(idx.cuda(), E, 128)
    r_rop, r_por, r_offs, r_counts = orc.moe_permute(idx, E, 128)
    torch.cuda.synchronize()
    assert torch.equal(counts.cpu(), r_counts)
    assert torch.equal(offs.cpu(), r_offs)
    assert torch.equal(rop.cpu(), r_rop)
    R = int(r_offs[-1])
    assert torch.equal(por.cpu()[:R], r_por)
    assert (por.cpu()[R:] == -1).all()


def test_permute_skewed_and_empty_experts(capi, orc):
    """Zipf-like popularity: some experts get thousands of pairs, many get none."""
    T, E, k = 4096, 256, 8
    g = torch.Generator().manual_seed(5)
    p = (torch.randperm(E, generator=g).float() + 1) ** -1.1
    logits = torch.randn(T, E, generator=g) + torch.log(p / p.sum())[None]
    logits[:, 200:] = -1e9                                   # experts 200.. never chosen
    idx, _ = orc.moe_route(logits, k)
    rop, por, offs, counts = capi.moe_permute(idx.cuda(), E, 128)
    r = orc.moe_permute(idx, E, 128)
    assert torch.equal(rop.cpu(), r[0]) and torch.equal(offs.cpu(), r[2]) and torch.equal(counts.cpu(), r[3])
    assert int(counts[200:].sum()) == 0


def test_permute_segments_match_ep_layout(capi, orc):
    T, E, k, P = 1024, 32, 4, 4
    g = torch.Generator().manual_seed(11)
    idx, _ = orc.moe_route(torch.randn(T, E, generator=g), k)
    rop, por, offs, counts = capi.moe_permute(idx.cuda(), E, 128, experts_per_segment=E // P)
    recv_pair, recv_offs, r_rop, dest = orc.ep_layout(idx, E, P)
    assert torch.equal(rop.cpu(), r_rop)
    for d in range(P):
        assert torch.equal(offs.cpu()[d], recv_offs[d])
        R = int(recv_offs[d][-1])
        assert torch.equal(por.cpu()[d, :R], recv_pair[d])


def test_quant_bit_exact_and_golden(capi, orc):
    fx = np.load(GOLD / "moe_small.npz")
    x = _bf16(fx["x"])
    q, s = capi.quant_block128(x.cuda())
    assert np.array_equal(q.cpu().numpy(), fx["q"]) and np.array_equal(s.cpu().numpy(), fx["s"])
    g = torch.Generator().manual_seed(0)
    # 1e-30 and 1e30 put the block scales outside the range in which the kernel replaces the division
    # by its FMA form; the heavy-tailed case spreads the quotients over the whole e4m3 range
    for scale in (1.0, 1e-3, 300.0, 1e-30, 1e30, "heavy"):
        if scale == "heavy":
            x = (torch.randn(4096, 512, generator=g) * torch.exp(3.0 * torch.randn(4096, 512, generator=g))).to(torch.bfloat16)
        else:
            x = (torch.randn(512, 384, generator=g) * scale).to(torch.bfloat16)
        x[5, 7] = 0.0
        q, s = capi.quant_block128(x.cuda())
        rq, rs = orc.quant_block128(x)
        assert torch.equal(s.cpu(), rs)
        assert torch.equal(q.cpu(), rq)


def test_gather_quant_matches_oracle(capi, orc):
    T, H, E, k = 300, 256, 8, 2
    g = torch.Generator().manual_seed(3)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    idx, _ = orc.moe_route(torch.randn(T, E, generator=g), k)
    rop, por, offs, _ = orc.moe_permute(idx, E)
    want_q, want_s = orc.quant_block128(orc.moe_gather_rows(x, por, k))
    q, s = capi.quant_block128(x.cuda(), rows=por.numel(), row_map=por.cuda(), map_mode=1, k=k)
    assert torch.equal(q.cpu(), want_q) and torch.equal(s.cpu(), want_s)
    # rows already in place, padding rows holding garbage
    xp = orc.moe_gather_rows(x, por, k)
    dirty = xp.clone()
    dirty[por < 0] = 77.0
    q2, s2 = capi.quant_block128(dirty.cuda(), row_map=por.cuda(), map_mode=2)
    assert torch.equal(q2.cpu(), want_q) and torch.equal(s2.cpu(), want_s)


def test_combine_matches_oracle(capi, orc):
    T, H, E, k = 257, 520, 8, 2
    g = torch.Generator().manual_seed(4)
    idx, w = orc.moe_route(torch.randn(T, E, generator=g), k)
    rop, por, offs, _ = orc.moe_permute(idx, E)
    y = torch.randn(int(offs[-1]), H, generator=g).to(torch.bfloat16)
    out = capi.moe_combine(y.cuda(), rop.cuda(), w.cuda())
    want = orc.moe_combine_ref(y, rop, w)
    assert orc.rel_fro(out.float().cpu(), want) <= 1e-2     # bf16 output rounding


def test_moe_argument_errors(capi):
    with pytest.raises(capi.DkError):
        capi.moe_route(torch.zeros(4, 300, device="cuda"), 2)            # E > 256
    with pytest.raises(capi.DkError):
        capi.moe_route(torch.zeros(4, 8, device="cuda"), 9)              # k > 8
    with pytest.raises(capi.DkError):
        capi.quant_block128(torch.zeros(100, 128, dtype=torch.bfloat16, device="cuda"))
