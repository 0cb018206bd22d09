"""CPU oracle for the multi-GPU hot path. TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs may import
this module, and only as the checker (or as the timed CPU baseline): nothing that ships routes
through it.

What each function restates, by path inside the reference project:

  gemm_ref            torch.matmul(A, B.t())           distributed-kernels/bf16_gemm/example.py:105
                      (the kernel's contract, C = A . B^T with fp32 accumulate,
                       distributed-kernels/bf16_gemm/kernel.cpp:188-243)
  example_inputs      the example's seeds and init     distributed-kernels/bf16_gemm/example.py:93-96
  example_check       max |C - C_ref| < 0.1            distributed-kernels/bf16_gemm/example.py:119-121
  quant_block128 /    pattern of the reference's block-scaled fixtures (quantise, then the CPU truth
  dequant_block128    dequantises per block): tests/unit/cdna4/warp/register/tile/mma_scaled.cu:200-258,
                      kernels/cdna4/gemm/mxfp8/MXFP8_8wave/8_wave_NT.cu:286-327. Those use 1x32 e8m0
                      scales; here the blocks are 128x128 with fp32 scales.
  grouped / ffn       CPU-loop pattern of kernels/cdna4/gemm/fp8fp32/FP8_8wave/8_wave.cu:445-476
  quant_rows128_pow2 / the same quantise-then-dequantise pattern for 1x128 row groups with power-of-two
  moe_ffn_rows_pow2_ref  scales (what the expert-parallel layer sends between GPUs as fp8); no counterpart
                      in the reference, which quantises nothing on the way between GPUs

PARITY PINNING. The reference holds exactly one check on this path: the example's seeds,
initialisation and threshold for the GEMM; `example_inputs` + `example_check` restate it and
tests/golden/ holds vectors generated with it. Reduce-scatter, all-reduce, routing, permutation,
block quantisation, grouped GEMM, dispatch and combine do not exist in the reference at all
(no implementation, no test, no golden vector): for those this oracle is the definition and their
parity is UNPINNED by the reference.
"""
from __future__ import annotations

import math

import torch

FP8_MAX = 448.0
BLOCK = 128


# --------------------------------------------------------------------------- helpers
def rel_fro(x: torch.Tensor, ref: torch.Tensor) -> float:
    """Relative Frobenius error ||x - ref|| / ||ref|| in fp64."""
    x = x.double()
    ref = ref.double()
    d = (x - ref).norm().item()
    n = ref.norm().item()
    return d / n if n > 0 else d


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


# --------------------------------------------------------------------------- GEMM
def make_gemm_inputs(M: int, N: int, K: int, seed: int = 0):
    """A ~ N(0,1) bf16 [M,K]; B ~ N(0,1/K) bf16 [K,N]; returns (A, Bt = B^T contiguous [N,K])."""
    g = _gen(seed)
    A = torch.randn(M, K, generator=g).to(torch.bfloat16)
    B = (torch.randn(K, N, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    return A, B.t().contiguous()


def gemm_ref(A: torch.Tensor, Bt: torch.Tensor) -> torch.Tensor:
    """fp32 C = A . Bt^T from the bf16-rounded inputs (example.py:105, in fp32 instead of bf16)."""
    return A.float() @ Bt.float().t()


def example_inputs(M_local: int, N: int, K: int, rank: int = 0, scale: float = 10.0):
    """Inputs exactly as the reference example draws them (example.py:93-96): global torch seed
    1234+rank for A, 0 for B, bf16 randn divided by `scale`. Drawn on the CPU generator here."""
    torch.manual_seed(1234 + rank)
    A = torch.randn(M_local, K, dtype=torch.bfloat16) / scale
    torch.manual_seed(0)
    B = torch.randn(N, K, dtype=torch.bfloat16) / scale
    return A, B


def example_check(C: torch.Tensor, A: torch.Tensor, B: torch.Tensor):
    """The example's own acceptance test (example.py:105,119-121): bf16 matmul reference,
    max-abs error below 0.1. Returns (passed, max_error)."""
    C_ref = torch.matmul(A, B.t())
    err = (C.float() - C_ref.float()).abs().max().item()
    return err < 0.1, err


# --------------------------------------------------------------------------- GEMM + reduce-scatter
def shard_k(A: torch.Tensor, Bt: torch.Tensor, world: int):
    """Row-parallel shards: rank r gets A[:, rK/P:(r+1)K/P] and Bt[:, rK/P:(r+1)K/P]."""
    K = A.shape[1]
    assert K % world == 0
    kl = K // world
    return ([A[:, r * kl:(r + 1) * kl].contiguous() for r in range(world)],
            [Bt[:, r * kl:(r + 1) * kl].contiguous() for r in range(world)])


def gemm_rs_ref(A_shards, Bt_shards):
    """full = sum_r A_r . Bt_r^T in fp32; rank r owns rows [rM/P, (r+1)M/P). Returns the list of
    per-rank fp32 outputs."""
    world = len(A_shards)
    full = None
    for a, b in zip(A_shards, Bt_shards):
        p = gemm_ref(a, b)
        full = p if full is None else full + p
    M = full.shape[0]
    assert M % world == 0
    ml = M // world
    return [full[r * ml:(r + 1) * ml] for r in range(world)]


def gemm_rs_bf16_partials_ref(A_shards, Bt_shards):
    """The same, but modelling what travels: each rank's partial is rounded to bf16 before the
    owner sums the partials in fp32 in rank order. The device result is compared with
    gemm_rs_ref by tolerance; this variant bounds the extra rounding."""
    world = len(A_shards)
    parts = [gemm_ref(a, b).to(torch.bfloat16).float() for a, b in zip(A_shards, Bt_shards)]
    full = parts[0].clone()
    for p in parts[1:]:
        full += p
    ml = full.shape[0] // world
    return [full[r * ml:(r + 1) * ml] for r in range(world)]


# --------------------------------------------------------------------------- all-reduce
def make_allreduce_inputs(shape, world: int, seed_base: int = 100):
    return [torch.randn(*shape, generator=_gen(seed_base + r)).to(torch.bfloat16) for r in range(world)]


def allreduce_ref(xs):
    """fp32 sum over ranks, in rank order."""
    s = xs[0].float().clone()
    for x in xs[1:]:
        s += x.float()
    return s


# --------------------------------------------------------------------------- MoE: routing
def moe_route(logits: torch.Tensor, k: int):
    """Top-k on the raw fp32 logits; ties go to the lower expert index; weights are the softmax
    over all experts, gathered at the chosen experts and renormalised to sum to one.
    Returns (topk_idx int32 [T,k] sorted by descending logit, topk_w fp32 [T,k])."""
    assert logits.dtype == torch.float32
    T, E = logits.shape
    # stable descending sort keeps the lower index first among equal logits
    order = torch.sort(logits, dim=1, descending=True, stable=True).indices
    idx = order[:, :k].contiguous()
    p = torch.softmax(logits, dim=1)
    w = torch.gather(p, 1, idx)
    w = w / w.sum(dim=1, keepdim=True)
    return idx.to(torch.int32), w


def moe_permute(topk_idx: torch.Tensor, E: int, pad: int = BLOCK):
    """Group the (token, slot) pairs by expert.

    counts[e]   pairs routed to expert e
    offsets     exclusive scan of counts rounded up to `pad` ([E+1], offsets[E] = padded rows R)
    row_of_pair [T,k]: offsets[e] + rank of the pair among e's pairs in (token, slot) order
    pair_of_row [R]: inverse map, -1 for padding rows
    All int32, all bit-exact by construction."""
    T, k = topk_idx.shape
    flat = topk_idx.reshape(-1).long()
    counts = torch.bincount(flat, minlength=E)
    padded = (counts + pad - 1) // pad * pad
    offsets = torch.zeros(E + 1, dtype=torch.long)
    offsets[1:] = torch.cumsum(padded, 0)
    # rank within expert in (t, j) order = stable sort by expert
    order = torch.sort(flat, stable=True).indices            # pairs grouped by expert
    starts = torch.zeros(E, dtype=torch.long)
    starts[1:] = torch.cumsum(counts, 0)[:-1]
    rank_in_e = torch.empty(T * k, dtype=torch.long)
    rank_in_e[order] = torch.arange(T * k) - starts[flat[order]]
    row_of_pair = offsets[flat] + rank_in_e
    R = int(offsets[E])
    pair_of_row = torch.full((R,), -1, dtype=torch.long)
    pair_of_row[row_of_pair] = torch.arange(T * k)
    return (row_of_pair.reshape(T, k).to(torch.int32), pair_of_row.to(torch.int32),
            offsets.to(torch.int32), counts.to(torch.int32))


def moe_gather_rows(x: torch.Tensor, pair_of_row: torch.Tensor, k: int) -> torch.Tensor:
    """Permuted activations [R,H]: row r holds token pair_of_row[r] // k, zeros for padding."""
    R = pair_of_row.shape[0]
    out = torch.zeros(R, x.shape[1], dtype=x.dtype)
    valid = pair_of_row >= 0
    out[valid] = x[(pair_of_row[valid].long() // k)]
    return out


# --------------------------------------------------------------------------- fp8 block quantisation
def quant_block128(x: torch.Tensor):
    """Per 128x128 block: s = amax/448 (fp32; s = 1 when amax == 0); q = clamp(x/s, +-448) rounded
    to e4m3 (nearest even). x is [R,C] with R, C multiples of 128 (bf16 or fp32).
    Returns (q as uint8 bytes [R,C], s fp32 [R/128, C/128])."""
    R, Cc = x.shape
    assert R % BLOCK == 0 and Cc % BLOCK == 0
    xf = x.float().reshape(R // BLOCK, BLOCK, Cc // BLOCK, BLOCK)
    amax = xf.abs().amax(dim=(1, 3))
    s = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    q = (xf / s[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(R, Cc).view(torch.uint8), s.contiguous()


def quant_block128_pow2(x: torch.Tensor):
    """The same block quantiser with the scale rounded UP to a power of two (what an e8m0 scale can
    hold): s = 2^ceil(log2(amax/448)), 1 for an all-zero block. The block maximum then lands in
    (224, 448], so no element saturates and at most one bit of the e4m3 range is given up.
    Returns (q uint8 [R,C], s fp32 [R/128, C/128], e8m0 uint8 [R/128, C/128] = log2(s) + 127).
    A definition of this build (the reference has no 128x128 quantiser); it exists so that the
    tensor core can apply block scales itself."""
    R, Cc = x.shape
    assert R % BLOCK == 0 and Cc % BLOCK == 0
    xf = x.float().reshape(R // BLOCK, BLOCK, Cc // BLOCK, BLOCK)
    amax = xf.abs().amax(dim=(1, 3))
    m, e = torch.frexp(amax / FP8_MAX)                       # amax/448 = m * 2^e, m in [0.5, 1)
    e = torch.where(m == 0.5, e - 1, e).to(torch.int32)      # exact powers of two stay as they are
    e = torch.where(amax > 0, e, torch.zeros_like(e)).clamp(-127, 127)
    s = torch.ldexp(torch.ones_like(amax), e)
    q = (xf / s[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(R, Cc).view(torch.uint8), s.contiguous(), (e + 127).to(torch.uint8)


def block128_scales_to_sf_atoms(e8m0: torch.Tensor) -> torch.Tensor:
    """128x128 power-of-two block scales as the tensor core's 1x32 scale atoms (see mx_sf_atoms):
    every row of a block and each of its four 32-element K groups carries the block's byte.
    [R/128, C/128] -> [R/128, C/128, 32, 4, 4]."""
    return e8m0[:, :, None, None, None].expand(-1, -1, 32, 4, 4).contiguous()


def block128_scales_to_block_atoms(e8m0: torch.Tensor) -> torch.Tensor:
    """128x128 power-of-two block scales in the compact form the grouped GEMM reads: the four scale
    bytes the tensor core holds per row carry four consecutive K blocks. [R/128, C/128] ->
    [R/128, ceil(C/512), 128, 4] bytes, byte [rb, j, r, g] = e8m0[rb, 4j + g] for every row slot r
    (127 where the block does not exist)."""
    Rb, Cb = e8m0.shape
    j = (Cb + 3) // 4
    pad = torch.full((Rb, 4 * j), 127, dtype=torch.uint8)
    pad[:, :Cb] = e8m0
    return pad.reshape(Rb, j, 1, 4).expand(-1, -1, 128, -1).contiguous()


def quant_rows128_pow2(x: torch.Tensor):
    """Per-token quantiser of the fp8 dispatch: the power-of-two rule of quant_block128_pow2 applied
    to every 1x128 group of a row (s = 2^ceil(log2(amax/448)), 1 for an all-zero group). Any number
    of rows. Returns (q uint8 [R,C], s fp32 [R, C/128], e8m0 uint8 [R, C/128]).
    A definition of this build (the reference quantises nothing on the way between GPUs)."""
    R, Cc = x.shape
    assert Cc % BLOCK == 0
    xf = x.float().reshape(R, Cc // BLOCK, BLOCK)
    amax = xf.abs().amax(dim=2)
    m, e = torch.frexp(amax / FP8_MAX)
    e = torch.where(m == 0.5, e - 1, e).to(torch.int32)
    e = torch.where(amax > 0, e, torch.zeros_like(e)).clamp(-127, 127)
    s = torch.ldexp(torch.ones_like(amax), e)
    q = (xf / s[:, :, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(R, Cc).view(torch.uint8), s.contiguous(), (e + 127).to(torch.uint8)


def dequant_rows128(q_u8: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    R, Cc = q_u8.shape
    qf = q_u8.view(torch.float8_e4m3fn).float().reshape(R, Cc // BLOCK, BLOCK)
    return (qf * s[:, :, None]).reshape(R, Cc)


def rows128_scales_to_block_atoms(e8m0: torch.Tensor) -> torch.Tensor:
    """1x128 power-of-two row scales [R, C/128] (R a multiple of 128) in the atoms the grouped GEMM
    reads: [R/128, ceil(C/512), 512] bytes; inside an atom row slot i = 32*i1 + i0 of the 128-row
    block owns the four bytes at i0*16 + i1*4, byte g = the scale of column block 4j + g (127 where
    that block does not exist)."""
    R, Cb = e8m0.shape
    assert R % BLOCK == 0
    j = (Cb + 3) // 4
    pad = torch.full((R, 4 * j), 127, dtype=torch.uint8)
    pad[:, :Cb] = e8m0
    # [rb, i1, i0, j, g] -> [rb, j, i0, i1, g]
    return pad.reshape(R // BLOCK, 4, 32, j, 4).permute(0, 3, 2, 1, 4).contiguous().reshape(R // BLOCK, j, 512)


def dequant_block128(q_u8: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    R, Cc = q_u8.shape
    qf = q_u8.view(torch.float8_e4m3fn).float().reshape(R // BLOCK, BLOCK, Cc // BLOCK, BLOCK)
    return (qf * s[:, None, :, None]).reshape(R, Cc)


# --------------------------------------------------------------------------- fp8 grouped GEMM / FFN
def grouped_gemm_ref(xq, xs, wq, ws, offsets):
    """Y[rows of e] = dequant(X)[rows of e] . dequant(W[e])^T in fp32.
    xq [R,K] u8 + xs [R/128,K/128]; wq [E,N,K] u8 + ws [E,N/128,K/128]; offsets [E+1]."""
    E = wq.shape[0]
    X = dequant_block128(xq, xs)
    Y = torch.zeros(X.shape[0], wq.shape[1], dtype=torch.float32)
    for e in range(E):
        a, b = int(offsets[e]), int(offsets[e + 1])
        if b > a:
            W = dequant_block128(wq[e], ws[e])
            Y[a:b] = X[a:b] @ W.t()
    return Y


def silu_mul(gu: torch.Tensor) -> torch.Tensor:
    """gu [R,2F] = [gate | up] -> silu(gate) * up, fp32."""
    F = gu.shape[1] // 2
    g, u = gu[:, :F], gu[:, F:]
    return g * torch.sigmoid(g) * u


def moe_ffn_ref(xq, xs, w13q, w13s, w2q, w2s, offsets):
    """gate/up grouped GEMM -> SiLU(gate)*up -> requantise with the same block rule -> down
    grouped GEMM. Returns (Y fp32 [R,H], hq u8 [R,F], hs fp32)."""
    gu = grouped_gemm_ref(xq, xs, w13q, w13s, offsets)
    h = silu_mul(gu)
    hq, hs = quant_block128(h)
    y = grouped_gemm_ref(hq, hs, w2q, w2s, offsets)
    return y, hq, hs


def moe_ffn_pow2_ref(xq, xs, w13q, w13s, w2q, w2s, offsets):
    """moe_ffn_ref with the intermediate requantised by quant_block128_pow2 (the scales handed in
    are powers of two as well; the arithmetic is the same block dequantisation).
    Returns (Y fp32 [R,H], hq u8 [R,F], hs fp32, h_e8 u8)."""
    gu = grouped_gemm_ref(xq, xs, w13q, w13s, offsets)
    h = silu_mul(gu)
    hq, hs, he = quant_block128_pow2(h)
    y = grouped_gemm_ref(hq, hs, w2q, w2s, offsets)
    return y, hq, hs, he


def moe_ffn_rows_pow2_ref(xq, xs_rows, w13q, w13s, w2q, w2s, offsets):
    """moe_ffn_pow2_ref for activations that arrive with 1x128 row scales (quant_rows128_pow2): the
    gate/up GEMM dequantises every row with its own scales; from the SiLU on it is the same.
    Returns (Y fp32 [R,H], hq u8 [R,F], hs fp32, h_e8 u8)."""
    X = dequant_rows128(xq, xs_rows)
    gu = torch.zeros(X.shape[0], w13q.shape[1], dtype=torch.float32)
    for e in range(w13q.shape[0]):
        a, b = int(offsets[e]), int(offsets[e + 1])
        if b > a:
            gu[a:b] = X[a:b] @ dequant_block128(w13q[e], w13s[e]).t()
    h = silu_mul(gu)
    hq, hs, he = quant_block128_pow2(h)
    y = grouped_gemm_ref(hq, hs, w2q, w2s, offsets)
    return y, hq, hs, he


def moe_combine_ref(y: torch.Tensor, row_of_pair: torch.Tensor, topk_w: torch.Tensor):
    """out[t] = sum_j w[t,j] * Y[row(t,j)] in fp32 (slot order)."""
    T, k = row_of_pair.shape
    out = torch.zeros(T, y.shape[1], dtype=torch.float32)
    for j in range(k):
        out += topk_w[:, j:j + 1] * y[row_of_pair[:, j].long()].float()
    return out


# --------------------------------------------------------------------------- expert-parallel layout
def ep_layout(topk_idx: torch.Tensor, E: int, world: int, pad: int = BLOCK):
    """Expert-parallel dispatch plan. Token t lives on rank t // (T/P); expert e on rank
    e // (E/P). On the receiving rank the rows are ordered by (local expert, global token, slot),
    each expert padded to `pad` rows. Returns per destination rank d:
      recv_pair[d]    int32 [R_d]: global pair index t*k+j held by each row (-1 = padding)
      recv_offsets[d] int32 [E/P + 1]
    and the global row_of_pair [T,k] (row inside the destination rank) and dest_of_pair [T,k]."""
    T, k = topk_idx.shape
    epr = E // world
    dest = (topk_idx.long() // epr)
    recv_pair, recv_offsets = [], []
    row_of_pair = torch.empty(T, k, dtype=torch.long)
    flat_e = topk_idx.reshape(-1).long()
    for d in range(world):
        sel = (dest.reshape(-1) == d).nonzero().flatten()          # pairs in (t, j) order
        le = flat_e[sel] - d * epr
        counts = torch.bincount(le, minlength=epr)
        padded = (counts + pad - 1) // pad * pad
        offs = torch.zeros(epr + 1, dtype=torch.long)
        offs[1:] = torch.cumsum(padded, 0)
        order = torch.sort(le, stable=True).indices
        starts = torch.zeros(epr, dtype=torch.long)
        starts[1:] = torch.cumsum(counts, 0)[:-1]
        rank_in_e = torch.empty(sel.numel(), dtype=torch.long)
        rank_in_e[order] = torch.arange(sel.numel()) - starts[le[order]]
        rows = offs[le] + rank_in_e
        rp = torch.full((int(offs[epr]),), -1, dtype=torch.long)
        rp[rows] = sel
        row_of_pair.reshape(-1)[sel] = rows
        recv_pair.append(rp.to(torch.int32))
        recv_offsets.append(offs.to(torch.int32))
    return recv_pair, recv_offsets, row_of_pair.to(torch.int32), dest.to(torch.int32)


# --------------------------------------------------------------------------- synthetic MoE configs
def make_moe_inputs(T: int, H: int, F: int, E: int, k: int, seed: int = 0, zipf_s: float = 0.0,
                    perm_seed: int = 1):
    """Tokens x ~ N(0,1) bf16 [T,H]; logits fp32 [T,E] = N(0,1) (+ log p_e with
    p_e ~ (pi(e)+1)^-s for a seeded permutation pi when zipf_s > 0); per expert
    W13 ~ N(0,1/H) [2F,H], W2 ~ N(0,1/F) [H,F], block-quantised."""
    g = _gen(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    if zipf_s > 0:
        pi = torch.randperm(E, generator=_gen(perm_seed)).float()
        p = (pi + 1.0) ** (-zipf_s)
        logits = logits + torch.log(p / p.sum())[None, :]
    w13q, w13s, w2q, w2s = [], [], [], []
    for _ in range(E):
        q, s = quant_block128(torch.randn(2 * F, H, generator=g) / math.sqrt(H))
        w13q.append(q); w13s.append(s)
        q, s = quant_block128(torch.randn(H, F, generator=g) / math.sqrt(F))
        w2q.append(q); w2s.append(s)
    return (x, logits.contiguous(), torch.stack(w13q), torch.stack(w13s), torch.stack(w2q),
            torch.stack(w2s))


# --------------------------------------------------------------------------- MXFP8 (1x32 e8m0 blocks)
# The block-scaled format the reference ships and tests: e4m3 elements with one e8m0 (power of
# two) scale per 32 consecutive elements of K. Follows the host code of its fixtures:
# compute_e8m0 and the quantisation loop at tests/unit/cdna4/warp/register/tile/mma_scaled.cu:200-232
# (the same code is at kernels/cdna4/gemm/mxfp8/MXFP8_8wave/8_wave_NT.cu:286-327), the CPU
# expectation at mma_scaled.cu:234-247, the per-iteration scale packing at mma_scaled.cu:249-264.
# Pinned by tests/golden/mx_fixture.npz, regenerated from that fixture's seed and distribution
# (std::mt19937(123), N(0, 0.5)) by tests/golden/make_mx_golden.cpp.
MX_BLOCK = 32


def mx_quant(x: torch.Tensor):
    """x fp32 [R, K], K % 32 == 0 -> (q e4m3 bytes as uint8 [R, K], s e8m0 as uint8 [R, K/32]).
    s = clamp(floor(log2(amax)) + 127, 0, 254), 0 for an all-zero block; q = e4m3(x * 2^(127-s)):
    the block maximum lands in [1, 2)."""
    R, K = x.shape
    assert K % MX_BLOCK == 0
    xb = x.float().reshape(R, K // MX_BLOCK, MX_BLOCK)
    amax = xb.abs().amax(dim=-1)
    # floor(log2(.)) of an fp32 value is its unbiased exponent (frexp gives amax = m * 2^e, m in [0.5, 1))
    e = torch.frexp(amax)[1].to(torch.int32) - 1
    s = torch.where(amax == 0, torch.zeros_like(e), (e + 127).clamp(0, 254))
    inv = torch.ldexp(torch.ones_like(amax), (127 - s).to(torch.int32))
    q = (xb * inv[..., None]).reshape(R, K).to(torch.float8_e4m3fn).view(torch.uint8)
    return q, s.to(torch.uint8)


def mx_dequant(q_u8: torch.Tensor, s_u8: torch.Tensor) -> torch.Tensor:
    R, K = q_u8.shape
    f = torch.ldexp(torch.ones(R, K // MX_BLOCK), s_u8.to(torch.int32) - 127)
    return (q_u8.view(torch.float8_e4m3fn).float().reshape(R, K // MX_BLOCK, MX_BLOCK) * f[..., None]).reshape(R, K)


def mx_gemm_ref(aq, sa, bq, sb) -> torch.Tensor:
    """C[M, N] = dequant(A) @ dequant(B)^T in fp32 (products of e4m3 values and powers of two are
    exact in fp32; only the order of the fp32 additions differs between implementations)."""
    return mx_dequant(aq, sa) @ mx_dequant(bq, sb).t()


def mx_pack_iter(s_u8: torch.Tensor) -> torch.Tensor:
    """The reference's device layout of the scales: per K iteration of 128 elements one uint32 per
    row holding its four e8m0 bytes, little endian: [K/128, R] (mma_scaled.cu:249-264)."""
    R, SK = s_u8.shape
    assert SK % 4 == 0
    b = s_u8.reshape(R, SK // 4, 4).to(torch.int64)
    w = b[..., 0] | (b[..., 1] << 8) | (b[..., 2] << 16) | (b[..., 3] << 24)
    return w.t().contiguous().to(torch.int64)


def mx_sf_atoms(s_u8: torch.Tensor) -> torch.Tensor:
    """The layout the sm_100 tensor core wants the scales in (one 512-byte atom per 128 rows x 128
    elements of K, byte offset r0*16 + r1*4 + k for row r0 + 32*r1 and 32-element group k), which a
    32x128b.warpx4 tcgen05.cp moves to four tensor-memory columns: [R/128, K/128, 32, 4, 4] bytes."""
    R, SK = s_u8.shape
    assert R % 128 == 0 and SK % 4 == 0
    t = s_u8.reshape(R // 128, 4, 32, SK // 4, 4)          # [rb, r1, r0, kb, k]
    return t.permute(0, 3, 2, 1, 4).contiguous()            # [rb, kb, r0, r1, k]
