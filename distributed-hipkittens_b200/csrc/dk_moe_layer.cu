// One expert-parallel fp8 MoE layer as a single host call: route -> exchange the routing table ->
// permutation and token slots -> dispatch (each token crosses to a destination GPU ONCE, however
// many of that GPU's experts it is routed to) -> block quantisation of the rows that arrived ->
// gate/up grouped GEMM + SiLU*mul + requantise -> down grouped GEMM -> expert-side combine (one
// weighted partial sum per (token, GPU), pushed back to the token's home rank) -> final sum at home.
//
// The reference has no MoE and no exchange between ranks; the calling convention is the one of its
// GEMM (a device view addressing the same offset on every rank,
// distributed-kernels/bf16_gemm/kernel.cpp:25,39,58-59). No NCCL, no allocation, no separate
// barrier launches: a kernel that writes into peers ends by publishing a per-source flag, the kernel
// that consumes starts by waiting (bounded) for the flags of all sources (dk_moe_int.h).
//
// Layout: token t lives on rank t / T_loc, expert e on rank e / (E / P).
//   all_idx, all_w   [T, k]        every rank's routing results, written by their route kernels
//   slot[d][t]                     position of token t among the tokens that have an expert on rank d
//                                  (in token order), -1 if it has none; tok_of_slot[d][s] the inverse
//   tokbuf           [T, H] bf16   on rank d: row slot[d][t] = hidden vector of token t
//   rows             per rank the usual permuted, 128-padded expert rows; the quantiser gathers row r
//                    from tokbuf[slot[me][pair_of_row[r] / k]]
//                    With scale_mode 2 the tokens cross as fp8: the source quantises every token per 128
//                    channels with a power-of-two scale (1x128 scales, one e8m0 byte each) and sends
//                    H + H/128 bytes instead of 2H; tokbuf then holds [T, H] e4m3 followed by
//                    [T, sb] scale bytes (sb = H/128 rounded up to 16), and the receiving side only
//                    gathers bytes into expert order and lays the rows' scale bytes out as the atoms
//                    the block-scaled tensor-core path reads (they are per row by construction).
//   partial[d]       [T_loc, H] bf16 on the home rank: sum over the token's experts on rank d of
//                    w * y, formed in fp32 on rank d; the home rank adds the partials in rank order
#include <algorithm>

#include <cuda_fp8.h>

#include "dk_moe_int.h"

namespace dk {

constexpr int EP_CHUNK = 1024;  // tokens per block in the slot kernels, one per thread
enum : unsigned { SITE_EP_EXPERT = 91 };

// Byte offsets of the regions inside the workspace; identical on every rank.
struct EpLayout {
    size_t all_idx, all_w, tokbuf, partial;                       // written by peers
    size_t rop, por, offsets, counts, scratch, slot, tos, ntok, chunk_cnt;  // local index data
    size_t xq, xs, hq, hs, he, y;                                 // local activations
    size_t total;
    int T, cap, epr, nchunks;
};

static size_t up256(size_t v) { return (v + 255) / 256 * 256; }

static EpLayout ep_layout(int T_loc, int k, int E, int H, int F, int world) {
    EpLayout L{};
    L.T = T_loc * world;
    L.epr = E / world;
    L.cap = static_cast<int>(dk_moe_rows_capacity(L.T, k, L.epr, 128));
    L.nchunks = (L.T + EP_CHUNK - 1) / EP_CHUNK;
    const size_t T = L.T, cap = L.cap;
    size_t o = 0;
    auto take = [&](size_t bytes) {
        const size_t at = o;
        o += up256(bytes);
        return at;
    };
    L.all_idx = take(T * k * 4);
    L.all_w = take(T * k * 4);
    L.tokbuf = take(T * H * 2);
    L.partial = take(static_cast<size_t>(world) * T_loc * H * 2);
    L.rop = take(T * k * 4);
    L.por = take(static_cast<size_t>(world) * cap * 4);
    L.offsets = take(static_cast<size_t>(world) * (L.epr + 1) * 4);
    L.counts = take(static_cast<size_t>(E) * 4);
    L.scratch = take(dk_moe_permute_scratch_bytes(L.T, k, E));
    L.slot = take(static_cast<size_t>(world) * T * 4);
    L.tos = take(static_cast<size_t>(world) * T * 4);
    L.ntok = take(static_cast<size_t>(world) * 4);
    L.chunk_cnt = take(static_cast<size_t>(L.nchunks) * DK_MAX_RANKS * 4);
    L.xq = take(cap * H);
    // scales: fp32 per 128x128 block, or block atoms (512 bytes per 128 rows x 512 columns); take the larger
    const size_t xs_f32 = (cap / 128) * (static_cast<size_t>(H) / 128) * 4;
    const size_t xs_atoms = (cap / 128) * ((static_cast<size_t>(H) / 128 + 3) / 4) * 512;
    L.xs = take(xs_f32 > xs_atoms ? xs_f32 : xs_atoms);
    L.hq = take(cap * F);
    const size_t hs_f32 = (cap / 128) * (static_cast<size_t>(F) / 128) * 4;
    const size_t hs_atoms = (cap / 128) * ((static_cast<size_t>(F) / 128 + 3) / 4) * 512;
    L.hs = take(hs_f32 > hs_atoms ? hs_f32 : hs_atoms);
    L.he = take((cap / 128) * (static_cast<size_t>(F) / 128));
    L.y = take(cap * H * 2);
    L.total = o;
    return L;
}

// Destination ranks of a token as a bit mask; an expert id no rank holds is left out (and recorded).
__device__ __forceinline__ unsigned dest_mask(const int* idx, int k, int epr, int world, unsigned* status,
                                              int token) {
    unsigned m = 0;
    for (int j = 0; j < k; ++j) {
        const int e = idx[j];
        const int d = e >= 0 ? e / epr : -1;
        if (d >= 0 && d < world) m |= 1u << d;
        else record_bad_index(status, SITE_EP_EXPERT, static_cast<unsigned>(token * k + j));
    }
    return m;
}

// ---- token slots: slot[d][t] = number of tokens t' < t with an expert on rank d (or -1)
// Pass 1: per chunk of 1024 tokens and per destination, how many tokens go there.
__global__ void __launch_bounds__(EP_CHUNK) ep_tokcount_kernel(const int* __restrict__ all_idx, int T, int k,
                                                               int epr, int world, int* __restrict__ chunk_cnt,
                                                               unsigned* status) {
    __shared__ int cnt[DK_MAX_RANKS];
    if (threadIdx.x < DK_MAX_RANKS) cnt[threadIdx.x] = 0;
    __syncthreads();
    const int t = blockIdx.x * EP_CHUNK + threadIdx.x;
    const unsigned m = t < T ? dest_mask(all_idx + static_cast<size_t>(t) * k, k, epr, world, status, t) : 0u;
    for (int d = 0; d < world; ++d) {
        const unsigned b = __ballot_sync(0xffffffffu, (m >> d) & 1u);
        if ((threadIdx.x & 31) == 0 && b) atomicAdd(&cnt[d], __popc(b));  // a count: order-independent
    }
    __syncthreads();
    if (threadIdx.x < DK_MAX_RANKS) chunk_cnt[blockIdx.x * DK_MAX_RANKS + threadIdx.x] = cnt[threadIdx.x];
}

// Pass 2: slot = tokens to d in earlier chunks + in earlier warps of this chunk + in earlier lanes.
__global__ void __launch_bounds__(EP_CHUNK) ep_tokslot_kernel(const int* __restrict__ all_idx, int T, int k, int epr,
                                                              int world, const int* __restrict__ chunk_cnt,
                                                              int* __restrict__ slot, int* __restrict__ tok_of_slot,
                                                              int* __restrict__ ntok) {
    __shared__ int warp_cnt[EP_CHUNK / 32][DK_MAX_RANKS];
    __shared__ int base[DK_MAX_RANKS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x < world) {
        int run = 0;
        for (int c = 0; c < static_cast<int>(blockIdx.x); ++c) run += chunk_cnt[c * DK_MAX_RANKS + threadIdx.x];
        base[threadIdx.x] = run;
        if (blockIdx.x == gridDim.x - 1) ntok[threadIdx.x] = run + chunk_cnt[blockIdx.x * DK_MAX_RANKS + threadIdx.x];
    }
    const int t = blockIdx.x * EP_CHUNK + threadIdx.x;
    const unsigned m = t < T ? dest_mask(all_idx + static_cast<size_t>(t) * k, k, epr, world, nullptr, t) : 0u;
    unsigned before_in_warp[DK_MAX_RANKS];
#pragma unroll
    for (int d = 0; d < DK_MAX_RANKS; ++d) {
        const unsigned b = d < world ? __ballot_sync(0xffffffffu, (m >> d) & 1u) : 0u;
        before_in_warp[d] = __popc(b & ((1u << lane) - 1u));
        if (lane == 0) warp_cnt[warp][d] = __popc(b);
    }
    __syncthreads();
    if (t < T) {
#pragma unroll
        for (int d = 0; d < DK_MAX_RANKS; ++d) {
            if (d >= world) break;
            int s = -1;
            if ((m >> d) & 1u) {
                s = base[d] + static_cast<int>(before_in_warp[d]);
                for (int w = 0; w < warp; ++w) s += warp_cnt[w][d];
                tok_of_slot[static_cast<size_t>(d) * T + s] = t;
            }
            slot[static_cast<size_t>(d) * T + t] = s;
        }
    }
}

// ---- dispatch: every local token goes ONCE to each rank that holds at least one of its experts
struct EpDispatchArgs {
    const uint4* x;                  // [T_loc, H/8] local tokens
    const int* all_idx;              // [T, k]
    const int* slot;                 // [P][T]
    uint4* tokbuf[DK_MAX_RANKS];     // token buffer of rank d as seen from here, [T, H/8]
    int T, T_loc, k, hvec, epr, world, rank;
    EpSignal sig;
};
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const EpDispatchArgs a) {
    __shared__ int slot_s[DK_MAX_RANKS];
    for (int tl = blockIdx.x; tl < a.T_loc; tl += gridDim.x) {
        const int t = a.rank * a.T_loc + tl;
        __syncthreads();  // the previous token's slots have been used
        if (threadIdx.x < a.world)
            slot_s[threadIdx.x] = a.slot[static_cast<size_t>(threadIdx.x) * a.T + t];  // -1: nothing to send there
        __syncthreads();
        for (int c = threadIdx.x; c < a.hvec; c += blockDim.x) {
            const uint4 v = a.x[static_cast<size_t>(tl) * a.hvec + c];
#pragma unroll
            for (int d = 0; d < DK_MAX_RANKS; ++d)
                if (d < a.world && slot_s[d] >= 0) a.tokbuf[d][static_cast<size_t>(slot_s[d]) * a.hvec + c] = v;
        }
    }
    ep_signal_done(a.sig);
}

// ---- dispatch as fp8 (scale_mode 2): the token is quantised here, once, per 128 channels with a
// power-of-two scale (the rule of the 128x128 quantiser applied to a 1x128 group: s =
// 2^ceil(log2(amax/448)), 1 for zeros), and its H e4m3 bytes + H/128 scale bytes go to each rank that
// holds one of its experts. Thread c owns 16 channels; eight neighbouring lanes own one group.
struct EpDispatchQArgs {
    const uint4* x;                  // [T_loc, H/8] local tokens (bf16)
    const int* slot;                 // [P][T]
    uint8_t* tokq[DK_MAX_RANKS];     // [T, H] e4m3 at rank d
    uint8_t* toks[DK_MAX_RANKS];     // [T, sb] e8m0 at rank d
    int T, T_loc, H, sb, world, rank;
    EpSignal sig;
};
constexpr int EP_MAX_SB = 256;  // scale bytes per token the kernels hold in shared memory (H <= 32768)

__global__ void __launch_bounds__(256) ep_dispatch_q_kernel(const EpDispatchQArgs a) {
    __shared__ int slot_s[DK_MAX_RANKS];
    __shared__ __align__(16) uint8_t sc_s[EP_MAX_SB];
    const int nvec = a.H / 16;
    for (int tl = blockIdx.x; tl < a.T_loc; tl += gridDim.x) {
        const int t = a.rank * a.T_loc + tl;
        __syncthreads();  // the previous token's slots and scale bytes have been used
        if (threadIdx.x < a.world) slot_s[threadIdx.x] = a.slot[static_cast<size_t>(threadIdx.x) * a.T + t];
        for (int i = threadIdx.x; i < a.sb; i += blockDim.x) sc_s[i] = 127;  // bytes past H/128: scale 1
        __syncthreads();
        for (int c0 = 0; c0 < nvec; c0 += blockDim.x) {  // uniform trip count: the shuffles need whole warps
            const int c = c0 + threadIdx.x;
            const bool live = c < nvec;
            uint4 u[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
            if (live) {
                u[0] = a.x[static_cast<size_t>(tl) * (a.H / 8) + 2 * c];
                u[1] = a.x[static_cast<size_t>(tl) * (a.H / 8) + 2 * c + 1];
            }
            __nv_bfloat162 m2 = __float2bfloat162_rn(0.f);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u[i]);
#pragma unroll
                for (int j = 0; j < 4; ++j) m2 = __hmax2(m2, __habs2(h[j]));
            }
            float amax = fmaxf(__low2float(m2), __high2float(m2));
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            int ex = 0;
            if (amax > 0.f) {
                const float m = frexpf(amax / 448.0f, &ex);
                if (m == 0.5f) ex -= 1;
                ex = max(-127, min(127, ex));
            }
            const float inv = ldexpf(1.0f, -ex);
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u[i]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(h[j]);
                    const uint32_t p2 = __nv_cvt_float2_to_fp8x2(make_float2(f.x * inv, f.y * inv), __NV_SATFINITE, __NV_E4M3);
                    if (j & 1) w[2 * i + (j >> 1)] |= p2 << 16;
                    else w[2 * i + (j >> 1)] = p2;
                }
            }
            if (live) {
                const uint4 qv = make_uint4(w[0], w[1], w[2], w[3]);
#pragma unroll
                for (int d = 0; d < DK_MAX_RANKS; ++d)
                    if (d < a.world && slot_s[d] >= 0)
                        *reinterpret_cast<uint4*>(a.tokq[d] + static_cast<size_t>(slot_s[d]) * a.H + static_cast<size_t>(c) * 16) = qv;
                if ((threadIdx.x & 7) == 0) sc_s[c >> 3] = static_cast<uint8_t>(ex + 127);
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < a.sb / 16; i += blockDim.x) {
            const uint4 v = reinterpret_cast<const uint4*>(sc_s)[i];
#pragma unroll
            for (int d = 0; d < DK_MAX_RANKS; ++d)
                if (d < a.world && slot_s[d] >= 0)
                    *reinterpret_cast<uint4*>(a.toks[d] + static_cast<size_t>(slot_s[d]) * a.sb + i * 16) = v;
        }
    }
    ep_signal_done(a.sig);
}

// ---- the receiving side of the fp8 dispatch: expert row r takes the bytes of the token it belongs to
// (zeros for padding rows), and the row's scale bytes go into the scale atoms of its 128-row block:
// per four column blocks one 512-byte atom, in which row slot i = 32*i1 + i0 owns the four bytes at
// i0*16 + i1*4 (the order in which the tensor core's scale copy spreads an atom over its 128 lanes).
// One warp per row.
struct EpGatherQArgs {
    const uint8_t* tokq;             // [T, H]
    const uint8_t* toks;             // [T, sb]
    const int* por;                  // [cap] pair of every row, -1 = padding
    const int* slot;                 // [T] slot of every token on this rank
    const int* row_limit;            // rows at or beyond *row_limit are not produced
    uint8_t* xq;                     // [cap, H]
    uint8_t* atoms;                  // [cap/128][ceil(H/512)][512]
    int cap, H, sb, k;
    EpWait wait;
};
__global__ void __launch_bounds__(256) ep_gather_q_kernel(const EpGatherQArgs a) {
    const int rows = min(*a.row_limit, a.cap);
    if (static_cast<int>(blockIdx.x) * 8 >= rows) return;
    if (!ep_wait_sources(a.wait)) return;
    const int lane = threadIdx.x & 31;
    // grid-stride over the rows that exist (a CTA per eight rows of the capacity would mostly launch
    // CTAs that exit)
    for (int r = blockIdx.x * 8 + (threadIdx.x >> 5); r < rows; r += gridDim.x * 8) {
    const int pair = a.por[r];
    const int src = pair >= 0 ? a.slot[pair / a.k] : -1;
    const int nvec = a.H / 16;
    const uint4* from = reinterpret_cast<const uint4*>(a.tokq + static_cast<size_t>(src < 0 ? 0 : src) * a.H);
    uint4* to = reinterpret_cast<uint4*>(a.xq + static_cast<size_t>(r) * a.H);
    for (int c = lane; c < nvec; c += 32 * 4) {  // four loads in flight per lane
        uint4 v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            v[i] = (src >= 0 && c + 32 * i < nvec) ? __ldcg(from + c + 32 * i) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (c + 32 * i < nvec) to[c + 32 * i] = v[i];
    }
    const int nj = (a.H / 128 + 3) / 4;
    const int i = r & 127;
    uint8_t* atom_row = a.atoms + static_cast<size_t>(r >> 7) * nj * 512 + (i & 31) * 16 + (i >> 5) * 4;
    const uint32_t* sc = reinterpret_cast<const uint32_t*>(a.toks + static_cast<size_t>(src < 0 ? 0 : src) * a.sb);
    for (int j = lane; j < nj; j += 32)
        *reinterpret_cast<uint32_t*>(atom_row + static_cast<size_t>(j) * 512) = src >= 0 ? __ldcg(sc + j) : 0x7f7f7f7fu;
    }  // rows of this warp
}

// ---- expert-side combine: for every token that arrived here, the weighted sum of the outputs of its
// experts on THIS rank, in fp32, pushed as one bf16 vector to the token's home rank.
struct EpCombineArgs {
    const uint4* y;                  // [cap, H/8] expert outputs of this rank
    const int* all_idx;              // [T, k]
    const float* all_w;              // [T, k]
    const int* rop;                  // [T, k] row of every pair inside its destination rank
    const int* tok_of_slot;          // [T] for this rank
    const int* ntok;                 // [1] tokens that arrived here
    uint4* partial[DK_MAX_RANKS];    // at home rank h: partial[this rank] as [T_loc, H/8]
    int T_loc, k, hvec, epr, rank;
    EpSignal sig;
};
// One warp per token (eight tokens per CTA at a time, no CTA-wide barrier per token): lanes < k fetch
// the token's pairs, the warp shares them by shuffle, then every lane sums its 16-byte columns with
// the rows of two column steps requested before the first is used.
__global__ void __launch_bounds__(256) ep_combine_push_kernel(const EpCombineArgs a) {
    const int n = *a.ntok;
    const int lane = threadIdx.x & 31;
    const int nwarps = gridDim.x * (blockDim.x >> 5);
    for (int s = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); s < n; s += nwarps) {
        const int t = a.tok_of_slot[s];
        int my_row = -1;
        float my_w = 0.f;
        if (lane < a.k) {
            const size_t at = static_cast<size_t>(t) * a.k + lane;
            const int e = a.all_idx[at];
            const bool here = e >= 0 && e / a.epr == a.rank;
            my_row = here ? a.rop[at] : -1;   // -1 also for a pair the permutation left out
            my_w = a.all_w[at];
        }
        int row[8];
        float wt[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            row[j] = __shfl_sync(0xffffffffu, my_row, j);
            wt[j] = __shfl_sync(0xffffffffu, my_w, j);
        }
        const int home = t / a.T_loc;
        uint4* dst = a.partial[home] + static_cast<size_t>(t - home * a.T_loc) * a.hvec;
        for (int c0 = lane; c0 < a.hvec; c0 += 64) {
            uint4 v[2][8];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int c = c0 + 32 * u;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    v[u][j] = (c < a.hvec && row[j] >= 0) ? a.y[static_cast<size_t>(row[j]) * a.hvec + c]
                                                          : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int c = c0 + 32 * u;
                if (c >= a.hvec) break;
                float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (row[j] >= 0) {
                        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u][j]);
                        const float wj = wt[j];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float2 f = __bfloat1622float2(h[i]);
                            acc[2 * i] += wj * f.x;
                            acc[2 * i + 1] += wj * f.y;
                        }
                    }
                }
                uint4 o;
                o.x = pack_bf16x2(acc[0], acc[1]);
                o.y = pack_bf16x2(acc[2], acc[3]);
                o.z = pack_bf16x2(acc[4], acc[5]);
                o.w = pack_bf16x2(acc[6], acc[7]);
                dst[c] = o;
            }
        }
    }
    ep_signal_done(a.sig);
}

// ---- final: out[t] = sum over the ranks the token was sent to, in rank order, of their partials
struct EpFinalArgs {
    const uint4* partial;            // [P][T_loc, H/8] on this rank
    const int* slot;                 // [P][T]
    uint4* out;                      // [T_loc, H/8]
    int T, T_loc, hvec, world, rank;
    EpWait wait;
};
__global__ void __launch_bounds__(256) ep_final_kernel(const EpFinalArgs a) {
    if (!ep_wait_sources(a.wait)) return;
    const int lane = threadIdx.x & 31;
    const int nwarps = gridDim.x * (blockDim.x >> 5);
    // one warp per token
    for (int tl = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); tl < a.T_loc; tl += nwarps) {
        const int t = a.rank * a.T_loc + tl;
        const bool mine = lane < a.world && a.slot[static_cast<size_t>(lane) * a.T + t] >= 0;
        const unsigned has = __ballot_sync(0xffffffffu, mine);  // ranks the token was sent to
        for (int c0 = lane; c0 < a.hvec; c0 += 64) {
            uint4 v[2][DK_MAX_RANKS];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int c = c0 + 32 * u;
#pragma unroll
                for (int d = 0; d < DK_MAX_RANKS; ++d)
                    // written by rank d during this call: read past L1
                    v[u][d] = (c < a.hvec && ((has >> d) & 1u))
                                  ? __ldcg(a.partial + (static_cast<size_t>(d) * a.T_loc + tl) * a.hvec + c)
                                  : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int c = c0 + 32 * u;
                if (c >= a.hvec) break;
                float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
                for (int d = 0; d < DK_MAX_RANKS; ++d) {
                    if ((has >> d) & 1u) {
                        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u][d]);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float2 f = __bfloat1622float2(h[i]);
                            acc[2 * i] += f.x;
                            acc[2 * i + 1] += f.y;
                        }
                    }
                }
                uint4 o;
                o.x = pack_bf16x2(acc[0], acc[1]);
                o.y = pack_bf16x2(acc[2], acc[3]);
                o.z = pack_bf16x2(acc[4], acc[5]);
                o.w = pack_bf16x2(acc[6], acc[7]);
                a.out[static_cast<size_t>(tl) * a.hvec + c] = o;
            }
        }
    }
}

// control-block words (inside DK_CTRL_MOE; the peer barrier uses words 0..7 of that region)
constexpr size_t EP_FLAG_BASE = DK_CTRL_MOE + 64;     // flags [3 phases][8 sources]
constexpr size_t EP_COUNTER_BASE = DK_CTRL_MOE + 128;  // CTA counters [3 phases], local use only
// Calls whose number lives on the device (DK_EPOCH_DEVICE) have flags of their own, so that they can be
// mixed with host-numbered calls on one heap, and the word that counts them.
constexpr size_t EP_DEV_FLAG_BASE = DK_CTRL_MOE + 192;
constexpr size_t EP_DEV_EPOCH = DK_CTRL_MOE + 256;
enum : int { EP_PH_ROUTE = 0, EP_PH_DISPATCH = 1, EP_PH_COMBINE = 2 };

static EpSignal make_signal(const dk_view* v, int phase, unsigned epoch) {
    EpSignal s{};
    if (v->world <= 1) return s;
    const bool dev = epoch == DK_EPOCH_DEVICE;
    const size_t base = dev ? EP_DEV_FLAG_BASE : EP_FLAG_BASE;
    s.counter = ctrl_words(v, v->rank) + EP_COUNTER_BASE + phase;
    for (int r = 0; r < v->world; ++r) s.flag[r] = ctrl_words(v, r) + base + phase * DK_MAX_RANKS + v->rank;
    s.world = v->world;
    s.epoch = epoch;
    s.epoch_ptr = dev ? ctrl_words(v, v->rank) + EP_DEV_EPOCH : nullptr;
    return s;
}
static int make_wait(const dk_view* v, int phase, unsigned epoch, EpWait* w) {
    *w = EpWait{};
    if (v->world <= 1) return DK_OK;
    const bool dev = epoch == DK_EPOCH_DEVICE;
    w->flags = ctrl_words(v, v->rank) + (dev ? EP_DEV_FLAG_BASE : EP_FLAG_BASE) + phase * DK_MAX_RANKS;
    w->world = v->world;
    w->epoch = epoch;
    w->epoch_ptr = dev ? ctrl_words(v, v->rank) + EP_DEV_EPOCH : nullptr;
    w->limit_ns = peer_wait_ns();
    return device_status_ptr(&w->status);
}

// the last launch of a device-numbered call: the next call is one later
__global__ void ep_epoch_advance_kernel(unsigned* word) { *word += 1u; }

}  // namespace dk

extern "C" {

size_t dk_moe_ep_workspace_bytes(int T_loc, int k, int E, int H, int F, int world) {
    if (T_loc <= 0 || k < 1 || k > 8 || E < 1 || world < 1 || world > DK_MAX_RANKS || E % world != 0 || H <= 0 ||
        F <= 0 || H % 128 != 0 || F % 128 != 0)
        return 0;
    return dk::ep_layout(T_loc, k, E, H, F, world).total;
}

int dk_moe_ep_layer(const dk_moe_ep_args* a, const dk_view* view, unsigned epoch, int phases, void* stream) {
    using namespace dk;
    DK_REQUIRE(a != nullptr, "null arguments");
    dk_view one{};
    if (view == nullptr) {  // single GPU: a view of one rank without a heap
        one.world = 1;
        view = &one;
    }
    const int world = view->world, rank = view->rank;
    DK_REQUIRE(world >= 1 && world <= DK_MAX_RANKS && rank >= 0 && rank < world, "bad view");
    DK_REQUIRE(a->T_loc > 0 && a->k >= 1 && a->k <= 8, "T_loc must be positive and k 1..8");
    DK_REQUIRE(a->E >= 1 && a->E <= 256 && a->E % world == 0 && a->k <= a->E, "E must be 1..256, a multiple of world, >= k");
    DK_REQUIRE(a->H > 0 && a->H % 256 == 0 && a->F > 0 && a->F % 128 == 0,
               "H must be a multiple of 256 and F a multiple of 128");
    DK_REQUIRE(a->scale_mode >= 0 && a->scale_mode <= 2,
               "scale_mode must be 0 (fp32 scales), 1 (power-of-two) or 2 (power-of-two, tokens dispatched as fp8)");
    DK_REQUIRE(a->scale_mode != 2 || a->H / 128 <= EP_MAX_SB, "H too large for the fp8 dispatch");
    DK_REQUIRE(phases >= 1 && phases <= 15, "phases is a mask of 1 | 2 | 4 | 8");
    DK_REQUIRE(a->x && a->logits && a->w13q && a->w13s && a->w2q && a->w2s && a->out && a->workspace, "null buffer");
    DK_REQUIRE((reinterpret_cast<uintptr_t>(a->workspace) & 255) == 0, "the workspace must be 256-byte aligned");
    const EpLayout L = ep_layout(a->T_loc, a->k, a->E, a->H, a->F, world);
    if (world > 1) {
        DK_REQUIRE(in_heap(view, a->workspace, L.total), "the workspace must lie inside the symmetric heap");
        if (const int pending = device_status_pending()) return pending;
        if (epoch == 0) {
            DK_REQUIRE(view->heap != nullptr, "view has no heap handle: pass an explicit epoch");
            epoch = heap_next_epoch(static_cast<dk_heap*>(view->heap));
        }
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char* ws = static_cast<char*>(a->workspace);
    auto at = [&](size_t off) { return ws + off; };
    auto peer = [&](size_t off, int r) {
        return world > 1 ? static_cast<char*>(peer_ptr(view, ws + off, r)) : ws + off;
    };
    const int T = L.T, k = a->k, E = a->E, H = a->H, F = a->F, epr = L.epr, cap = L.cap;
    const int sb = (H / 128 + 15) / 16 * 16;  // scale bytes per token of the fp8 dispatch
    int* all_idx = reinterpret_cast<int*>(at(L.all_idx));
    float* all_w = reinterpret_cast<float*>(at(L.all_w));
    int* rop = reinterpret_cast<int*>(at(L.rop));
    int* por = reinterpret_cast<int*>(at(L.por));
    int* offsets = reinterpret_cast<int*>(at(L.offsets));
    int* counts = reinterpret_cast<int*>(at(L.counts));
    int* slot = reinterpret_cast<int*>(at(L.slot));
    int* tos = reinterpret_cast<int*>(at(L.tos));
    int* ntok = reinterpret_cast<int*>(at(L.ntok));
    int* chunk_cnt = reinterpret_cast<int*>(at(L.chunk_cnt));
    int* my_offsets = offsets + static_cast<size_t>(rank) * (epr + 1);
    int sms = 0;
    int rc = sm_count(&sms);
    if (rc != DK_OK) return rc;
    unsigned* status = nullptr;
    rc = device_status_ptr(&status);
    if (rc != DK_OK) return rc;

    if (phases & 1) {
        // routing of the local tokens, written into every rank's table
        RouteOut ro{};
        for (int r = 0; r < world; ++r) {
            ro.idx[r] = reinterpret_cast<int*>(peer(L.all_idx, r));
            ro.w[r] = reinterpret_cast<float*>(peer(L.all_w, r));
        }
        ro.n_out = world;
        ro.row_base = rank * a->T_loc;
        rc = moe_route_launch(a->logits, a->T_loc, E, k, ro, make_signal(view, EP_PH_ROUTE, epoch), st);
        if (rc != DK_OK) return rc;
    }
    if (phases & 2) {
        EpWait w;
        rc = make_wait(view, EP_PH_ROUTE, epoch, &w);
        if (rc != DK_OK) return rc;
        rc = moe_permute_launch(all_idx, T, k, E, 128, epr, rop, por, cap, offsets, counts,
                                reinterpret_cast<int*>(at(L.scratch)), w, st);
        if (rc != DK_OK) return rc;
        ep_tokcount_kernel<<<L.nchunks, EP_CHUNK, 0, st>>>(all_idx, T, k, epr, world, chunk_cnt, status);
        DK_CUDA_OK(cudaGetLastError());
        ep_tokslot_kernel<<<L.nchunks, EP_CHUNK, 0, st>>>(all_idx, T, k, epr, world, chunk_cnt, slot, tos, ntok);
        DK_CUDA_OK(cudaGetLastError());
        // (one rank: nothing to send; the quantiser gathers straight from x)
        EpDispatchArgs d{};
        d.x = static_cast<const uint4*>(a->x);
        d.all_idx = all_idx;
        d.slot = slot;
        for (int r = 0; r < world; ++r) d.tokbuf[r] = reinterpret_cast<uint4*>(peer(L.tokbuf, r));
        d.T = T;
        d.T_loc = a->T_loc;
        d.k = k;
        d.hvec = H / 8;
        d.epr = epr;
        d.world = world;
        d.rank = rank;
        d.sig = make_signal(view, EP_PH_DISPATCH, epoch);
        const int grid = a->T_loc < 4 * sms ? a->T_loc : 4 * sms;
        if (a->scale_mode == 2) {
            // quantise at the source, send fp8 (one rank: the same kernel fills the local buffer)
            EpDispatchQArgs dq{};
            dq.x = d.x;
            dq.slot = slot;
            for (int r = 0; r < world; ++r) {
                dq.tokq[r] = reinterpret_cast<uint8_t*>(peer(L.tokbuf, r));
                dq.toks[r] = dq.tokq[r] + static_cast<size_t>(T) * H;
            }
            dq.T = T;
            dq.T_loc = a->T_loc;
            dq.H = H;
            dq.sb = sb;
            dq.world = world;
            dq.rank = rank;
            dq.sig = d.sig;
            ep_dispatch_q_kernel<<<grid, 256, 0, st>>>(dq);
            DK_CUDA_OK(cudaGetLastError());
        } else if (world > 1) {
            ep_dispatch_kernel<<<grid, 256, 0, st>>>(d);
            DK_CUDA_OK(cudaGetLastError());
        }
        if (a->counts_out != nullptr)
            DK_CUDA_OK(cudaMemcpyAsync(a->counts_out, counts + static_cast<size_t>(rank) * epr, epr * sizeof(int),
                                       cudaMemcpyDeviceToDevice, st));
    }
    if (phases & 4) {
        EpWait w;
        rc = make_wait(view, EP_PH_DISPATCH, epoch, &w);
        if (rc != DK_OK) return rc;
        // rows of this rank's experts, gathered from the token buffer and quantised; only the rows
        // that exist (offsets[E/P], read on the device) are produced
        const bool pow2 = a->scale_mode != 0;
        if (a->scale_mode == 2) {
            EpGatherQArgs g{};
            g.tokq = reinterpret_cast<const uint8_t*>(at(L.tokbuf));
            g.toks = g.tokq + static_cast<size_t>(T) * H;
            g.por = por + static_cast<size_t>(rank) * cap;
            g.slot = slot + static_cast<size_t>(rank) * T;
            g.row_limit = my_offsets + epr;
            g.xq = reinterpret_cast<uint8_t*>(at(L.xq));
            g.atoms = reinterpret_cast<uint8_t*>(at(L.xs));
            g.cap = cap;
            g.H = H;
            g.sb = sb;
            g.k = k;
            g.wait = w;
            ep_gather_q_kernel<<<std::min((cap + 7) / 8, 16 * sms), 256, 0, st>>>(g);
            DK_CUDA_OK(cudaGetLastError());
        } else {
            rc = quant_block128_launch(world > 1 ? at(L.tokbuf) : a->x, cap, H, por + static_cast<size_t>(rank) * cap,
                                       world > 1 ? 3 : 1, k, slot + static_cast<size_t>(rank) * T, my_offsets + epr,
                                       at(L.xq), pow2 ? nullptr : reinterpret_cast<float*>(at(L.xs)), nullptr,
                                       pow2 ? at(L.xs) : nullptr, pow2, w, st);
            if (rc != DK_OK) return rc;
        }
        if (a->ev_gemm_begin != nullptr) DK_CUDA_OK(cudaEventRecord(static_cast<cudaEvent_t>(a->ev_gemm_begin), st));
        if (pow2) {
            rc = dk_moe_grouped_gemm_mxfp8(at(L.xq), at(L.xs), a->w13q, a->w13s, my_offsets, epr, cap, F, H, 1,
                                           at(L.hq), at(L.he), at(L.hs), st);
            if (rc != DK_OK) return rc;
            rc = dk_moe_grouped_gemm_mxfp8(at(L.hq), at(L.hs), a->w2q, a->w2s, my_offsets, epr, cap, H, F, 0,
                                           at(L.y), nullptr, nullptr, st);
        } else {
            rc = dk_moe_grouped_gemm_fp8(at(L.xq), reinterpret_cast<const float*>(at(L.xs)), a->w13q,
                                         static_cast<const float*>(a->w13s), my_offsets, epr, cap, F, H, 1, at(L.hq),
                                         reinterpret_cast<float*>(at(L.hs)), st);
            if (rc != DK_OK) return rc;
            rc = dk_moe_grouped_gemm_fp8(at(L.hq), reinterpret_cast<const float*>(at(L.hs)), a->w2q,
                                         static_cast<const float*>(a->w2s), my_offsets, epr, cap, H, F, 0, at(L.y),
                                         nullptr, st);
        }
        if (rc != DK_OK) return rc;
        if (a->ev_gemm_end != nullptr) DK_CUDA_OK(cudaEventRecord(static_cast<cudaEvent_t>(a->ev_gemm_end), st));
        EpCombineArgs c{};
        c.y = reinterpret_cast<const uint4*>(at(L.y));
        c.all_idx = all_idx;
        c.all_w = all_w;
        c.rop = rop;
        c.tok_of_slot = tos + static_cast<size_t>(rank) * T;
        c.ntok = ntok + rank;
        for (int h = 0; h < world; ++h)
            c.partial[h] = reinterpret_cast<uint4*>(peer(L.partial, h)) + static_cast<size_t>(rank) * a->T_loc * (H / 8);
        c.T_loc = a->T_loc;
        c.k = k;
        c.hvec = H / 8;
        c.epr = epr;
        c.rank = rank;
        c.sig = make_signal(view, EP_PH_COMBINE, epoch);
        ep_combine_push_kernel<<<4 * sms, 256, 0, st>>>(c);
        DK_CUDA_OK(cudaGetLastError());
    }
    if (phases & 8) {
        EpFinalArgs f{};
        f.partial = reinterpret_cast<const uint4*>(at(L.partial));
        f.slot = slot;
        f.out = static_cast<uint4*>(a->out);
        f.T = T;
        f.T_loc = a->T_loc;
        f.hvec = H / 8;
        f.world = world;
        f.rank = rank;
        rc = make_wait(view, EP_PH_COMBINE, epoch, &f.wait);
        if (rc != DK_OK) return rc;
        const int grid = std::min((a->T_loc + 7) / 8, 4 * sms);  // a warp per token
        ep_final_kernel<<<grid, 256, 0, st>>>(f);
        DK_CUDA_OK(cudaGetLastError());
        if (world > 1 && epoch == DK_EPOCH_DEVICE) {
            ep_epoch_advance_kernel<<<1, 1, 0, st>>>(ctrl_words(view, rank) + EP_DEV_EPOCH);
            DK_CUDA_OK(cudaGetLastError());
        }
    }
    return DK_OK;
}

}  // extern "C"
