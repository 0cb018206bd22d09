// MoE routing, permutation, 128x128 block quantisation to e4m3, and combine: the HBM-bound
// integer/byte kernels around the fp8 grouped GEMM.
//
// The reference has no MoE code. The nearest patterns it holds are the block-scaled fp8 fixtures
// (tests/unit/cdna4/warp/register/tile/mma_scaled.cu:200-258: quantise, CPU truth dequantises per
// block), whose scale format (1x32 e8m0) differs from the 128x128 fp32 blocks used here.
//
// Everything index-like is deterministic and order-preserving (scans, no atomics whose order
// could leak into the result), so it is bit-exact against the CPU definition:
//   route     top-k on the raw fp32 logits, ties to the lower expert index, output in descending
//             logit order; weights = softmax over all experts gathered and renormalised
//   permute   pairs (token, slot) grouped by expert, each expert padded to `pad` rows; inside an
//             expert, pairs keep their (token, slot) order
//   quant     per 128x128 block s = amax/448 (1 when the block is all zero), q = RNE(x / s)
//   combine   out[t] = sum_j w[t,j] * Y[row(t,j)] in fp32, slot order
#include <cuda_fp8.h>

#include <mutex>
#include <string>

#include <algorithm>

#include "dk_moe_int.h"

namespace dk {

// ------------------------------------------------------------------------------------ route
constexpr int ROUTE_MAX_E = 256;
constexpr int ROUTE_MAX_K = 8;

// One warp per token. Lane l holds experts l, l+32, ... (E <= 256 -> at most 8 per lane).
__global__ void __launch_bounds__(256) moe_route_kernel(const float* __restrict__ logits, int T, int E,
                                                        int k, const RouteOut out, const EpSignal sig) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp < T) {
    const float* row = logits + static_cast<size_t>(warp) * E;
    float v[ROUTE_MAX_E / 32];
    bool taken[ROUTE_MAX_E / 32];
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_E / 32; ++i) {
        const int e = lane + 32 * i;
        v[i] = e < E ? row[e] : -INFINITY;
        taken[i] = e >= E;
    }
    // lane j keeps the j-th selection (no dynamically indexed arrays, and the results are written by
    // k lanes at once instead of one lane after the other)
    float my_v = -INFINITY, top_v = 0.f;
    int my_e = 0;
#pragma unroll 1
    for (int j = 0; j < k; ++j) {
        // best of this lane: largest value, lowest index among equals (ascending scan, strict >)
        float bv = -INFINITY;
        int be = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < ROUTE_MAX_E / 32; ++i) {
            const int e = lane + 32 * i;
            if (!taken[i] && (be == 0x7fffffff || v[i] > bv)) {
                bv = v[i];
                be = e;
            }
        }
        // warp arg-max with the same tie rule
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            const bool other_valid = oe != 0x7fffffff;
            const bool mine_valid = be != 0x7fffffff;
            if (other_valid && (!mine_valid || ov > bv || (ov == bv && oe < be))) {
                bv = ov;
                be = oe;
            }
        }
        if (j == 0) top_v = bv;
        if (lane == j) {
            my_v = bv;
            my_e = be;
        }
        if ((be & 31) == lane) {
#pragma unroll
            for (int i = 0; i < ROUTE_MAX_E / 32; ++i)
                if (lane + 32 * i == be) taken[i] = true;
        }
    }
    // renormalised softmax over the selection: the full-softmax denominator cancels. The sum is
    // formed in slot order, as a serial loop would, so the bits do not depend on the lane count.
    const float p = lane < k ? expf(my_v - top_v) : 0.f;
    float sum = 0.f;
    for (int j = 0; j < k; ++j) sum += __shfl_sync(0xffffffffu, p, j);
    if (lane < k) {
        const size_t at = static_cast<size_t>(out.row_base + warp) * k + lane;
        const float wj = p / sum;
        for (int r = 0; r < out.n_out; ++r) {
            out.idx[r][at] = my_e;
            out.w[r][at] = wj;
        }
    }
    }
    ep_signal_done(sig);
}

// ------------------------------------------------------------------------------------ permute
// Stable counting sort of the pairs by expert in three launches:
//   A  per-chunk histograms                 -> scratch[chunk][E]
//   B  (one block) per-expert scan over chunks, padded offsets (restarting every `seg` experts)
//   C  position of every pair = offset[e] + pairs of e in earlier chunks + earlier pairs of e in
//      this chunk (warp match + per-warp counts)
constexpr int PERM_CHUNK = 1024;  // pairs per block, one per thread
// sites of the bad-index record (DK_DEV_BAD_INDEX): an expert id outside [0, E) in topk_idx (the pair
// is left out: row_of_pair = -1), a row at or beyond the caller's capacity (the pair is left out)
enum : unsigned { SITE_PERM_EXPERT = 80, SITE_PERM_ROW = 81 };

__global__ void __launch_bounds__(PERM_CHUNK) moe_hist_kernel(const int* __restrict__ topk_idx,
                                                              int npairs, int E,
                                                              int* __restrict__ chunk_counts,
                                                              unsigned* status, const EpWait wait) {
    __shared__ int cnt[ROUTE_MAX_E];
    if (!ep_wait_sources(wait)) return;
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    const int i = blockIdx.x * PERM_CHUNK + threadIdx.x;
    if (i < npairs) {
        const int e = topk_idx[i];
        if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);  // a count: order-independent
        else record_bad_index(status, SITE_PERM_EXPERT, static_cast<unsigned>(i));
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) chunk_counts[static_cast<size_t>(blockIdx.x) * E + e] = cnt[e];
}

__global__ void __launch_bounds__(ROUTE_MAX_E) moe_scan_kernel(int* __restrict__ chunk_counts, int nchunks,
                                                               int E, int pad, int seg,
                                                               int* __restrict__ counts,
                                                               int* __restrict__ offsets) {
    __shared__ int padded[ROUTE_MAX_E];
    const int e = threadIdx.x;
    if (e < E) {
        int run = 0;
        // exclusive scan over chunks, in place; eight independent loads at a time (the loop is bound
        // by load latency, not by the additions)
        for (int c0 = 0; c0 < nchunks; c0 += 8) {
            int v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
                v[i] = c0 + i < nchunks ? chunk_counts[static_cast<size_t>(c0 + i) * E + e] : 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (c0 + i < nchunks) chunk_counts[static_cast<size_t>(c0 + i) * E + e] = run;
                run += v[i];
            }
        }
        counts[e] = run;
        padded[e] = (run + pad - 1) / pad * pad;
    }
    __syncthreads();
    if (e == 0) {
        // offsets restart at every segment of `seg` experts (one segment per destination rank);
        // offsets has E + E/seg entries: for segment g, entries [g*(seg+1), (g+1)*(seg+1))
        const int nseg = E / seg;
        for (int g = 0; g < nseg; ++g) {
            int run = 0;
            for (int j = 0; j < seg; ++j) {
                offsets[g * (seg + 1) + j] = run;
                run += padded[g * seg + j];
            }
            offsets[g * (seg + 1) + seg] = run;
        }
    }
}

__global__ void __launch_bounds__(PERM_CHUNK) moe_place_kernel(const int* __restrict__ topk_idx, int npairs,
                                                               int E, int seg,
                                                               const int* __restrict__ chunk_base,
                                                               const int* __restrict__ offsets,
                                                               int* __restrict__ row_of_pair,
                                                               int* __restrict__ pair_of_row,
                                                               int seg_row_capacity, unsigned* status) {
    __shared__ int warp_cnt[PERM_CHUNK / 32][ROUTE_MAX_E];  // 32 KiB
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int x = threadIdx.x; x < (PERM_CHUNK / 32) * ROUTE_MAX_E; x += blockDim.x)
        (&warp_cnt[0][0])[x] = 0;
    __syncthreads();
    const int i = blockIdx.x * PERM_CHUNK + threadIdx.x;
    bool live = i < npairs;
    int e = live ? topk_idx[i] : -1;
    if (live && (e < 0 || e >= E)) {  // recorded by the histogram kernel; the pair gets no row
        row_of_pair[i] = -1;
        live = false;
        e = -1;
    }
    // lanes of this warp holding the same expert; my rank among them = those before me
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1));
    if (live && rank_in_warp == 0) warp_cnt[warp][e] = __popc(peers);
    __syncthreads();
    if (live) {
        int before = 0;
        for (int w = 0; w < warp; ++w) before += warp_cnt[w][e];
        const int g = e / seg;
        const int row = offsets[g * (seg + 1) + (e - g * seg)] +
                        chunk_base[static_cast<size_t>(blockIdx.x) * E + e] + before + rank_in_warp;
        if (row < seg_row_capacity) {
            row_of_pair[i] = row;
            pair_of_row[static_cast<size_t>(g) * seg_row_capacity + row] = i;
        } else {
            row_of_pair[i] = -1;
            record_bad_index(status, SITE_PERM_ROW, static_cast<unsigned>(i));
        }
    }
}

// ------------------------------------------------------------------------------------ quantise
// One 128x128 block at a time per CTA (grid-stride over the blocks that exist). 256 threads; thread t owns column chunk (t % 16) * 8 of rows
// t/16 + 16*i, i = 0..7. Source rows come straight from x, or through a row map:
//   map_mode 0: row r of x;  1: row map[r] / k of x (gather), zeros where map[r] < 0;
//   2: row r of x where map[r] >= 0, zeros elsewhere (rows already in place, padding undefined)
//   3: row map2[map[r] / k] of x (a gather through two maps: pair of the row -> token -> where the
//      token's vector landed), zeros where either entry is negative
// row_limit (device memory, may be null): row blocks at or beyond *row_limit are not produced.
// POW2: the scale is rounded UP to a power of two, s = 2^ceil(log2(amax/448)) (1 for an all-zero
// block), and also written as an e8m0 byte (log2(s) + 127) and into the scale atoms the
// block-scaled tensor-core path reads: per 128 rows and four column blocks one 512-byte atom whose
// byte r*4 + g (r = row slot 0..127, g = 0..3) is the byte of column block 4j + g.
__device__ __forceinline__ float div_by_fma(float x, float d, float inv_d) {
    const float q0 = x * inv_d;
    const float r = fmaf(-q0, d, x);
    return fmaf(r, inv_d, q0);
}

template <bool POW2>
__global__ void __launch_bounds__(256, 4) quant_block128_kernel(const __nv_bfloat16* __restrict__ x, int R, int C,
                                                             const int* __restrict__ map, int map_mode,
                                                             int k, uint8_t* __restrict__ q,
                                                             float* __restrict__ s, uint8_t* __restrict__ e8,
                                                             uint8_t* __restrict__ atoms,
                                                             const int* __restrict__ map2,
                                                             const int* __restrict__ row_limit, const EpWait wait) {
    __shared__ float red[8];
    // The grid is sized for the GPU, not for R: with a row limit read on the device most of the R / 128
    // row blocks may not exist, and a CTA per block would spend the kernel launching CTAs that exit.
    const int cblocks = C / 128;
    const int rows = row_limit != nullptr ? min(*row_limit, R) : R;
    const int nblocks = (rows / 128) * cblocks;
    if (static_cast<int>(blockIdx.x) >= nblocks) return;
    if (!ep_wait_sources(wait)) return;
    const int cchunk = (threadIdx.x & 15) * 8;
    const int r0 = threadIdx.x >> 4;
    for (int blk_i = blockIdx.x; blk_i < nblocks; blk_i += gridDim.x) {
    const int br = blk_i / cblocks, bc = blk_i - br * cblocks;
    __syncthreads();  // the previous block's maxima have been read
    // The 8 x 8 values of this thread stay packed as bf16 (32 registers instead of 64): the kernel is
    // bound by how many row loads an SM keeps in flight, i.e. by how many CTAs fit.
    uint4 u[8];
    long src[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = br * 128 + r0 + 16 * i;
        src[i] = r;
        if (map_mode != 0) {
            const int mv = map[r];
            bool valid = mv >= 0;
            if (map_mode == 1) src[i] = valid ? mv / k : -1;
            if (map_mode == 2) src[i] = valid ? r : -1;
            if (map_mode == 3) {
                const int slot = valid ? map2[mv / k] : -1;
                src[i] = slot;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        u[i] = make_uint4(0, 0, 0, 0);
        if (src[i] >= 0) u[i] = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(src[i]) * C + bc * 128 + cchunk);
    }
    __nv_bfloat162 m2 = __float2bfloat162_rn(0.f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) m2 = __hmax2(m2, __habs2(h[j]));  // exact: a maximum of magnitudes
    }
    float amax = fmaxf(__low2float(m2), __high2float(m2));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
    float scale = amax > 0.f ? amax / 448.0f : 1.0f;
    const size_t blk = static_cast<size_t>(br) * (C / 128) + bc;
    if (POW2) {
        int ex = 0;
        if (amax > 0.f) {
            const float m = frexpf(scale, &ex);  // amax/448 = m * 2^ex, m in [0.5, 1)
            if (m == 0.5f) ex -= 1;              // exact powers of two stay as they are
            ex = max(-127, min(127, ex));
        }
        scale = ldexpf(1.0f, ex);
        const uint32_t b8 = static_cast<uint32_t>(ex + 127);
        if (threadIdx.x < 128) {
            // byte (bc % 4) of atom (bc / 4) of this row block, for each of its 128 rows
            const int kb4 = (C / 128 + 3) / 4;
            atoms[(static_cast<size_t>(br) * kb4 + (bc >> 2)) * 512 + threadIdx.x * 4 + (bc & 3)] =
                static_cast<uint8_t>(b8);
        }
        if (threadIdx.x == 0 && e8 != nullptr) e8[blk] = static_cast<uint8_t>(b8);
    }
    if (threadIdx.x == 0 && s != nullptr) s[blk] = scale;
    const float inv = 1.0f / scale;  // correctly rounded; exact for a power of two
    // The CPU definition divides (x / scale, correctly rounded). The same bits come from q0 = x * inv,
    // r = x - q0 * scale (exact in an FMA), q = q0 + r * inv whenever r does not underflow; with the scale
    // in this range it can underflow only for quotients below 1e-7, which round to zero in e4m3
    // either way (the smallest rounding boundary is 2^-10). A third of the instructions of a division.
    const bool fast_div = scale >= 0x1p-80f && scale <= 0x1p80f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = br * 128 + r0 + 16 * i;
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u[i]);
        uint32_t w[2];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            float2 y;
            if (POW2) {
                y = make_float2(f.x * inv, f.y * inv);
            } else if (fast_div) {
                y = make_float2(div_by_fma(f.x, scale, inv), div_by_fma(f.y, scale, inv));
            } else {
                y = make_float2(f.x / scale, f.y / scale);  // IEEE division: same bits as the CPU definition
            }
            // |x| <= amax, so |y| <= 448 up to rounding: the saturating conversion is the clamp
            const uint32_t p = __nv_cvt_float2_to_fp8x2(y, __NV_SATFINITE, __NV_E4M3);
            if (j & 1) w[j >> 1] |= p << 16;
            else w[j >> 1] = p;
        }
        *reinterpret_cast<uint2*>(q + static_cast<size_t>(r) * C + bc * 128 + cchunk) = make_uint2(w[0], w[1]);
    }
    }  // blocks of this CTA
}

// ------------------------------------------------------------------------------------ combine
// out[t, :] = sum_j w[t,j] * Y_j[row(t,j), :]. One block per token; y_base[j-th pair] selects the
// buffer (this rank's Y, or a peer's Y in the expert-parallel case).
struct CombineArgs {
    const __nv_bfloat16* y[DK_MAX_RANKS];  // Y of rank r as seen from here
    const int* row_of_pair;                // [T, k]
    const int* dest_of_pair;               // [T, k] rank holding the row; null = all local (y[0])
    const float* w;                        // [T, k]
    __nv_bfloat16* out;                    // [T, H]
    int T, k, H;
};
__global__ void __launch_bounds__(256) moe_combine_kernel(const CombineArgs a) {
    const int t = blockIdx.x;
    __shared__ int row_s[ROUTE_MAX_K];
    __shared__ int dst_s[ROUTE_MAX_K];
    __shared__ float w_s[ROUTE_MAX_K];
    if (threadIdx.x < a.k) {
        row_s[threadIdx.x] = a.row_of_pair[static_cast<size_t>(t) * a.k + threadIdx.x];
        dst_s[threadIdx.x] = a.dest_of_pair ? a.dest_of_pair[static_cast<size_t>(t) * a.k + threadIdx.x] : 0;
        w_s[threadIdx.x] = a.w[static_cast<size_t>(t) * a.k + threadIdx.x];
    }
    __syncthreads();
    for (int c = threadIdx.x * 8; c < a.H; c += blockDim.x * 8) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int j = 0; j < a.k; ++j) {
            if (row_s[j] < 0) continue;  // a pair the permutation left out (bad expert id / no room)
            const uint4 u = __ldcg(reinterpret_cast<const uint4*>(
                a.y[dst_s[j]] + static_cast<size_t>(row_s[j]) * a.H + c));
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
            const float wj = w_s[j];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(h[i]);
                acc[2 * i] += wj * f.x;
                acc[2 * i + 1] += wj * f.y;
            }
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]);
        o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]);
        o.w = pack_bf16x2(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(a.out + static_cast<size_t>(t) * a.H + c) = o;
    }
}

int moe_route_launch(const float* logits, int T, int E, int k, const RouteOut& out, const EpSignal& sig,
                     cudaStream_t st) {
    const int warps_per_block = 8;
    int blocks = (T + warps_per_block - 1) / warps_per_block;
    if (blocks < 1) blocks = 1;  // a launch with a signal must run even without tokens
    moe_route_kernel<<<blocks, warps_per_block * 32, 0, st>>>(logits, T, E, k, out, sig);
    DK_CUDA_OK(cudaGetLastError());
    return DK_OK;
}

// shared by the allocating and the non-allocating permute entry points
int moe_permute_launch(const int* topk_idx, int T, int k, int E, int pad, int seg, int* row_of_pair,
                       int* pair_of_row, int seg_row_capacity, int* offsets, int* counts,
                       int* scratch, const EpWait& wait, cudaStream_t st) {
    const int npairs = T * k;
    const int nseg = E / seg;
    unsigned* status = nullptr;
    const int src = device_status_ptr(&status);
    if (src != DK_OK) return src;
    DK_CUDA_OK(cudaMemsetAsync(pair_of_row, 0xff, static_cast<size_t>(nseg) * seg_row_capacity * sizeof(int), st));
    const int nchunks = (npairs + PERM_CHUNK - 1) / PERM_CHUNK;
    if (nchunks > 0) {
        moe_hist_kernel<<<nchunks, PERM_CHUNK, 0, st>>>(topk_idx, npairs, E, scratch, status, wait);
        DK_CUDA_OK(cudaGetLastError());
    }
    moe_scan_kernel<<<1, ROUTE_MAX_E, 0, st>>>(scratch, nchunks, E, pad, seg, counts, offsets);
    DK_CUDA_OK(cudaGetLastError());
    if (nchunks > 0) {
        moe_place_kernel<<<nchunks, PERM_CHUNK, 0, st>>>(topk_idx, npairs, E, seg, scratch, offsets,
                                                         row_of_pair, pair_of_row, seg_row_capacity, status);
        DK_CUDA_OK(cudaGetLastError());
    }
    return DK_OK;
}

int moe_permute_check(const void* topk_idx, int T, int k, int E, int pad, int seg, const void* a,
                      const void* b, const void* c, const void* d, int seg_row_capacity) {
    DK_REQUIRE(T >= 0 && k >= 1 && k <= ROUTE_MAX_K, "k must be 1..8");
    DK_REQUIRE(E >= 1 && E <= ROUTE_MAX_E, "E must be 1..256");
    DK_REQUIRE(pad >= 1, "pad must be positive");
    DK_REQUIRE(seg >= 1 && E % seg == 0, "experts per segment must divide E");
    DK_REQUIRE((T == 0 || (topk_idx != nullptr && a != nullptr)) && c && d, "null buffer");
    DK_REQUIRE(b != nullptr || seg_row_capacity == 0, "null buffer");
    DK_REQUIRE(seg_row_capacity >= 0, "negative capacity");
    return DK_OK;
}

int quant_block128_launch(const void* x, int R, int C, const int* map, int map_mode, int k, const int* map2,
                          const int* row_limit, void* q, float* s, void* e8, void* atoms, bool pow2,
                          const EpWait& wait, cudaStream_t st) {
    DK_REQUIRE(R >= 0 && C > 0 && R % 128 == 0 && C % 128 == 0, "R and C must be multiples of 128");
    DK_REQUIRE(map_mode >= 0 && map_mode <= 3, "map_mode must be 0..3");
    DK_REQUIRE(map_mode == 0 || map != nullptr, "row_map is null");
    DK_REQUIRE((map_mode != 1 && map_mode != 3) || k >= 1, "k must be positive");
    DK_REQUIRE(map_mode != 3 || map2 != nullptr, "second map is null");
    if (R == 0) return DK_OK;
    DK_REQUIRE(x && q, "null buffer");
    DK_REQUIRE(!pow2 || (reinterpret_cast<uintptr_t>(atoms) & 15) == 0, "the scale atoms must be 16-byte aligned");
    int sms = 0;
    const int src = sm_count(&sms);
    if (src != DK_OK) return src;
    const long long all = static_cast<long long>(C / 128) * (R / 128);
    const int grid = static_cast<int>(std::min<long long>(all, 4ll * sms * 2));  // two rounds of resident CTAs at most
    if (pow2)
        quant_block128_kernel<true><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), R, C, map, map_mode, k,
                                                          static_cast<uint8_t*>(q), s, static_cast<uint8_t*>(e8),
                                                          static_cast<uint8_t*>(atoms), map2, row_limit, wait);
    else
        quant_block128_kernel<false><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), R, C, map, map_mode,
                                                           k, static_cast<uint8_t*>(q), s, nullptr, nullptr, map2,
                                                           row_limit, wait);
    DK_CUDA_OK(cudaGetLastError());
    return DK_OK;
}

}  // namespace dk

extern "C" {

int dk_moe_route(const float* logits, int T, int E, int k, int* topk_idx, float* topk_w, void* stream) {
    using namespace dk;
    DK_REQUIRE(T >= 0 && E >= 1 && E <= ROUTE_MAX_E, "E must be 1..256");
    DK_REQUIRE(k >= 1 && k <= ROUTE_MAX_K && k <= E, "k must be 1..8 and <= E");
    if (T == 0) return DK_OK;
    DK_REQUIRE(logits && topk_idx && topk_w, "null buffer");
    RouteOut out{};
    out.idx[0] = topk_idx;
    out.w[0] = topk_w;
    out.n_out = 1;
    out.row_base = 0;
    return moe_route_launch(logits, T, E, k, out, EpSignal{}, static_cast<cudaStream_t>(stream));
}

size_t dk_moe_permute_scratch_bytes(int T, int k, int E) {
    if (T < 0 || k < 1 || E < 1) return 0;
    const size_t nchunks = (static_cast<size_t>(T) * k + dk::PERM_CHUNK - 1) / dk::PERM_CHUNK;
    return (nchunks > 0 ? nchunks : 1) * E * sizeof(int);
}

size_t dk_moe_rows_capacity(int T, int k, int E, int pad) {
    if (T < 0 || k < 1 || E < 1 || pad < 1) return 0;
    // every expert may waste up to pad-1 rows
    const size_t cap = static_cast<size_t>(T) * k + static_cast<size_t>(E) * (pad - 1);
    return (cap + pad - 1) / pad * pad;
}

int dk_moe_permute(const int* topk_idx, int T, int k, int E, int pad, int experts_per_segment,
                   int* row_of_pair, int* pair_of_row, int seg_row_capacity, int* offsets,
                   int* counts, void* scratch, size_t scratch_bytes, void* stream) {
    using namespace dk;
    int rc = moe_permute_check(topk_idx, T, k, E, pad, experts_per_segment, row_of_pair, pair_of_row,
                               offsets, counts, seg_row_capacity);
    if (rc != DK_OK) return rc;
    DK_REQUIRE(scratch != nullptr && scratch_bytes >= dk_moe_permute_scratch_bytes(T, k, E),
               "scratch too small: see dk_moe_permute_scratch_bytes");
    return moe_permute_launch(topk_idx, T, k, E, pad, experts_per_segment, row_of_pair, pair_of_row,
                              seg_row_capacity, offsets, counts, static_cast<int*>(scratch), EpWait{},
                              static_cast<cudaStream_t>(stream));
}

// ---- permutation without any allocation ----------------------------------------------------------
// Scratch for dk_moe_permute_static: the per-chunk histograms live in this fixed array instead of
// in memory the caller allocates. Every GPU that loads the library holds these 256 KiB until the
// process exits. In host code the symbol is only a stand-in; its device address is looked up once
// per device with cudaGetSymbolAddress and that pointer is what the kernels receive.
#define DK_PERMUTE_STATIC_MAX_BYTES (256u * 1024u)
static __device__ __align__(256) int g_permute_scratch[DK_PERMUTE_STATIC_MAX_BYTES / sizeof(int)];
static int* g_permute_scratch_addr[64] = {nullptr};
static std::mutex g_permute_scratch_mu;

size_t dk_moe_permute_static_max_bytes(void) { return DK_PERMUTE_STATIC_MAX_BYTES; }

int dk_moe_permute_static(const int* topk_idx, int T, int k, int E, int pad, int experts_per_segment,
                          int* row_of_pair, int* pair_of_row, int seg_row_capacity, int* offsets,
                          int* counts, void* stream) {
    using namespace dk;
    int rc = moe_permute_check(topk_idx, T, k, E, pad, experts_per_segment, row_of_pair, pair_of_row,
                               offsets, counts, seg_row_capacity);
    if (rc != DK_OK) return rc;
    const size_t need = dk_moe_permute_scratch_bytes(T, k, E);
    if (need > DK_PERMUTE_STATIC_MAX_BYTES) {
        set_last_error("argument error: this routing needs " + std::to_string(need) +
                       " bytes of scratch, more than the " + std::to_string(DK_PERMUTE_STATIC_MAX_BYTES) +
                       " bytes built into dk_moe_permute_static; use dk_moe_permute with caller scratch");
        return DK_ERR_ARG;
    }
    int dev = 0;
    DK_CUDA_OK(cudaGetDevice(&dev));
    DK_REQUIRE(dev >= 0 && dev < 64, "device index out of range");
    int* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_permute_scratch_mu);
        if (g_permute_scratch_addr[dev] == nullptr) {
            // first call on this device: resolve the array's address on the current device
            void* p = nullptr;
            DK_CUDA_OK(cudaGetSymbolAddress(&p, g_permute_scratch));
            g_permute_scratch_addr[dev] = static_cast<int*>(p);
        }
        scratch = g_permute_scratch_addr[dev];
    }
    // Nothing has to be cleared: the histogram kernel writes every [chunk][expert] entry this call
    // reads, so whatever an earlier call left behind is overwritten before use.
    return moe_permute_launch(topk_idx, T, k, E, pad, experts_per_segment, row_of_pair, pair_of_row,
                              seg_row_capacity, offsets, counts, scratch, EpWait{},
                              static_cast<cudaStream_t>(stream));
}

int dk_quant_block128(const void* x, int R, int C, const int* row_map, int map_mode, int k, void* q,
                      float* s, void* stream) {
    using namespace dk;
    DK_REQUIRE(map_mode >= 0 && map_mode <= 2, "map_mode must be 0, 1 or 2");
    DK_REQUIRE(R == 0 || s != nullptr, "null buffer");
    return quant_block128_launch(x, R, C, row_map, map_mode, k, nullptr, nullptr, q, s, nullptr, nullptr, false,
                                 EpWait{}, static_cast<cudaStream_t>(stream));
}

int dk_quant_block128_pow2(const void* x, int R, int C, const int* row_map, int map_mode, int k, void* q,
                           float* s, void* e8, void* sf_atoms, void* stream) {
    using namespace dk;
    DK_REQUIRE(map_mode >= 0 && map_mode <= 2, "map_mode must be 0, 1 or 2");
    DK_REQUIRE(R == 0 || sf_atoms != nullptr, "null buffer");
    return quant_block128_launch(x, R, C, row_map, map_mode, k, nullptr, nullptr, q, s, e8, sf_atoms, true,
                                 EpWait{}, static_cast<cudaStream_t>(stream));
}

int dk_moe_combine(const void* y, const int* row_of_pair, const float* topk_w, int T, int k, int H,
                   void* out, void* stream) {
    using namespace dk;
    DK_REQUIRE(T >= 0 && k >= 1 && k <= ROUTE_MAX_K && H > 0 && H % 8 == 0, "bad shape");
    if (T == 0) return DK_OK;
    DK_REQUIRE(y && row_of_pair && topk_w && out, "null buffer");
    CombineArgs a{};
    a.y[0] = static_cast<const __nv_bfloat16*>(y);
    a.row_of_pair = row_of_pair;
    a.dest_of_pair = nullptr;
    a.w = topk_w;
    a.out = static_cast<__nv_bfloat16*>(out);
    a.T = T;
    a.k = k;
    a.H = H;
    moe_combine_kernel<<<T, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
    DK_CUDA_OK(cudaGetLastError());
    return DK_OK;
}

}  // extern "C"
