// The block-scaled fp8 GEMM kernel (tcgen05.mma.kind::mxf8f6f4.block_scale) behind dk_gemm_mxfp8 and
// dk_moe_grouped_gemm_mxfp8; see dk_mx.cu for what it stands in for.
//
//   warp 0      TMA producer: A tile 128 rows x 128 K-bytes, B tile (128-byte swizzle) and three
//               scale atoms (one for A, two for B) per stage
//   warp 1      per stage: three tcgen05.cp (atoms -> 12 tensor-memory columns), four
//               tcgen05.mma (K = 32 each, scale byte selected by the instruction descriptor),
//               accumulating over all of K into one 256-column accumulator
//   warps 4-11  epilogue: tcgen05.ld, then bf16 / fp32 stores, or SiLU(gate)*up, tile-wide amax,
//               power-of-two scale, e4m3 bytes + scale atom (the 128x128 output tile is exactly one
//               scale block of the next GEMM's A operand)
//
// PAIR = 1: one CTA per 128x256 tile, 48 KiB + scales per stage, four stages.
// PAIR = 2: a cluster of two CTAs per 256x256 tile (cta_group::2): each CTA stages its own 128 rows
// of A, HALF of the B tile (gated: CTA 0 the gate rows, CTA 1 the up rows) and the scale atoms it
// needs (its own rows of A, all 256 rows of B), 32 KiB + scales per stage, six stages. Both CTAs'
// loads, the scale atoms included (as tensor-map loads: a plain bulk copy cannot complete on
// another CTA's barrier), complete on the LEADER's mbarrier; the leader issues the scale copies and
// MMAs for both; stage release and accumulator hand-over are the paired tcgen05.commit. Half the
// shared-memory fill per flop and a deeper ring. An expert with an odd number of 128-row tiles
// leaves the second CTA of its last pair without rows: it loads and multiplies whatever follows
// (the MMA is issued for both anyway) and stores nothing.
//
// Scales need tensor-memory columns too, so there is one accumulator (256 + 12 of the 512
// columns): the epilogue of a tile is not overlapped with the next tile's MMAs. It costs one drain
// (a few hundred cycles) per K/128 * 512 cycles of MMAs.
#pragma once
#include <cuda_fp8.h>

#include "dk_host.h"
#include "dk_ptx.cuh"

namespace dk {

constexpr int XM = 128;
constexpr int XN = 256;
constexpr int XK = 128;  // bytes = e4m3 elements per K block = one swizzle row = four scale groups
constexpr int XA_BYTES = XM * XK;
constexpr int X_ATOM = 512;
constexpr int X_MAX_E = 256;
constexpr int X_CTRL_BYTES = 256 + (X_MAX_E + 1) * 4 * 2 + 128;
constexpr int X_THREADS = 384;
constexpr int X_EPI_WARPS = 8;
constexpr int X_SF_COL = 256;  // tensor-memory columns 256..259: scales of A, 260..267: scales of B

template <int PAIR>
struct XCfg {
    static constexpr int B_ROWS = XN / PAIR;
    static constexpr int B_BYTES = B_ROWS * XK;
    static constexpr int STAGES = PAIR == 2 ? 6 : 4;
    static constexpr int STAGE_TX = XA_BYTES + B_BYTES + 3 * X_ATOM;  // with scale atoms
    static constexpr int STAGE_STRIDE = PAIR == 2 ? 34 * 1024 : 50 * 1024;  // keeps stages 1024-byte aligned
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_STRIDE + X_CTRL_BYTES;
};

enum : int { MX_OUT_BF16 = 0, MX_OUT_F32 = 1, MX_OUT_GATED = 2 };

struct MxMaps {
    CUtensorMap a;    // A [rows, K] bytes, box 128 x 128
    CUtensorMap b;    // B [rows, K] bytes, box 128 x (128 or 256 rows)
    CUtensorMap sfa;  // pair kernel: scale atoms of A as [atoms, 128] 32-bit words, box 128 x 1
    CUtensorMap sfb;  // pair kernel: the same for B
};

struct MxArgs {
    const int* offsets;   // [E+1] device (multiples of 128), or null: one group of rows_pad rows
    const uint8_t* sfa;   // scale atoms of A: [row blocks][K/128][512]; block mode: [row blocks][ceil(K/512)][512]
    const uint8_t* sfb;   // scale atoms of B, likewise
    int E, K, N;          // N: output columns (gated: F)
    int num_kb;           // K / 128
    int n_tiles;          // gated: F/128, plain: ceil(N/256)
    int band;             // row tiles per band of the tile walk (>= 1)
    int w_rows;           // rows of one group's B matrix: gated 2F, plain N
    int w_blocks;         // 128-row blocks of one group's B matrix
    int sfa_blocks;       // 128-row blocks in sfa / sfb altogether (atom indices are clamped to them)
    int sfb_blocks;
    int R;                // rows of the output that exist
    int rows_pad;         // R rounded up to 128 (used when offsets is null)
    void* out;            // bf16 / fp32 [R, N], or e4m3 bytes [R, F]
    uint8_t* out_e8;      // gated: e8m0 scale per 128x128 block [R/128, F/128]
    uint8_t* out_atoms;   // gated: the same scales as block-mode atoms [R/128][ceil(F/512)][512]
    unsigned* status;
};

enum : unsigned { XS_EMPTY = 64, XS_FULL = 65, XS_TEMPTY = 66, XS_TFULL = 67, XS_EPI = 68, XS_OFFSETS = 69 };

// Tile walk shared by all roles: tile t -> (group, first row of the tile, column tile, rows left in
// the group from there). A tile covers 128 * PAIR rows. Inside a group the tiles go band by band: a
// band is `band` row tiles; inside a band row tiles run fastest, then column tiles. CTAs running
// together share a B tile in L2, and a band's rows of A (sized by the host to a fraction of L2) stay
// there while all column tiles pass, so a group with more rows than L2 holds is still read from DRAM
// once, not once per column tile. cum[e] = tiles before group e.
struct MxWalk {
    const int* cum;   // [E+1] in shared memory
    const int* offs;  // [E+1] in shared memory
    int E, e, tile_rows, n_tiles, band;
    __device__ __forceinline__ bool locate(int t, int& group, int& row0, int& n, int& rows_left) {
        if (t >= cum[E]) return false;
        while (t >= cum[e + 1]) ++e;
        const int local = t - cum[e];
        const int mt = (offs[e + 1] - offs[e] + tile_rows - 1) / tile_rows;
        group = e;
        int rt;
        if (mt <= band) {
            rt = local % mt;
            n = local / mt;
        } else {
            const int per_band = band * n_tiles;
            const int b = local / per_band, rem = local - b * per_band;
            const int in_band = min(band, mt - b * band);
            n = rem / in_band;
            rt = b * band + rem - n * in_band;
        }
        row0 = offs[e] + rt * tile_rows;
        rows_left = offs[e + 1] - row0;
        return true;
    }
};

__device__ __forceinline__ float mx_rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// Hand the accumulator back to the MMA issuer (the leader's, which may sit in the other CTA).
__device__ __forceinline__ void mx_release_acc(uint32_t bar_tempty, bool remote, int lane) {
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
        if (remote) mbar_arrive_cluster(bar_tempty);
        else mbar_arrive(bar_tempty);
    }
}

// Epilogue of one tile for one of the eight epilogue warps: rows row0 + q*32 + lane of this CTA's 128
// rows, half h of the columns. `store` is false for a CTA of a pair whose rows do not exist.
// Returns false if a bounded wait gave up.
template <int MODE>
__device__ __forceinline__ bool mx_epilogue_tile(const MxArgs& g, const WaitCtx& wc, uint32_t tmem_base,
                                                 uint32_t bar_tempty, bool tempty_remote, uint32_t bar_epi,
                                                 float* red, int ew, int lane, int row0, int n, bool store,
                                                 unsigned tiles_done, int t) {
    const int q = ew & 3;   // tensor-memory lane quarter of this warp (warps 4..11: warp % 4 == ew % 4)
    const int h = ew >> 2;  // which half of the columns
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const int row = row0 + q * 32 + lane;
    if (MODE == MX_OUT_GATED) {
        // gate columns h*64.. of the tile sit at accumulator columns h*64.., the matching up
        // columns at 128 + h*64..
        uint32_t ga[32], gb[32], ua[32], ub[32];
        tmem_ld_32x32b_x32(t_row + h * 64, ga);
        tmem_ld_32x32b_x32(t_row + h * 64 + 32, gb);
        tmem_ld_32x32b_x32(t_row + 128 + h * 64, ua);
        tmem_ld_32x32b_x32(t_row + 128 + h * 64 + 32, ub);
        tmem_ld_wait(ga);
        tmem_ld_wait(gb);
        tmem_ld_wait(ua);
        tmem_ld_wait(ub);
        // the accumulator is in registers: the next tile's MMAs may overwrite it
        mx_release_acc(bar_tempty, tempty_remote, lane);
        float hv[64];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const float g0 = __uint_as_float(ga[i]);
            const float g1 = __uint_as_float(gb[i]);
            hv[i] = g0 * mx_rcp_approx(1.0f + __expf(-g0)) * __uint_as_float(ua[i]);
            hv[32 + i] = g1 * mx_rcp_approx(1.0f + __expf(-g1)) * __uint_as_float(ub[i]);
            amax = fmaxf(amax, fmaxf(fabsf(hv[i]), fabsf(hv[32 + i])));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        float* red_t = red + (tiles_done & 1) * X_EPI_WARPS;
        if (lane == 0) {
            red_t[ew] = amax;
            mbar_arrive(bar_epi);
        }
        if (!__all_sync(0xffffffffu, mbar_wait(bar_epi, tiles_done & 1, wc, XS_EPI, t))) return false;
        if (!store) return true;
        float tmax = red_t[0];
#pragma unroll
        for (int w = 1; w < X_EPI_WARPS; ++w) tmax = fmaxf(tmax, red_t[w]);
        // scale = 2^ceil(log2(tmax / 448)), 1 for an all-zero tile
        int ex = 0;
        if (tmax > 0.f) {
            const float m = frexpf(__fdiv_rn(tmax, 448.0f), &ex);
            if (m == 0.5f) ex -= 1;
            ex = max(-127, min(127, ex));
        }
        const float inv_scale = ldexpf(1.0f, -ex);
        const uint32_t e8 = static_cast<uint32_t>(ex + 127);
        const size_t blk = static_cast<size_t>(row0 / XM) * (g.N / 128) + n;
        if (ew == 0) {
            // this tile is K block n of the next GEMM's A operand: byte n % 4 of atom n / 4
            // of its row block, for every row
            const int fb = g.N / 128;
            uint8_t* atom =
                g.out_atoms + (static_cast<size_t>(row0 / XM) * ((fb + 3) / 4) + (n >> 2)) * X_ATOM + (n & 3);
#pragma unroll
            for (int r1 = 0; r1 < 4; ++r1) atom[lane * 16 + r1 * 4] = static_cast<uint8_t>(e8);
            if (lane == 0) g.out_e8[blk] = static_cast<uint8_t>(e8);
        }
        if (row < g.R) {
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint32_t lo = __nv_cvt_float2_to_fp8x2(
                    make_float2(hv[4 * i] * inv_scale, hv[4 * i + 1] * inv_scale), __NV_SATFINITE, __NV_E4M3);
                const uint32_t hi = __nv_cvt_float2_to_fp8x2(
                    make_float2(hv[4 * i + 2] * inv_scale, hv[4 * i + 3] * inv_scale), __NV_SATFINITE, __NV_E4M3);
                pk[i] = lo | (hi << 16);
            }
            uint8_t* dst = static_cast<uint8_t*>(g.out) + static_cast<size_t>(row) * g.N + n * 128 + h * 64;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                *reinterpret_cast<uint4*>(dst + 16 * j) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
        }
    } else {
        // columns n*256 + h*128 + c*32 .. of this thread's row, two chunks in flight
        const int col_base = n * XN + h * 128;
        uint32_t ra[32], rb[32];
        tmem_ld_32x32b_x32(t_row + h * 128, ra);
        tmem_ld_32x32b_x32(t_row + h * 128 + 32, rb);
#pragma unroll
        for (int c = 0; c < 4; c += 2) {
            tmem_ld_wait(ra);
            tmem_ld_wait(rb);
            uint32_t va[32], vb[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                va[i] = ra[i];
                vb[i] = rb[i];
            }
            if (c == 0) {
                tmem_ld_32x32b_x32(t_row + h * 128 + 64, ra);
                tmem_ld_32x32b_x32(t_row + h * 128 + 96, rb);
            } else {
                mx_release_acc(bar_tempty, tempty_remote, lane);
            }
            if (store && row < g.R) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const uint32_t* v = half == 0 ? va : vb;
                    const int col0 = col_base + (c + half) * 32;
                    if (MODE == MX_OUT_F32) {
                        float* dst = static_cast<float*>(g.out) + static_cast<size_t>(row) * g.N + col0;
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (col0 + 4 * j + 4 <= g.N)
                                *reinterpret_cast<uint4*>(dst + 4 * j) =
                                    make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    } else {
                        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(g.out) + static_cast<size_t>(row) * g.N + col0;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (col0 + 8 * j + 8 <= g.N) {
                                uint4 o;
                                o.x = pack_bf16x2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1]));
                                o.y = pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
                                o.z = pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
                                o.w = pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
                                *reinterpret_cast<uint4*>(dst + 8 * j) = o;
                            }
                        }
                    }
                }
            }
        }
    }
    return true;
}

// 2-D tiled load of one 512-byte scale atom (row `atom` of a [atoms, 128 x u32] tensor, no swizzle)
// issued by either CTA of a pair, completing on a barrier that may live in the other CTA.
__device__ __forceinline__ void tma_load_atom_pair(uint32_t dst, const CUtensorMap* m, uint32_t cluster_bar,
                                                   int atom) {
    tma_load_2d_pair(dst, m, cluster_bar, 0, atom);
}

// BLK = false: scales per 1x32 block (MXFP8): one atom per 128 rows and K block, scale byte k of the
// atom for the k-th MMA of the K block. BLK = true: scales per 128x128 block: one atom per 128 rows
// and FOUR K blocks, byte g of the atom holding the scale of K block 4j + g for every row, so the
// scale copies (and their bytes) are needed only every fourth K block and all four MMAs of K block
// kb select byte kb % 4.
template <int MODE, bool BLK, int PAIR>
__global__ void __launch_bounds__(X_THREADS, 1)
mx_gemm_kernel(const __grid_constant__ MxMaps maps, const MxArgs g) {
    constexpr bool GATED = MODE == MX_OUT_GATED;
    constexpr int STAGES = XCfg<PAIR>::STAGES;
    constexpr int STRIDE = XCfg<PAIR>::STAGE_STRIDE;
    constexpr int B_BYTES = XCfg<PAIR>::B_BYTES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
    const int crank = PAIR == 2 ? static_cast<int>(cluster_ctarank()) : 0;
    const int unit = blockIdx.x / PAIR;   // which tile walker this CTA belongs to
    const int nunits = gridDim.x / PAIR;
    const uint32_t ring = smem_base;
    uint8_t* ctrl = smem + STAGES * STRIDE;
    const uint32_t ctrl_u = ring + STAGES * STRIDE;
    const uint32_t bar_full = ctrl_u;                 // STAGES (a pair: both CTAs' bytes, on the leader)
    const uint32_t bar_empty = ctrl_u + 8 * STAGES;   // STAGES
    const uint32_t bar_tfull = ctrl_u + 16 * STAGES;  // 1
    const uint32_t bar_tempty = bar_tfull + 8;        // 1 (a pair: the leader hears both CTAs' epilogues)
    const uint32_t bar_epi = bar_tempty + 8;          // 1
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(ctrl + 16 * STAGES + 32);
    volatile int* abort_sm = reinterpret_cast<volatile int*>(ctrl + 16 * STAGES + 40);
    float* red = reinterpret_cast<float*>(ctrl + 16 * STAGES + 64);  // [2][8]
    int* offs_sm = reinterpret_cast<int*>(ctrl + 256);
    int* cum_sm = offs_sm + (X_MAX_E + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const WaitCtx wc{g.status, abort_sm};

    if (g.offsets != nullptr) {
        for (int e = threadIdx.x; e <= g.E; e += blockDim.x) offs_sm[e] = g.offsets[e];
    } else if (threadIdx.x == 0) {
        offs_sm[0] = 0;
        offs_sm[1] = g.rows_pad;
    }
    if (threadIdx.x == 0) {
        *abort_sm = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_tfull, 1);
        mbar_init(bar_tempty, X_EPI_WARPS * PAIR);
        mbar_init(bar_epi, X_EPI_WARPS);
        fence_mbar_init();
        tma_prefetch_desc(&maps.a);
        tma_prefetch_desc(&maps.b);
        if (PAIR == 2) {
            tma_prefetch_desc(&maps.sfa);
            tma_prefetch_desc(&maps.sfb);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // The offsets come from device memory: a group whose row range is not made of whole
        // 128-row tiles inside the output gets no tiles (and is recorded), so that no role ever
        // forms an address from it.
        int run = 0;
        for (int e = 0; e < g.E; ++e) {
            cum_sm[e] = run;
            const int lo = offs_sm[e], hi = offs_sm[e + 1];
            const bool ok = lo >= 0 && hi >= lo && hi <= g.rows_pad && (lo % XM) == 0 && (hi % XM) == 0;
            if (ok) run += ((hi - lo + XM * PAIR - 1) / (XM * PAIR)) * g.n_tiles;
            else if (blockIdx.x == 0) record_bad_index(g.status, XS_OFFSETS, static_cast<unsigned>(e));
        }
        cum_sm[g.E] = run;
    }
    if (warp == 1) {
        tmem_alloc<PAIR>(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
        tmem_relinquish<PAIR>();
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR == 2) {
        // both CTAs' barriers exist before either signals the other's
        cluster_arrive();
        cluster_wait();
    }
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    MxWalk walk{cum_sm, offs_sm, g.E, 0, XM * PAIR, g.n_tiles, g.band};

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            int e, row0, n, left;
            for (int t = unit; ok && walk.locate(t, e, row0, n, left); t += nunits) {
                const int my_row0 = row0 + crank * XM;  // may lie past the group's rows (see above)
                const int wrow = e * g.w_rows;
                const int wblk = e * g.w_blocks;
                int blk0, blk1, brow;
                if (GATED) {
                    blk0 = wblk + n;
                    blk1 = wblk + g.N / 128 + n;
                    brow = PAIR == 2 ? (crank == 0 ? wrow + n * 128 : wrow + g.N + n * 128) : wrow + n * 128;
                } else {
                    blk0 = wblk + 2 * n;
                    blk1 = blk0 + 1;
                    brow = wrow + n * XN + crank * XCfg<PAIR>::B_ROWS;
                }
                if (blk0 >= g.sfb_blocks) blk0 = g.sfb_blocks - 1;
                if (blk1 >= g.sfb_blocks) blk1 = g.sfb_blocks - 1;
                int ablk = my_row0 / XM;
                if (ablk >= g.sfa_blocks) ablk = g.sfa_blocks - 1;
                const int atoms_k = BLK ? (g.num_kb + 3) / 4 : g.num_kb;  // atoms per 128-row block
                for (int kb = 0; kb < g.num_kb; ++kb) {
                    if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, wc, XS_EMPTY, t)) {
                        ok = false;
                        break;
                    }
                    const uint32_t full = bar_full + 8 * s;
                    const bool with_sf = !BLK || (kb & 3) == 0;
                    const uint32_t tx = with_sf ? XCfg<PAIR>::STAGE_TX : XA_BYTES + B_BYTES;
                    const uint32_t st = ring + s * STRIDE;
                    const uint32_t sf = st + XA_BYTES + B_BYTES;
                    const int ai = BLK ? kb >> 2 : kb;
                    if (PAIR == 2) {
                        // both CTAs' loads complete on the LEADER's barrier, which expects the bytes
                        // of both; the follower's bytes may land before the leader has announced them
                        const uint32_t lead_full = mapa_shared(full, 0);
                        if (crank == 0) mbar_expect_tx(full, 2 * tx);
                        tma_load_2d_pair(st, &maps.a, lead_full, kb * XK, my_row0);
                        tma_load_2d_pair(st + XA_BYTES, &maps.b, lead_full, kb * XK, brow);
                        if (with_sf) {
                            tma_load_atom_pair(sf, &maps.sfa, lead_full, ablk * atoms_k + ai);
                            tma_load_atom_pair(sf + X_ATOM, &maps.sfb, lead_full, blk0 * atoms_k + ai);
                            tma_load_atom_pair(sf + 2 * X_ATOM, &maps.sfb, lead_full, blk1 * atoms_k + ai);
                        }
                    } else {
                        mbar_expect_tx(full, tx);
                        tma_load_2d(st, &maps.a, full, kb * XK, my_row0);
                        if (GATED) {
                            tma_load_2d(st + XA_BYTES, &maps.b, full, kb * XK, brow);
                            tma_load_2d(st + XA_BYTES + B_BYTES / 2, &maps.b, full, kb * XK, wrow + g.N + n * 128);
                        } else {
                            tma_load_2d(st + XA_BYTES, &maps.b, full, kb * XK, brow);
                        }
                        if (with_sf) {
                            const size_t ao = static_cast<size_t>(ai) * X_ATOM;
                            bulk_load_1d(sf, g.sfa + static_cast<size_t>(ablk) * atoms_k * X_ATOM + ao, X_ATOM, full);
                            bulk_load_1d(sf + X_ATOM, g.sfb + static_cast<size_t>(blk0) * atoms_k * X_ATOM + ao, X_ATOM, full);
                            bulk_load_1d(sf + 2 * X_ATOM, g.sfb + static_cast<size_t>(blk1) * atoms_k * X_ATOM + ao, X_ATOM,
                                         full);
                        }
                    }
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- scale copies + MMA issuer
        // (the follower of a pair issues nothing: its operands complete on the leader's barrier)
        if (lane == 0 && crank == 0) {
            int s = 0;
            uint32_t ph = 0, acc_ph = 0;
            const uint32_t sfa_t = tmem_base + X_SF_COL;
            const uint32_t sfb_t = tmem_base + X_SF_COL + 4;
            bool ok = true;
            int e, row0, n, left;
            for (int t = unit; ok && walk.locate(t, e, row0, n, left); t += nunits) {
                if (!mbar_wait(bar_tempty, acc_ph ^ 1, wc, XS_TEMPTY, t)) break;
                tc_fence_after();
                for (int kb = 0; kb < g.num_kb; ++kb) {
                    if (!mbar_wait(bar_full + 8 * s, ph, wc, XS_FULL, t)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t st = ring + s * STRIDE;
                    const uint32_t sf = st + XA_BYTES + B_BYTES;
                    // The scale columns are rewritten in place: tcgen05.cp and tcgen05.mma of one
                    // thread execute in issue order, so the copies wait for the previous MMAs and
                    // these MMAs for the copies. The copies occupy the tensor pipe: three per K
                    // block measured 10-20 % of the kernel depending on the board. Tried and
                    // measured no better or worse: separate scale columns per stage, a thread of
                    // their own for the copies, copies issued one K block ahead of their MMAs into a
                    // second set of columns, whether waiting for the next stage (2.6 -> 2.3 PFLOP/s)
                    // or only when it has already landed (2.38 -> 2.20).
                    if (!BLK || (kb & 3) == 0) {
                        tmem_cp_32x128b_warpx4<PAIR>(sfa_t, umma_desc_sf_atom(sf));
                        tmem_cp_32x128b_warpx4<PAIR>(sfb_t, umma_desc_sf_atom(sf + X_ATOM));
                        tmem_cp_32x128b_warpx4<PAIR>(sfb_t + 4, umma_desc_sf_atom(sf + 2 * X_ATOM));
                    }
                    const uint64_t da = umma_desc_sw128(st);
                    const uint64_t db = umma_desc_sw128(st + XA_BYTES);
#pragma unroll
                    for (int k = 0; k < XK / 32; ++k)
                        umma_mxf8<PAIR>(tmem_base, da + 2 * k, db + 2 * k,
                                        umma_idesc_mx(XM * PAIR, XN, BLK ? (kb & 3) : k), sfa_t, sfb_t, (kb | k) != 0);
                    if (PAIR == 2) umma_commit_pair(bar_empty + 8 * s, 3);
                    else umma_commit<1>(bar_empty + 8 * s);
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (!ok) break;
                if (PAIR == 2) umma_commit_pair(bar_tfull, 3);
                else umma_commit<1>(bar_tfull);
                acc_ph ^= 1;
            }
        }
    } else if (warp >= 4) {
        // ---------------------------------------------------------------- epilogue
        const int ew = warp - 4;  // 0..7
        const bool remote = PAIR == 2 && crank != 0;
        const uint32_t tempty = remote ? mapa_shared(bar_tempty, 0) : bar_tempty;
        uint32_t acc_ph = 0;
        unsigned tiles_done = 0;
        int e, row0, n, left;
        for (int t = unit; walk.locate(t, e, row0, n, left); t += nunits, ++tiles_done) {
            if (!__all_sync(0xffffffffu, mbar_wait(bar_tfull, acc_ph, wc, XS_TFULL, t))) break;
            acc_ph ^= 1;
            tc_fence_after();
            const bool store = crank * XM < left;  // this CTA's 128 rows exist
            if (!mx_epilogue_tile<MODE>(g, wc, tmem_base, tempty, remote, bar_epi, red, ew, lane, row0 + crank * XM, n,
                                        store, tiles_done, t))
                break;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (PAIR == 2) {
        // neither CTA leaves (or frees the pair's tensor memory) while the other may still signal it
        cluster_arrive();
        cluster_wait();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        if (*abort_sm) {
            // give copies still in flight time to land before the shared memory goes away
            const uint64_t t0 = globaltimer_ns();
            while (globaltimer_ns() - t0 < 200000ull) {
            }
        }
        tmem_dealloc<PAIR>(tmem_base, 512);
    }
}

}  // namespace dk
