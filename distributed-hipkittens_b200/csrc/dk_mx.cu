// Block-scaled fp8 GEMMs on the tensor core's own scaling path (tcgen05.mma.kind::mxf8f6f4.block_scale),
// sm_100a: e4m3 operands with one e8m0 (power-of-two) scale per row and per 32 elements of K, applied
// by the hardware while it accumulates the whole K extent in tensor memory.
//
//   dk_mx_quant          x (bf16 or fp32) -> e4m3 bytes + e8m0 scales per 1x32 block
//   dk_gemm_mxfp8        C[M,N] = dequant(A) dequant(B)^T, the MXFP8 GEMM
//   dk_moe_grouped_gemm_mxfp8   the MoE grouped GEMM (plain, or gate/up fused with SiLU*mul and
//                        requantisation) on the same instruction, for power-of-two 128x128 block
//                        scales: the four scale bytes the hardware holds per row then carry four
//                        consecutive K blocks, so scales are refreshed every fourth K block only
//
// Stands in for the reference's MXFP8 GEMM: host quantiser compute_e8m0 + quantisation loop
// (kernels/cdna4/gemm/mxfp8/MXFP8_8wave/8_wave_NT.cu:286-327), kernel with per-K-iteration packed
// scales fed to the scaled MFMA (:39-44, :432-496), and its register-tile fixture
// (tests/unit/cdna4/warp/register/tile/mma_scaled.cu:107-320). Same number format (e4m3 x e8m0 per
// 1x32 block), nothing of the mechanism: there the scales travel through registers into
// v_mfma_scale; here they are staged as 512-byte atoms in shared memory, copied to tensor memory
// with tcgen05.cp, and the MMA reads them from there.
//
//   warp 0      TMA producer: A tile 128 rows x 128 K-bytes, B tile 256 rows x 128 K-bytes
//               (128-byte swizzle) and three scale atoms (one for A, two for B) per stage, 4 stages
//   warp 1      per stage: three tcgen05.cp (atoms -> 12 tensor-memory columns), four
//               tcgen05.mma (K = 32 each, scale byte k selected by the instruction descriptor),
//               accumulating over all of K into one 256-column accumulator
//   warps 4-11  epilogue: tcgen05.ld, then bf16 / fp32 stores, or SiLU(gate)*up, tile-wide amax,
//               power-of-two scale, e4m3 bytes + scale atom (the 128x128 output tile is exactly one
//               scale block of the next GEMM's A operand)
//
// Scales need tensor-memory columns too, so there is one accumulator (256 + 12 of the 512
// columns): the epilogue of a tile is not overlapped with the next tile's MMAs. It costs one drain
// (a few hundred cycles) per K/128 * 512 cycles of MMAs.
#include <cuda_fp8.h>

#include "dk_host.h"
#include "dk_ptx.cuh"

namespace dk {

constexpr int XM = 128;
constexpr int XN = 256;
constexpr int XK = 128;  // bytes = e4m3 elements per K block = one swizzle row = four scale groups
constexpr int X_STAGES = 4;
constexpr int XA_BYTES = XM * XK;
constexpr int XB_BYTES = XN * XK;
constexpr int X_ATOM = 512;
constexpr int X_STAGE_TX = XA_BYTES + XB_BYTES + 3 * X_ATOM;
constexpr int X_STAGE_STRIDE = 50 * 1024;  // keeps every stage 1024-byte aligned
constexpr int X_MAX_E = 256;
constexpr int X_CTRL_BYTES = 256 + (X_MAX_E + 1) * 4 * 2 + 128;
constexpr int X_SMEM_BYTES = 1024 + X_STAGES * X_STAGE_STRIDE + X_CTRL_BYTES;
constexpr int X_THREADS = 384;
constexpr int X_EPI_WARPS = 8;
constexpr int X_SF_COL = 256;  // tensor-memory columns 256..259: scales of A, 260..267: scales of B

enum : int { MX_OUT_BF16 = 0, MX_OUT_F32 = 1, MX_OUT_GATED = 2 };

struct MxMaps {
    CUtensorMap a;  // A [rows, K] bytes, box 128 x 128
    CUtensorMap b;  // B [rows, K] bytes, box 128 x (gated ? 128 : 256)
};

struct MxArgs {
    const int* offsets;   // [E+1] device (multiples of 128), or null: one group of rows_pad rows
    const uint8_t* sfa;   // scale atoms of A: [row blocks][K/128][512]; block mode: [row blocks][ceil(K/512)][512]
    const uint8_t* sfb;   // scale atoms of B, likewise
    int E, K, N;          // N: output columns (gated: F)
    int num_kb;           // K / 128
    int n_tiles;          // gated: F/128, plain: ceil(N/256)
    int w_rows;           // rows of one group's B matrix: gated 2F, plain N
    int w_blocks;         // 128-row blocks of one group's B matrix
    int sfb_blocks;       // 128-row blocks in sfb altogether (atom indices are clamped to it)
    int R;                // rows of the output that exist
    int rows_pad;         // R rounded up to 128 (used when offsets is null)
    void* out;            // bf16 / fp32 [R, N], or e4m3 bytes [R, F]
    uint8_t* out_e8;      // gated: e8m0 scale per 128x128 block [R/128, F/128]
    uint8_t* out_atoms;   // gated: the same scales as block-mode atoms [R/128][ceil(F/512)][512]
    unsigned* status;
};

enum : unsigned { XS_EMPTY = 64, XS_FULL = 65, XS_TEMPTY = 66, XS_TFULL = 67, XS_EPI = 68, XS_OFFSETS = 69 };

// Tile walk shared by all roles: tile t -> (group, first row, column tile). Row tiles fastest, so
// CTAs running together share one B tile in L2.
struct MxWalk {
    const int* cum;   // [E+1] in shared memory: tiles before group e
    const int* offs;  // [E+1] in shared memory
    int E, e;
    __device__ __forceinline__ bool locate(int t, int& group, int& row0, int& n) {
        if (t >= cum[E]) return false;
        while (t >= cum[e + 1]) ++e;
        const int local = t - cum[e];
        const int mt = (offs[e + 1] - offs[e]) / XM;
        group = e;
        row0 = offs[e] + (local % mt) * XM;
        n = local / mt;
        return true;
    }
};

__device__ __forceinline__ float mx_rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// BLK = false: scales per 1x32 block (MXFP8): one atom per 128 rows and K block, scale byte k of the
// atom for the k-th MMA of the K block. BLK = true: scales per 128x128 block: one atom per 128 rows
// and FOUR K blocks, byte g of the atom holding the scale of K block 4j + g for every row, so the
// scale copies (and their bytes) are needed only every fourth K block and all four MMAs of K block
// kb select byte kb % 4.
template <int MODE, bool BLK>
__global__ void __launch_bounds__(X_THREADS, 1)
mx_gemm_kernel(const __grid_constant__ MxMaps maps, const MxArgs g) {
    constexpr bool GATED = MODE == MX_OUT_GATED;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t ring = smem_base;
    uint8_t* ctrl = smem + X_STAGES * X_STAGE_STRIDE;
    const uint32_t ctrl_u = ring + X_STAGES * X_STAGE_STRIDE;
    const uint32_t bar_full = ctrl_u;                   // X_STAGES
    const uint32_t bar_empty = ctrl_u + 8 * X_STAGES;   // X_STAGES
    const uint32_t bar_tfull = ctrl_u + 16 * X_STAGES;  // 1
    const uint32_t bar_tempty = bar_tfull + 8;          // 1
    const uint32_t bar_epi = bar_tempty + 8;            // 1
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(ctrl + 16 * X_STAGES + 32);
    volatile int* abort_sm = reinterpret_cast<volatile int*>(ctrl + 16 * X_STAGES + 40);
    float* red = reinterpret_cast<float*>(ctrl + 16 * X_STAGES + 64);  // [2][8]
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
        for (int s = 0; s < X_STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_tfull, 1);
        mbar_init(bar_tempty, X_EPI_WARPS);
        mbar_init(bar_epi, X_EPI_WARPS);
        fence_mbar_init();
        tma_prefetch_desc(&maps.a);
        tma_prefetch_desc(&maps.b);
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
            if (ok) run += ((hi - lo) / XM) * g.n_tiles;
            else if (blockIdx.x == 0) record_bad_index(g.status, XS_OFFSETS, static_cast<unsigned>(e));
        }
        cum_sm[g.E] = run;
    }
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
        tmem_relinquish<1>();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    MxWalk walk{cum_sm, offs_sm, g.E, 0};

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            int e, row0, n;
            for (int t = blockIdx.x; ok && walk.locate(t, e, row0, n); t += gridDim.x) {
                const int wrow = e * g.w_rows;
                const int wblk = e * g.w_blocks;
                int blk0, blk1;
                if (GATED) {
                    blk0 = wblk + n;
                    blk1 = wblk + g.N / 128 + n;
                } else {
                    blk0 = wblk + 2 * n;
                    blk1 = blk0 + 1;
                }
                if (blk0 >= g.sfb_blocks) blk0 = g.sfb_blocks - 1;
                if (blk1 >= g.sfb_blocks) blk1 = g.sfb_blocks - 1;
                const int atoms_k = BLK ? (g.num_kb + 3) / 4 : g.num_kb;  // atoms per 128-row block
                const uint8_t* sfa_p = g.sfa + static_cast<size_t>(row0 / XM) * atoms_k * X_ATOM;
                const uint8_t* sfb0_p = g.sfb + static_cast<size_t>(blk0) * atoms_k * X_ATOM;
                const uint8_t* sfb1_p = g.sfb + static_cast<size_t>(blk1) * atoms_k * X_ATOM;
                for (int kb = 0; kb < g.num_kb; ++kb) {
                    if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, wc, XS_EMPTY, t)) {
                        ok = false;
                        break;
                    }
                    const uint32_t full = bar_full + 8 * s;
                    const bool with_sf = !BLK || (kb & 3) == 0;
                    mbar_expect_tx(full, with_sf ? X_STAGE_TX : XA_BYTES + XB_BYTES);
                    const uint32_t st = ring + s * X_STAGE_STRIDE;
                    tma_load_2d(st, &maps.a, full, kb * XK, row0);
                    if (GATED) {
                        tma_load_2d(st + XA_BYTES, &maps.b, full, kb * XK, wrow + n * 128);
                        tma_load_2d(st + XA_BYTES + XB_BYTES / 2, &maps.b, full, kb * XK, wrow + g.N + n * 128);
                    } else {
                        tma_load_2d(st + XA_BYTES, &maps.b, full, kb * XK, wrow + n * XN);
                    }
                    const uint32_t sf = st + XA_BYTES + XB_BYTES;
                    if (with_sf) {
                        const size_t ai = static_cast<size_t>(BLK ? kb >> 2 : kb) * X_ATOM;
                        bulk_load_1d(sf, sfa_p + ai, X_ATOM, full);
                        bulk_load_1d(sf + X_ATOM, sfb0_p + ai, X_ATOM, full);
                        bulk_load_1d(sf + 2 * X_ATOM, sfb1_p + ai, X_ATOM, full);
                    }
                    if (++s == X_STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- scale copies + MMA issuer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0, acc_ph = 0;
            const uint32_t sfa_t = tmem_base + X_SF_COL;
            const uint32_t sfb_t = tmem_base + X_SF_COL + 4;
            bool ok = true;
            int e, row0, n;
            for (int t = blockIdx.x; ok && walk.locate(t, e, row0, n); t += gridDim.x) {
                if (!mbar_wait(bar_tempty, acc_ph ^ 1, wc, XS_TEMPTY, t)) break;
                tc_fence_after();
                for (int kb = 0; kb < g.num_kb; ++kb) {
                    if (!mbar_wait(bar_full + 8 * s, ph, wc, XS_FULL, t)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t st = ring + s * X_STAGE_STRIDE;
                    const uint32_t sf = st + XA_BYTES + XB_BYTES;
                    // The scale columns are rewritten in place: tcgen05.cp and tcgen05.mma of one
                    // thread execute in issue order, so the copies wait for the previous MMAs and
                    // these MMAs for the copies. (The copies occupy the tensor pipe: three per K
                    // block measured 10 % of the kernel; separate columns per stage or a thread of
                    // their own for the copies changed nothing.)
                    if (!BLK || (kb & 3) == 0) {
                        tmem_cp_32x128b_warpx4<1>(sfa_t, umma_desc_sf_atom(sf));
                        tmem_cp_32x128b_warpx4<1>(sfb_t, umma_desc_sf_atom(sf + X_ATOM));
                        tmem_cp_32x128b_warpx4<1>(sfb_t + 4, umma_desc_sf_atom(sf + 2 * X_ATOM));
                    }
                    const uint64_t da = umma_desc_sw128(st);
                    const uint64_t db = umma_desc_sw128(st + XA_BYTES);
#pragma unroll
                    for (int k = 0; k < XK / 32; ++k)
                        umma_mxf8<1>(tmem_base, da + 2 * k, db + 2 * k, umma_idesc_mx(XM, XN, BLK ? (kb & 3) : k),
                                     sfa_t, sfb_t, (kb | k) != 0);
                    umma_commit<1>(bar_empty + 8 * s);
                    if (++s == X_STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (!ok) break;
                umma_commit<1>(bar_tfull);
                acc_ph ^= 1;
            }
        }
    } else if (warp >= 4) {
        // ---------------------------------------------------------------- epilogue
        const int ew = warp - 4;  // 0..7
        const int q = warp & 3;   // tensor-memory lane quarter of this warp
        const int h = ew >> 2;    // which half of the columns
        uint32_t acc_ph = 0;
        unsigned tiles_done = 0;
        int e, row0, n;
        for (int t = blockIdx.x; walk.locate(t, e, row0, n); t += gridDim.x, ++tiles_done) {
            if (!__all_sync(0xffffffffu, mbar_wait(bar_tfull, acc_ph, wc, XS_TFULL, t))) break;
            acc_ph ^= 1;
            tc_fence_after();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
            const int row = row0 + q * 32 + lane;
            if (GATED) {
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
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_tempty);
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
                if (!__all_sync(0xffffffffu, mbar_wait(bar_epi, tiles_done & 1, wc, XS_EPI, t))) break;
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
                    uint8_t* atom = g.out_atoms +
                                    (static_cast<size_t>(row0 / XM) * ((fb + 3) / 4) + (n >> 2)) * X_ATOM + (n & 3);
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
                        *reinterpret_cast<uint4*>(dst + 16 * j) =
                            make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
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
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_tempty);
                    }
                    if (row < g.R) {
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
                                __nv_bfloat16* dst =
                                    static_cast<__nv_bfloat16*>(g.out) + static_cast<size_t>(row) * g.N + col0;
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
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        if (*abort_sm) {
            // give copies still in flight time to land before the shared memory goes away
            const uint64_t t0 = globaltimer_ns();
            while (globaltimer_ns() - t0 < 200000ull) {
            }
        }
        tmem_dealloc<1>(tmem_base, 512);
    }
}

// ------------------------------------------------------------------------------------ quantiser
// One thread per 1x32 block. scale byte = clamp(floor(log2(amax)) + 127, 0, 254), 0 for an
// all-zero block; q = e4m3(x * 2^(127 - scale)) (round to nearest even, saturating): the block
// maximum lands in [1, 2). Scales are written row-major [R, K/32] (optional) and as atoms
// [ceil(R/128)][K/128][r0 = row % 32][r1 = (row % 128) / 32][k].
template <typename T>
__device__ __forceinline__ void mx_load32(const T* src, float (&f)[32]);
template <>
__device__ __forceinline__ void mx_load32<__nv_bfloat16>(const __nv_bfloat16* src, float (&f)[32]) {
    const uint4* p = reinterpret_cast<const uint4*>(src);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 v = p[i];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 t = __bfloat1622float2(h[j]);
            f[8 * i + 2 * j] = t.x;
            f[8 * i + 2 * j + 1] = t.y;
        }
    }
}
template <>
__device__ __forceinline__ void mx_load32<float>(const float* src, float (&f)[32]) {
    const float4* p = reinterpret_cast<const float4*>(src);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 v = p[i];
        f[4 * i] = v.x;
        f[4 * i + 1] = v.y;
        f[4 * i + 2] = v.z;
        f[4 * i + 3] = v.w;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) mx_quant_kernel(const T* __restrict__ x, int R, int K,
                                                       uint8_t* __restrict__ q, uint8_t* __restrict__ s_rows,
                                                       uint8_t* __restrict__ atoms) {
    const int SK = K / 32, KB = K / 128;
    const size_t nblk = static_cast<size_t>(R) * SK;
    for (size_t b = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; b < nblk;
         b += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int row = static_cast<int>(b / SK), kg = static_cast<int>(b % SK);
        float f[32];
        mx_load32<T>(x + static_cast<size_t>(row) * K + kg * 32, f);
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(f[i]));
        int e = 0;
        if (amax != 0.f) {
            int ex;
            (void)frexpf(amax, &ex);  // amax = m * 2^ex with m in [0.5, 1): floor(log2(amax)) = ex - 1
            e = min(max(ex - 1 + 127, 0), 254);
        }
        const float inv = ldexpf(1.0f, 127 - e);
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t lo =
                __nv_cvt_float2_to_fp8x2(make_float2(f[4 * i] * inv, f[4 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * i + 2] * inv, f[4 * i + 3] * inv),
                                                         __NV_SATFINITE, __NV_E4M3);
            w[i] = lo | (hi << 16);
        }
        uint4* dst = reinterpret_cast<uint4*>(q + static_cast<size_t>(row) * K + kg * 32);
        dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
        dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
        if (s_rows != nullptr) s_rows[static_cast<size_t>(row) * SK + kg] = static_cast<uint8_t>(e);
        const int rb = row >> 7, r1 = (row & 127) >> 5, r0 = row & 31;
        atoms[((static_cast<size_t>(rb) * KB + (kg >> 2)) * 32 + r0) * 16 + r1 * 4 + (kg & 3)] =
            static_cast<uint8_t>(e);
    }
}

template <int MODE, bool BLK>
static int launch_mx(const MxMaps& maps, const MxArgs& g, int max_tiles, cudaStream_t st) {
    static bool attr_set[64] = {};
    int dev = 0;
    DK_CUDA_OK(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        DK_CUDA_OK(cudaFuncSetAttribute(mx_gemm_kernel<MODE, BLK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        X_SMEM_BYTES));
        attr_set[dev & 63] = true;
    }
    int sms = 0;
    int rc = sm_count(&sms);
    if (rc != DK_OK) return rc;
    const int grid = max_tiles < sms ? max_tiles : sms;
    mx_gemm_kernel<MODE, BLK><<<grid, X_THREADS, X_SMEM_BYTES, st>>>(maps, g);
    DK_CUDA_OK(cudaGetLastError());
    return DK_OK;
}

}  // namespace dk

extern "C" {

size_t dk_mx_sf_bytes(int R, int K) {
    if (R <= 0 || K <= 0 || K % 128 != 0) return 0;
    return static_cast<size_t>((R + 127) / 128) * (K / 128) * dk::X_ATOM;
}

int dk_mx_quant(const void* x, int x_is_f32, int R, int K, void* q, void* s_rows, void* sf_atoms, void* stream) {
    using namespace dk;
    DK_REQUIRE(x != nullptr && q != nullptr && sf_atoms != nullptr, "null buffer");
    DK_REQUIRE(R > 0 && K > 0 && K % 128 == 0, "K must be a positive multiple of 128");
    DK_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0,
               "buffers must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // rows of the last 128-row block that do not exist keep scale byte 0
    DK_CUDA_OK(cudaMemsetAsync(sf_atoms, 0, dk_mx_sf_bytes(R, K), st));
    const size_t nblk = static_cast<size_t>(R) * (K / 32);
    int sms = 0;
    int rc = sm_count(&sms);
    if (rc != DK_OK) return rc;
    size_t nb = (nblk + 255) / 256;
    if (nb > static_cast<size_t>(sms) * 8) nb = static_cast<size_t>(sms) * 8;
    if (x_is_f32)
        mx_quant_kernel<float><<<static_cast<unsigned>(nb), 256, 0, st>>>(
            static_cast<const float*>(x), R, K, static_cast<uint8_t*>(q), static_cast<uint8_t*>(s_rows),
            static_cast<uint8_t*>(sf_atoms));
    else
        mx_quant_kernel<__nv_bfloat16><<<static_cast<unsigned>(nb), 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(x), R, K, static_cast<uint8_t*>(q), static_cast<uint8_t*>(s_rows),
            static_cast<uint8_t*>(sf_atoms));
    DK_CUDA_OK(cudaGetLastError());
    return DK_OK;
}

int dk_gemm_mxfp8(const void* aq, const void* sfa, const void* bq, const void* sfb, void* C, int M, int N, int K,
                  int out_f32, void* stream) {
    using namespace dk;
    DK_REQUIRE(aq && sfa && bq && sfb && C, "null buffer");
    DK_REQUIRE(M > 0 && N > 0 && K > 0, "M, N, K must be positive");
    DK_REQUIRE(K % 128 == 0, "K must be a multiple of 128 (four 32-element scale groups per K block)");
    DK_REQUIRE(N % 8 == 0, "N must be a multiple of 8 (16-byte output vectors)");
    DK_REQUIRE((reinterpret_cast<uintptr_t>(sfa) & 15) == 0 && (reinterpret_cast<uintptr_t>(sfb) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(C) & 15) == 0,
               "scale and output buffers must be 16-byte aligned");
    MxMaps maps;
    MxArgs g{};
    int rc = make_tmap_2d(&maps.a, aq, 1, K, M, K, XK, XM);
    if (rc != DK_OK) return rc;
    rc = make_tmap_2d(&maps.b, bq, 1, K, N, K, XK, XN);
    if (rc != DK_OK) return rc;
    g.offsets = nullptr;
    g.sfa = static_cast<const uint8_t*>(sfa);
    g.sfb = static_cast<const uint8_t*>(sfb);
    g.E = 1;
    g.K = K;
    g.N = N;
    g.num_kb = K / XK;
    g.n_tiles = (N + XN - 1) / XN;
    g.w_rows = N;
    g.w_blocks = (N + 127) / 128;
    g.sfb_blocks = g.w_blocks;
    g.R = M;
    g.rows_pad = (M + XM - 1) / XM * XM;
    g.out = C;
    rc = device_status_ptr(&g.status);
    if (rc != DK_OK) return rc;
    const int tiles = (g.rows_pad / XM) * g.n_tiles;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return out_f32 ? launch_mx<MX_OUT_F32, false>(maps, g, tiles, st) : launch_mx<MX_OUT_BF16, false>(maps, g, tiles, st);
}

int dk_moe_grouped_gemm_mxfp8(const void* xq, const void* x_atoms, const void* wq, const void* w_atoms,
                              const int* offsets, int E, int R, int N, int K, int gated, void* out,
                              void* out_e8, void* out_atoms, void* stream) {
    using namespace dk;
    DK_REQUIRE(E >= 1 && E <= X_MAX_E, "E must be 1..256");
    DK_REQUIRE(R >= 0 && R % 128 == 0, "R must be a multiple of 128");
    DK_REQUIRE(K > 0 && K % 128 == 0, "K must be a multiple of 128");
    DK_REQUIRE(N > 0 && (gated ? N % 128 == 0 : N % 256 == 0),
               "N must be a multiple of 128 (gated: F) or 256 (plain)");
    if (R == 0) return DK_OK;
    DK_REQUIRE(xq && x_atoms && wq && w_atoms && offsets && out, "null buffer");
    DK_REQUIRE(!gated || (out_e8 != nullptr && out_atoms != nullptr), "gated output needs its scale buffers");
    DK_REQUIRE((reinterpret_cast<uintptr_t>(x_atoms) & 15) == 0 && (reinterpret_cast<uintptr_t>(w_atoms) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                   (!gated || (reinterpret_cast<uintptr_t>(out_atoms) & 15) == 0),
               "scale and output buffers must be 16-byte aligned");
    MxMaps maps;
    MxArgs g{};
    const int w_rows = gated ? 2 * N : N;
    int rc = make_tmap_2d(&maps.a, xq, 1, K, R, K, XK, XM);
    if (rc != DK_OK) return rc;
    rc = make_tmap_2d(&maps.b, wq, 1, K, static_cast<uint64_t>(E) * w_rows, K, XK, gated ? 128 : XN);
    if (rc != DK_OK) return rc;
    g.offsets = offsets;
    g.sfa = static_cast<const uint8_t*>(x_atoms);
    g.sfb = static_cast<const uint8_t*>(w_atoms);
    g.E = E;
    g.K = K;
    g.N = N;
    g.num_kb = K / XK;
    g.n_tiles = gated ? N / 128 : N / XN;
    g.w_rows = w_rows;
    g.w_blocks = w_rows / 128;
    g.sfb_blocks = E * g.w_blocks;
    g.R = R;
    g.rows_pad = R;
    g.out = out;
    g.out_e8 = static_cast<uint8_t*>(out_e8);
    g.out_atoms = static_cast<uint8_t*>(out_atoms);
    rc = device_status_ptr(&g.status);
    if (rc != DK_OK) return rc;
    const int tiles = (R / XM) * g.n_tiles;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return gated ? launch_mx<MX_OUT_GATED, true>(maps, g, tiles, st) : launch_mx<MX_OUT_BF16, true>(maps, g, tiles, st);
}

}  // extern "C"
