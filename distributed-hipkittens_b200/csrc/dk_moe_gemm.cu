// fp8 (e4m3) grouped GEMM with 128x128 fp32 block scales for the MoE FFN, sm_100a.
//
//   gated:  H[rows of e, F] = quant( silu(X W1_e^T) * (X W3_e^T) )   X [R,K] e4m3, W13 [E,2F,K] e4m3
//   plain:  Y[rows of e, N] = X W_e^T                                 Y bf16
//
// The reference has no grouped or block-scaled-by-128 GEMM. Its nearest kernels are the unscaled
// fp8 GEMM (kernels/cdna4/gemm/fp8fp32/FP8_8wave/8_wave.cu:17-255), the 1x32-e8m0 MXFP8 GEMM
// (kernels/cdna4/gemm/mxfp8/MXFP8_8wave/8_wave_NT.cu) and the per-row-scaled GEMM whose scales are
// applied in the epilogue (kernels/cdna4/torch_scaled/scaled_matmul.cu:254-265). 128x128 fp32
// scales fit neither hardware block-scaling format, so scaling is done in software:
//
//   warp 0     TMA producer: A tile 128 rows x 128 K-bytes, B tile 256 rows x 128 K-bytes
//              (gated: 128 gate rows + the matching 128 up rows), 128-byte swizzle, 4-stage ring
//   warp 1     MMA issuer: per 128-wide K block, four tcgen05.mma kind::f8f6f4 (128x256x32) into
//              one of two 256-column TMEM buffers, overwriting (no accumulation across K blocks)
//   warps 4-11 promotion + epilogue (warps 2-3 only give up their registers): per K block, tcgen05.ld the partial sums and add them, times
//              sa[m-block,kb] * sb[n-block,kb], to fp32 accumulators kept in registers (each thread
//              owns one row and 128 of the 256 columns), while the MMA warp fills the other buffer.
//              Gated: silu(g)*u, tile-wide amax (the 128x128 tile IS one scale block of the
//              output), requantise to e4m3, store bytes + one scale. Plain: bf16 stores.
//
// Experts own row ranges [offsets[e], offsets[e+1]) that are multiples of 128, read on the device
// (no host synchronisation): CTAs are persistent and walk tiles expert by expert, row-tiles fastest
// so that CTAs running together share one weight tile in L2.
#include <cuda_fp8.h>

#include "dk_host.h"
#include "dk_ptx.cuh"

namespace dk {

constexpr int GM = 128;
constexpr int GN = 256;
constexpr int GK = 128;  // bytes = e4m3 elements per K block = one swizzle row = one scale block
constexpr int G_STAGES = 4;
constexpr int GA_BYTES = GM * GK;
constexpr int GB_BYTES = GN * GK;
constexpr int G_STAGE_BYTES = GA_BYTES + GB_BYTES;
constexpr int G_MAX_E = 256;
constexpr int G_CTRL_BYTES = 256 + (G_MAX_E + 1) * 4 * 2 + 128;
constexpr int G_SMEM_BYTES = 1024 + G_STAGES * G_STAGE_BYTES + G_CTRL_BYTES;
constexpr int G_THREADS = 384;   // warp 0 TMA, warp 1 MMA, warps 2-3 idle, warps 4-11 promotion
constexpr int G_EPI_WARPS = 8;

struct GroupedMaps {
    CUtensorMap a;  // X  [R, K] bytes, box 128 x 128
    CUtensorMap b;  // W  [E*rows_per_expert, K] bytes, box 128 x (gated ? 128 : 256)
};

struct GroupedArgs {
    const int* offsets;  // [E+1] device, multiples of 128
    const float* xs;     // [R/128, K/128]
    const float* ws;     // [E, w_blocks, K/128]
    int E, K, N;         // N: output columns (gated: F)
    int R;               // rows of X and of the output
    int num_kb;          // K / 128
    int n_tiles;         // gated: F/128, plain: N/256
    int band;            // row tiles per band of the tile walk (>= 1)
    int w_rows;          // rows of one expert's weight: gated 2F, plain N
    int w_blocks;        // w_rows / 128
    uint8_t* hq;         // gated out [R, F]
    float* hs;           // gated out scales [R/128, F/128]
    __nv_bfloat16* y;    // plain out [R, N]
    unsigned* status;
    long long* dbg;  // [gridDim.x][DBG_SLOTS] stall counters, or null
};

enum : unsigned { GS_EMPTY = 32, GS_FULL = 33, GS_TEMPTY = 34, GS_TFULL = 35, GS_EPI = 36, GS_OFFSETS = 37 };

// Tile walk shared by all roles: tile t -> (expert, row0, n). cum[e] = tiles before expert e.
struct TileWalk {
    const int* cum;      // [E+1] in shared memory
    const int* offs;     // [E+1] in shared memory
    int E, n_tiles, e, band;
    __device__ __forceinline__ bool locate(int t, int& expert, int& row0, int& n) {
        if (t >= cum[E]) return false;
        while (t >= cum[e + 1]) ++e;
        const int local = t - cum[e];
        const int mt = (offs[e + 1] - offs[e]) / GM;
        expert = e;
        int rt;
        if (mt <= band) {
            rt = local % mt;
            n = local / mt;
        } else {  // band by band: a band's rows of X stay in L2 while all column tiles pass
            const int per_band = band * n_tiles;
            const int b = local / per_band, rem = local - b * per_band;
            const int in_band = min(band, mt - b * band);
            n = rem / in_band;
            rt = b * band + rem - n * in_band;
        }
        row0 = offs[e] + rt * GM;
        return true;
    }
};

__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi) {
    unsigned long long v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(__float_as_uint(lo)), "r"(__float_as_uint(hi)));
    return v;
}
// acc.{lo,hi} += {x0,x1} * s.{lo,hi}: one two-wide fp32 FMA
__device__ __forceinline__ void fma_f32x2(unsigned long long& acc, uint32_t x0, uint32_t x1,
                                          unsigned long long s) {
    unsigned long long v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(x0), "r"(x1));
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(v), "l"(s));
}
__device__ __forceinline__ float rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
// First TMEM column (inside a 256-column buffer) of this thread's chunk c (0..3)
template <bool GATED>
__device__ __forceinline__ int chunk_col(int c, int h) {
    return GATED ? ((c >> 1) * 128 + h * 64 + (c & 1) * 32) : (h * 128 + c * 32);
}

template <bool GATED>
__global__ void __launch_bounds__(G_THREADS, 1)
moe_grouped_gemm_kernel(const __grid_constant__ GroupedMaps maps, const GroupedArgs g) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t ring = smem_base;
    uint8_t* ctrl = smem + G_STAGES * G_STAGE_BYTES;
    const uint32_t ctrl_u = ring + G_STAGES * G_STAGE_BYTES;
    const uint32_t bar_full = ctrl_u;                     // G_STAGES
    const uint32_t bar_empty = ctrl_u + 8 * G_STAGES;     // G_STAGES
    const uint32_t bar_tfull = ctrl_u + 16 * G_STAGES;    // 2
    const uint32_t bar_tempty = bar_tfull + 16;           // 2
    const uint32_t bar_epi = bar_tempty + 16;             // 1
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(ctrl + 16 * G_STAGES + 48);
    volatile int* abort_sm = reinterpret_cast<volatile int*>(ctrl + 16 * G_STAGES + 56);
    float* red = reinterpret_cast<float*>(ctrl + 16 * G_STAGES + 64);  // [2][8]
    int* offs_sm = reinterpret_cast<int*>(ctrl + 256);
    int* cum_sm = offs_sm + (G_MAX_E + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const WaitCtx wc{g.status, abort_sm};
    const long long dbg_t0 = clock64();

    for (int e = threadIdx.x; e <= g.E; e += blockDim.x) offs_sm[e] = g.offsets[e];
    if (threadIdx.x == 0) {
        *abort_sm = 0;
        for (int s = 0; s < G_STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_tfull + 8 * a, 1);
            mbar_init(bar_tempty + 8 * a, G_EPI_WARPS);
        }
        mbar_init(bar_epi, G_EPI_WARPS);
        fence_mbar_init();
        tma_prefetch_desc(&maps.a);
        tma_prefetch_desc(&maps.b);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // The offsets come from device memory: an expert whose row range is not made of whole
        // 128-row tiles inside the output gets no tiles (and is recorded), so that no role ever
        // forms an address from it.
        int run = 0;
        for (int e = 0; e < g.E; ++e) {
            cum_sm[e] = run;
            const int lo = offs_sm[e], hi = offs_sm[e + 1];
            const bool ok = lo >= 0 && hi >= lo && hi <= g.R && (lo % GM) == 0 && (hi % GM) == 0;
            if (ok) run += ((hi - lo) / GM) * g.n_tiles;
            else if (blockIdx.x == 0) record_bad_index(g.status, GS_OFFSETS, static_cast<unsigned>(e));
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
    TileWalk walk{cum_sm, offs_sm, g.E, g.n_tiles, 0, g.band};

    // Registers are re-balanced between the warpgroups: the promotion warps hold 128 accumulators
    // plus 64 values in flight from TMEM, far above the 168 registers a 384-thread block is
    // compiled for (a spill in the K loop costs more than anything else in this kernel), while the
    // TMA and MMA warps need a few dozen.
    // (Each setmaxnreg sits at the head of the branch it governs: placed before a join it would
    // bind the code after the join to the smaller value. The increase can only draw on what this
    // CTA's own warps gave back: 128 x (168 - 40) = 256 x (232 - 168); asking for more blocks for ever.)
    // Tried and measured slower: sixteen promotion warps (four per lane quarter, 64 accumulators and one
    // 32-column load in flight each, 112 registers): Mixtral-shape GEMMs 1419 against 1709 TFLOP/s.
    if (warp < 4) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
      if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            int e, row0, n;
            for (int t = blockIdx.x; ok && walk.locate(t, e, row0, n); t += gridDim.x) {
                const int wrow = e * g.w_rows;
                for (int kb = 0; kb < g.num_kb; ++kb) {
                    if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, wc, GS_EMPTY, t)) {
                        ok = false;
                        break;
                    }
                    const uint32_t full = bar_full + 8 * s;
                    mbar_expect_tx(full, G_STAGE_BYTES);
                    const uint32_t sa = ring + s * G_STAGE_BYTES;
                    tma_load_2d(sa, &maps.a, full, kb * GK, row0);
                    if (GATED) {
                        tma_load_2d(sa + GA_BYTES, &maps.b, full, kb * GK, wrow + n * 128);
                        tma_load_2d(sa + GA_BYTES + GB_BYTES / 2, &maps.b, full, kb * GK,
                                    wrow + g.N + n * 128);
                    } else {
                        tma_load_2d(sa + GA_BYTES, &maps.b, full, kb * GK, wrow + n * GN);
                    }
                    if (++s == G_STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
      } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(0, 0, GM, GN);  // e4m3 x e4m3 -> fp32
            int s = 0;
            uint32_t ph = 0;
            unsigned kbc = 0;  // K blocks issued so far: TMEM buffer = kbc & 1
            bool ok = true;
            long long dbg_tmem = 0, dbg_full = 0;
            int e, row0, n;
            for (int t = blockIdx.x; ok && walk.locate(t, e, row0, n); t += gridDim.x) {
                for (int kb = 0; kb < g.num_kb; ++kb, ++kbc) {
                    const int buf = kbc & 1;
                    long long c0 = clock64();
                    if (!mbar_wait(bar_tempty + 8 * buf, ((kbc >> 1) & 1) ^ 1, wc, GS_TEMPTY, t)) {
                        ok = false;
                        break;
                    }
                    dbg_tmem += clock64() - c0;
                    c0 = clock64();
                    if (!mbar_wait(bar_full + 8 * s, ph, wc, GS_FULL, t)) {
                        ok = false;
                        break;
                    }
                    dbg_full += clock64() - c0;
                    tc_fence_after();
                    const uint32_t sa = ring + s * G_STAGE_BYTES;
                    const uint64_t da = umma_desc_sw128(sa);
                    const uint64_t db = umma_desc_sw128(sa + GA_BYTES);
                    const uint32_t d_tmem = tmem_base + buf * GN;
#pragma unroll
                    for (int k = 0; k < GK / 32; ++k)
                        umma_f8<1>(d_tmem, da + 2 * k, db + 2 * k, idesc, k != 0);
                    umma_commit<1>(bar_empty + 8 * s);
                    umma_commit<1>(bar_tfull + 8 * buf);
                    if (++s == G_STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
            if (g.dbg != nullptr) {
                g.dbg[blockIdx.x * DBG_SLOTS + DBG_MMA_WAIT_TMEM] = dbg_tmem;
                g.dbg[blockIdx.x * DBG_SLOTS + DBG_MMA_WAIT_FULL] = dbg_full;
            }
        }
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
        // ---------------------------------------------------------------- promotion + epilogue
        const int ew = warp - 4;   // 0..7
        const int q = warp & 3;    // TMEM lane quarter of this warp
        const int h = ew >> 2;     // which half of the columns
        const int KB = g.num_kb;
        unsigned kbc = 0;
        unsigned tiles_done = 0;
        int e, row0, n;
        for (int t = blockIdx.x; walk.locate(t, e, row0, n); t += gridDim.x, ++tiles_done) {
            // 128 fp32 accumulators per thread: one row, 128 of the tile's 256 columns
            float acc[128];
#pragma unroll
            for (int i = 0; i < 128; ++i) acc[i] = 0.f;
            const float* sa_p = g.xs + static_cast<size_t>(row0 / GM) * KB;
            const float* sb0_p;
            const float* sb1_p;
            if (GATED) {
                sb0_p = g.ws + (static_cast<size_t>(e) * g.w_blocks + n) * KB;
                sb1_p = g.ws + (static_cast<size_t>(e) * g.w_blocks + g.N / 128 + n) * KB;
            } else {
                sb0_p = g.ws + (static_cast<size_t>(e) * g.w_blocks + 2 * n + h) * KB;
                sb1_p = sb0_p;
            }
            bool ok = true;
            for (int kb = 0; kb < KB; ++kb, ++kbc) {
                const int buf = kbc & 1;
                const float sa = __ldg(sa_p + kb);
                const float s0 = sa * __ldg(sb0_p + kb);
                const float s1 = GATED ? sa * __ldg(sb1_p + kb) : s0;
                if (!__all_sync(0xffffffffu, mbar_wait(bar_tfull + 8 * buf, (kbc >> 1) & 1, wc, GS_TFULL, t))) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * GN;
                // gated: chunks 0,1 = gate columns h*64.., chunks 2,3 = up columns 128 + h*64..
                // A warp drains 32 columns in about 100 cycles whatever the batching, and the FMAs
                // of a K block fill half the FP32 pipe of its scheduler, so the two are interleaved:
                // while chunk c is folded into the accumulators, chunk c+1 is already on its way.
                uint32_t ra[32], rb[32];
                tmem_ld_32x32b_x32(t_row + chunk_col<GATED>(0, h), ra);
                tmem_ld_32x32b_x32(t_row + chunk_col<GATED>(1, h), rb);
                tmem_ld_wait(ra);
                tmem_ld_wait(rb);
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[i] = fmaf(s0, __uint_as_float(ra[i]), acc[i]);
                tmem_ld_32x32b_x32(t_row + chunk_col<GATED>(2, h), ra);
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[32 + i] = fmaf(s0, __uint_as_float(rb[i]), acc[32 + i]);
                tmem_ld_32x32b_x32(t_row + chunk_col<GATED>(3, h), rb);
                tmem_ld_wait(ra);
                tmem_ld_wait(rb);
                // every TMEM read of this buffer has completed: hand it back before the last FMAs
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[64 + i] = fmaf(s1, __uint_as_float(ra[i]), acc[64 + i]);
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[96 + i] = fmaf(s1, __uint_as_float(rb[i]), acc[96 + i]);
            }
            if (!ok) break;

            const int row = row0 + q * 32 + lane;
            if (GATED) {
                // acc[0..63] gate, acc[64..127] up, columns n*128 + h*64 + i
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const float gv = acc[i];
                    const float hv = gv * rcp_approx(1.0f + __expf(-gv)) * acc[64 + i];
                    acc[i] = hv;
                    amax = fmaxf(amax, fabsf(hv));
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                float* red_t = red + (tiles_done & 1) * G_EPI_WARPS;
                if (lane == 0) {
                    red_t[ew] = amax;
                    mbar_arrive(bar_epi);
                }
                if (!__all_sync(0xffffffffu, mbar_wait(bar_epi, tiles_done & 1, wc, GS_EPI, t))) break;
                float tmax = red_t[0];
#pragma unroll
                for (int w = 1; w < G_EPI_WARPS; ++w) tmax = fmaxf(tmax, red_t[w]);
                const float scale = tmax > 0.f ? tmax / 448.0f : 1.0f;
                const float inv_scale = 1.0f / scale;
                if (ew == 0 && lane == 0)
                    g.hs[static_cast<size_t>(row0 / GM) * (g.N / 128) + n] = scale;
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    // two values per conversion instruction; satfinite clamps to +-448 by itself
                    const uint32_t lo = __nv_cvt_float2_to_fp8x2(
                        make_float2(acc[4 * i] * inv_scale, acc[4 * i + 1] * inv_scale), __NV_SATFINITE, __NV_E4M3);
                    const uint32_t hi = __nv_cvt_float2_to_fp8x2(
                        make_float2(acc[4 * i + 2] * inv_scale, acc[4 * i + 3] * inv_scale), __NV_SATFINITE, __NV_E4M3);
                    pk[i] = lo | (hi << 16);
                }
                uint8_t* dst = g.hq + static_cast<size_t>(row) * g.N + n * 128 + h * 64;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    *reinterpret_cast<uint4*>(dst + 16 * j) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
            } else {
                __nv_bfloat16* dst = g.y + static_cast<size_t>(row) * g.N + n * GN + h * 128;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    uint4 o;
                    o.x = pack_bf16x2(acc[8 * j], acc[8 * j + 1]);
                    o.y = pack_bf16x2(acc[8 * j + 2], acc[8 * j + 3]);
                    o.z = pack_bf16x2(acc[8 * j + 4], acc[8 * j + 5]);
                    o.w = pack_bf16x2(acc[8 * j + 6], acc[8 * j + 7]);
                    *reinterpret_cast<uint4*>(dst + 8 * j) = o;
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (g.dbg != nullptr && threadIdx.x == 0) g.dbg[blockIdx.x * DBG_SLOTS + DBG_TOTAL] = clock64() - dbg_t0;
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        if (*abort_sm) {
            const uint64_t t0 = globaltimer_ns();
            while (globaltimer_ns() - t0 < 200000ull) {
            }
        }
        tmem_dealloc<1>(tmem_base, 512);
    }
}

}  // namespace dk

static long long* g_moe_dbg = nullptr;

// Stall accounting as for the bf16 GEMM (see dk_gemm_debug_counters): slots 0-3 and 7 are filled.
extern "C" int dk_moe_gemm_debug_counters(long long* device_buffer) {
    g_moe_dbg = device_buffer;
    return DK_OK;
}

extern "C" int dk_moe_grouped_gemm_fp8(const void* xq, const float* xs, const void* wq, const float* ws,
                                       const int* offsets, int E, int R, int N, int K, int gated,
                                       void* out, float* out_scales, void* stream) {
    using namespace dk;
    DK_REQUIRE(E >= 1 && E <= G_MAX_E, "E must be 1..256");
    DK_REQUIRE(R >= 0 && R % 128 == 0, "R must be a multiple of 128");
    DK_REQUIRE(K > 0 && K % 128 == 0, "K must be a multiple of 128");
    DK_REQUIRE(N > 0 && (gated ? N % 128 == 0 : N % 256 == 0),
               "N must be a multiple of 128 (gated: F) or 256 (plain)");
    if (R == 0) return DK_OK;
    DK_REQUIRE(xq && xs && wq && ws && offsets && out, "null buffer");
    DK_REQUIRE(!gated || out_scales != nullptr, "gated output needs a scale buffer");
    GroupedMaps maps;
    GroupedArgs g{};
    const int w_rows = gated ? 2 * N : N;
    int rc = make_tmap_2d(&maps.a, xq, 1, K, R, K, GK, GM);
    if (rc != DK_OK) return rc;
    rc = make_tmap_2d(&maps.b, wq, 1, K, static_cast<uint64_t>(E) * w_rows, K, GK, gated ? 128 : GN);
    if (rc != DK_OK) return rc;
    g.offsets = offsets;
    g.xs = xs;
    g.ws = ws;
    g.E = E;
    g.K = K;
    g.N = N;
    g.R = R;
    g.num_kb = K / GK;
    g.n_tiles = gated ? N / 128 : N / GN;
    // an expert with more rows than L2 holds is read from DRAM once, not once per column tile
    g.band = walk_band_tiles(GM, K);
    g.w_rows = w_rows;
    g.w_blocks = w_rows / 128;
    g.hq = static_cast<uint8_t*>(out);
    g.hs = out_scales;
    g.y = static_cast<__nv_bfloat16*>(out);
    rc = device_status_ptr(&g.status);
    if (rc != DK_OK) return rc;
    g.dbg = g_moe_dbg;
    int sms = 0;
    rc = sm_count(&sms);
    if (rc != DK_OK) return rc;
    const int max_tiles = (R / GM) * g.n_tiles;
    const int grid = max_tiles < sms ? max_tiles : sms;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    static bool attr_set[2][64] = {};
    int dev = 0;
    DK_CUDA_OK(cudaGetDevice(&dev));
    if (gated) {
        if (!attr_set[1][dev & 63]) {
            DK_CUDA_OK(cudaFuncSetAttribute(moe_grouped_gemm_kernel<true>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM_BYTES));
            attr_set[1][dev & 63] = true;
        }
        moe_grouped_gemm_kernel<true><<<grid, G_THREADS, G_SMEM_BYTES, st>>>(maps, g);
    } else {
        if (!attr_set[0][dev & 63]) {
            DK_CUDA_OK(cudaFuncSetAttribute(moe_grouped_gemm_kernel<false>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM_BYTES));
            attr_set[0][dev & 63] = true;
        }
        moe_grouped_gemm_kernel<false><<<grid, G_THREADS, G_SMEM_BYTES, st>>>(maps, g);
    }
    DK_CUDA_OK(cudaGetLastError());
    return DK_OK;
}
