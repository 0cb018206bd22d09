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
// The kernel itself (one-CTA and two-CTA forms) is in dk_mx_kernel.cuh.
#include "dk_mx_kernel.cuh"

namespace dk {

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

// pair != 0: clusters of two CTAs per 256-row tile (cta_group::2); `tiles` then counts pair tiles.
template <int MODE, bool BLK, int PAIR>
static int launch_mx_p(const MxMaps& maps, const MxArgs& g, int max_tiles, cudaStream_t st) {
    static bool attr_set[64] = {};
    int dev = 0;
    DK_CUDA_OK(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        DK_CUDA_OK(cudaFuncSetAttribute(mx_gemm_kernel<MODE, BLK, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        XCfg<PAIR>::SMEM_BYTES));
        attr_set[dev & 63] = true;
    }
    int sms = 0;
    int rc = sm_count(&sms);
    if (rc != DK_OK) return rc;
    const int units = sms / PAIR;
    const int grid = (max_tiles < units ? max_tiles : units) * PAIR;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(X_THREADS);
    cfg.dynamicSmemBytes = XCfg<PAIR>::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = PAIR;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    DK_CUDA_OK(cudaLaunchKernelEx(&cfg, mx_gemm_kernel<MODE, BLK, PAIR>, maps, g));
    return DK_OK;
}

// -1 (default, or DK_MX_PAIR unset): pairs for the plain GEMM, one CTA per tile for the grouped GEMMs;
// 0 / 1 (dk_mx_pair_mode, DK_MX_PAIR): one form for both. The pair form moves 30 % fewer bytes
// through L1/L2; on the plain GEMM it measured 0-5 % faster depending on the board, on many small
// experts it loses (an odd number of 128-row tiles leaves half a pair idle).
static int g_mx_pair = -2;
static bool mx_use_pair(bool grouped) {
    if (g_mx_pair == -2) {
        const char* e = std::getenv("DK_MX_PAIR");
        g_mx_pair = (e && *e) ? (std::atoi(e) != 0 ? 1 : 0) : -1;
    }
    return g_mx_pair == 1 || (g_mx_pair == -1 && !grouped);
}

// [atoms, 128 x u32] view of a scale-atom array for tensor-map loads of whole atoms (no swizzle).
static int make_atom_map(CUtensorMap* out, const void* base, size_t n_atoms) {
    const DriverApi* api;
    int rc = driver_api(&api);
    if (rc != DK_OK) return rc;
    cuuint64_t dims[2] = {128, n_atoms};
    cuuint64_t strides[1] = {X_ATOM};
    cuuint32_t box[2] = {128, 1};
    cuuint32_t estr[2] = {1, 1};
    DK_CU_OK(api->cuTensorMapEncodeTiled(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides,
                                         box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    return DK_OK;
}

// Fills the maps for either form and launches. b_rows_total: rows of the whole B matrix.
template <int MODE, bool BLK>
static int launch_mx(MxMaps& maps, MxArgs& g, const void* aq, int a_rows, const void* bq, uint64_t b_rows_total,
                     int row_tiles_upper, cudaStream_t st) {
    const bool pair = mx_use_pair(g.offsets != nullptr);
    // rows of A that stay in L2 while all column tiles of a band pass (a quarter of L2)
    g.band = walk_band_tiles(XM * (pair ? 2 : 1), g.K);  // dk_host.cu
    int rc = make_tmap_2d(&maps.a, aq, 1, g.K, a_rows, g.K, XK, XM);
    if (rc != DK_OK) return rc;
    const bool gated = MODE == MX_OUT_GATED;
    rc = make_tmap_2d(&maps.b, bq, 1, g.K, b_rows_total, g.K, XK, (pair || gated) ? 128 : XN);
    if (rc != DK_OK) return rc;
    const size_t atoms_k = BLK ? (g.num_kb + 3) / 4 : g.num_kb;
    if (pair) {
        rc = make_atom_map(&maps.sfa, g.sfa, static_cast<size_t>(g.sfa_blocks) * atoms_k);
        if (rc != DK_OK) return rc;
        rc = make_atom_map(&maps.sfb, g.sfb, static_cast<size_t>(g.sfb_blocks) * atoms_k);
        if (rc != DK_OK) return rc;
        // every group may end in a half-filled pair tile
        const int pair_tiles = (row_tiles_upper + g.E + 1) / 2;
        return launch_mx_p<MODE, BLK, 2>(maps, g, pair_tiles * g.n_tiles, st);
    }
    maps.sfa = maps.a;
    maps.sfb = maps.a;
    return launch_mx_p<MODE, BLK, 1>(maps, g, row_tiles_upper * g.n_tiles, st);
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
    g.sfa_blocks = (M + 127) / 128;
    g.sfb_blocks = g.w_blocks;
    g.R = M;
    g.rows_pad = (M + XM - 1) / XM * XM;
    g.out = C;
    int rc = device_status_ptr(&g.status);
    if (rc != DK_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return out_f32 ? launch_mx<MX_OUT_F32, false>(maps, g, aq, M, bq, N, g.rows_pad / XM, st)
                   : launch_mx<MX_OUT_BF16, false>(maps, g, aq, M, bq, N, g.rows_pad / XM, st);
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
    g.sfa_blocks = R / 128;
    g.sfb_blocks = E * g.w_blocks;
    g.R = R;
    g.rows_pad = R;
    g.out = out;
    g.out_e8 = static_cast<uint8_t*>(out_e8);
    g.out_atoms = static_cast<uint8_t*>(out_atoms);
    int rc = device_status_ptr(&g.status);
    if (rc != DK_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint64_t b_rows = static_cast<uint64_t>(E) * w_rows;
    return gated ? launch_mx<MX_OUT_GATED, true>(maps, g, xq, R, wq, b_rows, R / XM, st)
                 : launch_mx<MX_OUT_BF16, true>(maps, g, xq, R, wq, b_rows, R / XM, st);
}

int dk_mx_pair_mode(int mode) {
    if (mode < -1 || mode > 1) {
        dk::set_last_error("argument error: mode must be -1 (automatic), 0 or 1");
        return DK_ERR_ARG;
    }
    dk::g_mx_pair = mode;
    return DK_OK;
}

}  // extern "C"
