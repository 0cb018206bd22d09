// Thin inline-PTX layer for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (UMMA + TMEM).
//
// This replaces the role that the reference's CDNA4 tile layer plays for its distributed GEMM
// (include/cdna4/ops/warp/memory/tile/global_to_shared.cuh:13-107 buffer_load->LDS,
//  include/cdna4/ops/warp/register/tile/mma.cuh:13-148 MFMA wrappers): only the roles carry over
// (async global->shared copy, shared->tensor-core contraction); the mechanisms are Blackwell's.
//
// Every wait in this file is bounded: it gives up after DK_WAIT_LIMIT_NS, records where, and
// returns false so that the caller can leave its loop and the kernel can exit cleanly.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#ifndef DK_WAIT_LIMIT_NS
#define DK_WAIT_LIMIT_NS 2000000000ull  // 2 s of wall time per wait
#endif

namespace dk {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n"
        ".reg .b32 %%rx;\n"
        ".reg .pred %%px;\n"
        "elect.sync %%rx|%%px, 0xffffffff;\n"
        "selp.b32 %0, 1, 0, %%px;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrive on an mbarrier that lives in another CTA of the cluster (address from mapa).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.b32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Error record written by the first wait that gives up: {code, block, site, detail}.
// Optional per-CTA stall accounting (clock64 ticks), enabled by handing the kernel a buffer.
enum : int { DBG_MMA_WAIT_TMEM = 0, DBG_MMA_WAIT_FULL, DBG_EPI_WAIT_ACC, DBG_EPI_WAIT_SMEM,
             DBG_EPI_WAIT_LANDED, DBG_RED_WAIT_FLAG, DBG_RED_WORK, DBG_TOTAL, DBG_SLOTS };

struct WaitCtx {
    unsigned* status;        // 4 words in host-mapped memory (may be null)
    volatile int* abort_sm;  // CTA-wide abort flag in shared memory
    // Limit for waits on ANOTHER GPU's signal. These also absorb host-side skew between ranks
    // (a peer whose launch is late), so the limit is a run-time setting, far above the limit for
    // waits inside one CTA.
    unsigned long long peer_limit_ns = 20000000000ull;
};

// DK_DEV_BAD_INDEX: a kernel met an index from device memory (an expert id, a row, an offset) that
// points outside the buffers it was given; it skipped the access and recorded {code, block, site, detail}.
enum : unsigned { DK_DEV_OK = 0, DK_DEV_TIMEOUT = 1, DK_DEV_PEER_TIMEOUT = 2, DK_DEV_BAD_INDEX = 3 };

static __device__ __noinline__ void record_timeout(const WaitCtx& w, unsigned code, unsigned site,
                                            unsigned detail) {
    *w.abort_sm = 1;
    if (w.status != nullptr && atomicCAS(w.status, 0u, code) == 0u) {
        w.status[1] = blockIdx.x;
        w.status[2] = site;
        w.status[3] = detail;
        __threadfence_system();
    }
}

// A kernel that meets an index from device memory pointing outside its buffers skips the access and
// leaves this record (first one wins) for the host: {DK_DEV_BAD_INDEX, block, site, detail}.
static __device__ __noinline__ void record_bad_index(unsigned* status, unsigned site, unsigned detail) {
    if (status != nullptr && atomicCAS(status, 0u, static_cast<unsigned>(DK_DEV_BAD_INDEX)) == 0u) {
        status[1] = blockIdx.x;
        status[2] = site;
        status[3] = detail;
        __threadfence_system();
    }
}

// Bounded wait on an mbarrier phase. Returns false when the limit ran out or another role of
// this CTA already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& w,
                                          unsigned site, unsigned detail = 0) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    unsigned spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0xff) == 0) {
            if (*w.abort_sm) return false;
            if (globaltimer_ns() - t0 > DK_WAIT_LIMIT_NS) {
                record_timeout(w, DK_DEV_TIMEOUT, site, detail);
                return false;
            }
        }
    }
    return true;
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load into this CTA only: coordinates are {x = innermost element index, y = row}.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar,
                                            int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
// The same load issued by either CTA of a cta_group::2 pair: the data lands in the issuing CTA's
// shared memory, the byte count completes on `cluster_bar`, an mbarrier that may live in the
// OTHER CTA of the pair (address from mapa). No multicast: one CTA receives the tile.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m,
                                                 uint32_t cluster_bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(cluster_bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar,
                                            int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(m)),
                 "r"(src), "r"(x), "r"(y)
                 : "memory");
}
// Contiguous bulk copy shared -> global (16-byte aligned, size a multiple of 16), same bulk-group
// completion mechanism as the tensor store.
__device__ __forceinline__ void bulk_store_1d(void* dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM
template <int CTAS>
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    if constexpr (CTAS == 1)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         dst_smem),
                     "r"(ncols)
                     : "memory");
    else
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         dst_smem),
                     "r"(ncols)
                     : "memory");
}
template <int CTAS>
__device__ __forceinline__ void tmem_relinquish() {
    if constexpr (CTAS == 1)
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    else
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CTAS>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    if constexpr (CTAS == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr),
                     "r"(ncols)
                     : "memory");
    else
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr),
                     "r"(ncols)
                     : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes with
// the 128-byte swizzle (what a TMA load with CU_TENSOR_MAP_SWIZZLE_128B and a 128-byte inner box
// produces). Groups of 8 rows are 1024 bytes apart (stride byte offset); the leading byte offset
// is not used by swizzled K-major layouts and is set to 1. Bits: [0,14) address>>4,
// [16,30) LBO>>4, [32,46) SBO>>4, [46,48) version = 1, [61,64) layout = 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// Instruction descriptor, dense, fp32 accumulate, A and B K-major.
// fmt: kind::f16 -> 0 = f16, 1 = bf16; kind::f8f6f4 -> 0 = e4m3, 1 = e5m2.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t fmt_a, uint32_t fmt_b, uint32_t m,
                                                  uint32_t n) {
    return (1u << 4) | (fmt_a << 7) | (fmt_b << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T, issued by ONE thread.
template <int CTAS>
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
    if constexpr (CTAS == 1)
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
            "}\n" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
            "}\n" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
}
template <int CTAS>
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
    if constexpr (CTAS == 1)
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
            "}\n" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
            "}\n" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
}
// ---- block-scaled MMA (kind::mxf8f6f4.block_scale): D (+)= (A * 2^(sfa-127)) * (B * 2^(sfb-127))^T
// with one e8m0 scale byte per row and per 32 elements of K, read from tensor memory.
//
// Scale bytes reach tensor memory as 512-byte "atoms" covering 128 rows x 128 elements of K: byte
// r0*16 + r1*4 + k is the scale of row r0 + 32*r1 for the 32-element group k. One
// tcgen05.cp.32x128b.warpx4 moves an atom from shared memory into four consecutive 32-bit columns
// (lane r0 of every lane quarter, column r1, byte k); the MMA picks byte k with the scale ids of
// its instruction descriptor.
//
// Shared-memory descriptor of one atom: 32 rows of 16 bytes, no swizzle, K-major; 8-row core
// matrices 128 bytes apart (stride byte offset), a single 16-byte column (leading offset unused).
__device__ __forceinline__ uint64_t umma_desc_sf_atom(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
    d |= static_cast<uint64_t>(128 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    return d;  // layout type 0: no swizzle
}
template <int CTAS>
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
    if constexpr (CTAS == 1)
        asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
    else
        asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// Instruction descriptor of the block-scaled kind: e4m3 x e4m3 (formats 0), both K-major, fp32
// accumulate implied; N>>3 at bit 17, scale format e8m0 at bit 23, M>>4 at bit 24, the byte of the
// scale columns to use at bits 4 (B) and 29 (A).
__host__ __device__ constexpr uint32_t umma_idesc_mx(uint32_t m, uint32_t n, uint32_t sf_id) {
    return (sf_id << 4) | ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24) | (sf_id << 29);
}
template <int CTAS>
__device__ __forceinline__ void umma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    if constexpr (CTAS == 1)
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
            "}\n" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
            : "memory");
    else
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
            "}\n" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
            : "memory");
}
// Contiguous bulk copy global -> this CTA's shared memory (16-byte aligned, size a multiple of 16),
// byte count completing on an mbarrier.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// Make the mbarrier track completion of all tcgen05 operations this thread issued so far.
// Implies tcgen05.fence::before_thread_sync.
template <int CTAS>
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    if constexpr (CTAS == 1)
        asm volatile(
            "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
            : "memory");
    else
        asm volatile(
            "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
            : "memory");
}
// Pair form: one commit whose arrive is delivered to the barrier at this offset in every CTA of
// cta_mask (both CTAs of the pair). This is the tensor pipe's completion signal, not a load.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
        " [%0], %1;" ::"r"(bar),
        "h"(cta_mask)
        : "memory");
}

// TMEM -> registers: this thread's lane (row), 32 consecutive fp32 columns starting at taddr.
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32"
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15,"
        " %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31},"
        " [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// The same wait, naming the registers a tcgen05.ld is filling as in/out operands: their uses can
// then not be scheduled ahead of the wait (the load writes them asynchronously).
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]),
                   "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]),
                   "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]),
                   "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
                   "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]),
                   "+r"(r[31])
                 :
                 : "memory");
}

// ---------------------------------------------------------------- cluster helpers
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta));
    return r;
}
__device__ __forceinline__ void cluster_arrive() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- misc
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Signals between GPUs: 4-byte counters in peer-visible memory, written with release and read
// with acquire at system scope. Counters only grow (epoch numbering), so nothing is reset.
__device__ __forceinline__ void signal_add_release_sys(unsigned* p, unsigned v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void signal_store_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void signal_store_relaxed_sys(unsigned* p, unsigned v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned signal_load_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// NVLink multicast (NVLS). `mc` is an address inside a mapping of a multicast object: the switch
// performs the access on the same offset of every bound GPU's memory.
// Sum over all GPUs of 8 bf16 values, accumulated in fp32 inside the switch, returned as bf16.
__device__ __forceinline__ uint4 multimem_ld_reduce_add_bf16x8(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
}
// Store 16 bytes to the same offset of every GPU's memory.
__device__ __forceinline__ void multimem_st_bf16x8(void* mc, const uint4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x),
                 "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// Bounded wait until *p >= target (wrap-safe). Returns false on timeout.
__device__ __forceinline__ bool signal_wait_ge(const unsigned* p, unsigned target,
                                               const WaitCtx& w, unsigned site,
                                               unsigned detail = 0) {
    if (static_cast<int>(signal_load_acquire_sys(p) - target) >= 0) return true;
    const uint64_t t0 = globaltimer_ns();
    unsigned spins = 0;
    while (static_cast<int>(signal_load_acquire_sys(p) - target) < 0) {
        if ((++spins & 0x3f) == 0) {
            if (*w.abort_sm) return false;
            // An error record the host has not read yet means an earlier wait already ran out
            // (here or in an earlier launch): the job is broken, so do not wait the limit again.
            if ((spins & 0x3fff) == 0 && w.status != nullptr &&
                *reinterpret_cast<volatile unsigned*>(w.status) != 0u) {
                *w.abort_sm = 1;
                return false;
            }
            if (globaltimer_ns() - t0 > w.peer_limit_ns) {
                record_timeout(w, DK_DEV_PEER_TIMEOUT, site, detail);
                return false;
            }
        }
    }
    return true;
}

}  // namespace dk
