// bf16 GEMM for sm_100a, with an optional fused reduce-scatter epilogue over peer memory.
//
//   C[M,N] = A[M,K] * Bt[N,K]^T      bf16 in, fp32 accumulate in TMEM, bf16 out (RNE)
//
// Stands in for micro_tk / kittens_store / dispatch_micro of the reference
// (distributed-kernels/bf16_gemm/kernel.cpp:89-245, :24-70, :247-251). The reference kernel is a
// producer/consumer MFMA kernel with a 128x256x64 CTA tile whose epilogue stores each element
// through iris.store to its own rank. This kernel keeps the contract (same operand layouts, same
// CTA tile footprint) and nothing of the mechanism:
//
//   warp 0      TMA producer: cp.async.bulk.tensor loads of A (128x64) and Bt tiles, 128-byte swizzle,
//               into a shared-memory ring, completion on mbarriers
//   warp 1      MMA issuer: one thread issues tcgen05.mma (kind::f16, K = 16 per instruction) reading
//               the ring through shared-memory descriptors, accumulating into one of two
//               256-column TMEM buffers; tcgen05.commit frees ring stages and publishes finished
//               accumulators
//   warps 2-5   epilogue: tcgen05.ld (lane quarter = warp % 4), fp32 -> bf16, then either 16-byte
//               global stores or swizzled shared-memory staging + TMA bulk stores
//
// Two instantiations. PAIR = 2 (default where M and the rows per rank are multiples of 256): a
// cluster of two CTAs computes a 256x256 tile with tcgen05.mma.cta_group::2 issued by the leader;
// each CTA stages its 128 rows of A and half of the Bt tile (32 KiB stages, six deep), and both
// CTAs' loads complete on the leader's mbarrier. PAIR = 1: one CTA per 128x256 tile, 48 KiB stages,
// four deep.
//
// Persistent: one CTA per SM walks a static tile list in a grouped raster (2048 rows per group) so
// that concurrently running CTAs share A and Bt tiles in L2.
//
// Reduce-scatter mode (world > 1): A and Bt hold this rank's K-shard. Each finished 128x256 tile
// of the partial product is written, as bf16, into slot [rank] of the staging area of the rank
// that OWNS those rows (peer memory, over NVLink) as sixteen contiguous 4 KiB bulk copies (the
// staging area is tile-major, so a peer write never has to be scattered over rows), followed by
// a release store of the call number into that tile's flag [rank] at the owner. Tiles are visited
// with the owners rotating fastest (rank+1, rank+2, ..., this rank), see tile_coords: every link is
// busy all the time and the partials of a tile arrive at its owner at about the same time.
//   warps 6-11  reducers: the tiles of this rank's own rows are dealt, a quarter tile at a time and in
//               the order in which they are computed, over the reducer warps of the whole grid; for
//               each the warps wait (bounded) for the `world` flags, sum the `world` bf16 partials in
//               fp32 in rank order and write bf16, while the MMA warps are working on later tiles.
//
// All-gather mode (column-parallel GEMM, the projection BEFORE the row-parallel one): the rows of A
// are sharded over the ranks (A_r [M/P, K]), every rank needs all of them against its own columns of
// the weight. The six warps that have nothing to do in a plain GEMM push this rank's shard into the
// peers' staging copies of A, two rows at a time with 16-byte peer stores, and count each piece into a
// per-(source, 128-row tile) counter at the destination with a release add. The TMA producer starts
// with the tiles of its own rows (read from the caller's A), then walks the other shards in the
// order rank+1, rank+2, ...; before the first load of a tile whose rows come from a peer it waits
// (bounded) for that tile's counter and crosses to the async proxy with a fence. No remote tile is
// ever read over NVLink by TMA: every CTA loads from this GPU's own memory.
#include "dk_heap.h"
#include "dk_host.h"
#include "dk_ptx.cuh"

#include <algorithm>
#include <cstdlib>

namespace dk {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr int EPI_BUF_BYTES = 32 * 128;  // 32 rows x 64 bf16 per epilogue warp
constexpr int EPI_BYTES = 4 * 2 * EPI_BUF_BYTES;
constexpr int CTRL_BYTES = 256;
// PAIR = 1: one CTA per 128x256 tile. PAIR = 2: a cluster of two CTAs per 256x256 tile
// (tcgen05.mma.cta_group::2): each CTA holds its 128 rows of A and HALF of the Bt tile, so a stage
// is 32 KiB instead of 48 and the ring is six stages deep instead of four.
template <int PAIR>
struct Cfg {
    static constexpr int B_ROWS = BN / PAIR;
    static constexpr int B_BYTES = B_ROWS * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = PAIR == 2 ? 6 : 4;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + EPI_BYTES + CTRL_BYTES;
};
constexpr int GEMM_THREADS = 384;  // TMA, MMA, 4 epilogue warps, 6 reducer warps
constexpr int RED_THREADS = 192;
constexpr int GROUP_M = 16;
constexpr int TMEM_COLS = 512;

struct GemmMaps {
    CUtensorMap a;
    CUtensorMap a_stage;  // all-gather mode: this rank's staging copy of the whole A [M, K]
    CUtensorMap b;
    CUtensorMap out[DK_MAX_RANKS];  // destination seen as [rows_per_rank, N], box 64 x 32
};

struct GemmArgs {
    int M, N, K;
    int tiles_m, tiles_n, num_kb;
    int world, rank;
    int rows_per_rank;  // rows of the output owned by one rank (M when world == 1)
    int tiles_per_owner;  // reduce-scatter: row-tiles (of 128 * PAIR rows) per owner; 0 = one rank
    int m_tile_rot;       // all-gather mode: first row-tile visited
    int group_m;          // row-tiles per raster group (reduce-scatter: per owner)
    int epi_mode;       // 0 direct stores, 1 TMA stores
    int phases;         // bit 0: GEMM tiles, bit 1: reduce this rank's rows
    __nv_bfloat16* dst[DK_MAX_RANKS];  // per owner: where this rank's partial (or C) goes
    unsigned* flag_dst[DK_MAX_RANKS];  // per owner: flags [tiles_per_shard][world] at the owner
    unsigned epoch;
    const __nv_bfloat16* red_src;  // local staging [world][rows_per_rank][N]
    __nv_bfloat16* red_out;        // [rows_per_rank][N]
    const unsigned* red_flags;     // local flags [tiles_per_shard][world]
    unsigned* status;
    unsigned long long peer_wait_ns;
    long long* dbg;  // [gridDim.x][DBG_SLOTS] stall counters, or null
    // all-gather mode (ag_world > 1); `a` then holds this rank's shard only
    int ag_world, ag_rank;
    int ag_shard_rows;                   // M / ag_world
    int ag_push;                         // this launch pushes the shard to the peers
    const uint4* ag_src;                 // this rank's shard [shard_rows, K]
    uint4* ag_dst[DK_MAX_RANKS];         // staging copy of A at rank d (current parity), [M, K]
    unsigned* ag_cnt_dst[DK_MAX_RANKS];  // counters [ag_world][tiles per shard] at rank d
    const unsigned* ag_cnt;              // the local ones
    unsigned ag_target;                  // value a counter has reached when its tile is complete
};

// Rows per pushed piece. Small pieces matter twice: every pusher warp of the grid gets work (a warp
// keeps 4 KB in flight, so the aggregate rate needs all of them to fill NVLink), and because the
// pieces are dealt in the order nearest consumer first, the shard the next rank needs first arrives
// first at full bandwidth instead of all shards arriving together at the end.
constexpr int AG_ROWS = 2;
constexpr int AG_PIECES = BM / AG_ROWS;      // pieces per 128-row tile

enum : unsigned {
    SITE_EMPTY = 1,
    SITE_FULL = 2,
    SITE_TMEM_EMPTY = 3,
    SITE_TMEM_FULL = 4,
    SITE_EPI_DONE = 5,
    SITE_RS_FLAG = 6,
    SITE_AG_TILE = 7
};

// t -> (m, n) in units of the launch's tiles (tiles_m counts tiles of 128 * PAIR rows).
// One rank: grouped raster, group_m row-tiles x all column tiles, rows fastest.
// Reduce-scatter (tiles_per_owner > 0): inside a group, owners rotate fastest: the tiles with the
// same position (row-tile inside the owner's rows, column tile) are computed for owner rank+1,
// rank+2, ..., and last for this rank itself, before the position advances. All ranks walk the
// positions in the same order, so the `world` partials of an output tile are produced at about the
// same time everywhere: each tile can be reduced right after it was computed, while its staged
// partials are still in L2, and the reduction work is spread over the whole kernel instead of
// piling up behind a last phase of own tiles. group_m * world row-tiles are live at a time.
__device__ __forceinline__ void tile_coords(int t, const GemmArgs& g, int& m, int& n) {
    const int group_m = g.group_m;
    if (g.tiles_per_owner > 0) {
        const int per_group = group_m * g.world * g.tiles_n;
        const int grp = t / per_group;
        const int first = grp * group_m;
        const int gsz = min(g.tiles_per_owner - first, group_m);
        const int r = t - grp * per_group;
        const int span = gsz * g.world;
        n = r / span;
        const int w = r - n * span;
        const int m_in = w / g.world;
        int owner = g.rank + 1 + (w - m_in * g.world);
        if (owner >= g.world) owner -= g.world;
        m = owner * g.tiles_per_owner + first + m_in;
        return;
    }
    const int per_group = group_m * g.tiles_n;
    const int grp = t / per_group;
    const int first_m = grp * group_m;
    const int gsz = min(g.tiles_m - first_m, group_m);
    const int r = t - grp * per_group;
    m = first_m + r % gsz;
    n = r / gsz;
    // all-gather mode starts with the rows that are already here
    m += g.m_tile_rot;
    if (m >= g.tiles_m) m -= g.tiles_m;
}

// Epilogue warps call this once the bulk stores of a tile have completed (each warp's issuing lane
// has waited on its own store groups): meet on the CTA's mbarrier (release/acquire at CTA scope),
// then one thread release-stores the call number into the tile's flag at the owner at system
// scope; by cumulativity that release covers the completed stores of all four warps.
// Returns false if the bounded wait gave up.
__device__ __forceinline__ bool epi_signal(const GemmArgs& g, const WaitCtx& wc, uint32_t bar_epi,
                                           uint32_t epi_ph, int ew, int lane, int owner,
                                           int tile_in_shard) {
    if (lane == 0) mbar_arrive(bar_epi);
    if (ew != 0) return true;
    bool landed = true;
    if (lane == 0) {
        landed = mbar_wait(bar_epi, epi_ph, wc, SITE_EPI_DONE, tile_in_shard);
        if (landed)
            signal_store_release_sys(
                g.flag_dst[owner] + static_cast<size_t>(tile_in_shard) * g.world + g.rank, g.epoch);
    }
    return __all_sync(0xffffffffu, landed);
}

// Sum `world` staged partial tiles into bf16 rows of the output. A staged tile is the 64 KiB image
// the epilogue wrote: block (q, c) of 4 KiB holds rows q*32.. x columns c*64.. as 32 rows of 128
// bytes whose 16-byte chunks are XOR-swizzled by (row & 7). UNR vectors per thread in flight per slot.
template <int UNR, int W>
__device__ __forceinline__ void reduce_tile(const __nv_bfloat16* __restrict__ src,
                                            __nv_bfloat16* __restrict__ dst, int N, int world, int rt,
                                            int tm, int n, int rtile, size_t slot_elems, int vec_lo,
                                            int vec_hi) {
    const uint4* tsrc = reinterpret_cast<const uint4*>(src + static_cast<size_t>(rtile) * (BM * BN));
    __nv_bfloat16* tdst = dst + static_cast<size_t>(tm) * BM * N + n * BN;
    const size_t slot_vecs = slot_elems / 8;
#pragma unroll 1
    for (int base = vec_lo + rt; base < vec_hi; base += RED_THREADS * UNR) {
        uint4 v[UNR][W];
        int off[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int vi = base + u * RED_THREADS;
            const int blk = vi >> 8;             // 256 vectors per 4 KiB block
            const int row_in = (vi >> 3) & 31;
            const int j = (vi & 7) ^ (row_in & 7);
            const int row = (blk >> 2) * 32 + row_in;
            const int col = (blk & 3) * 64 + j * 8;
            off[u] = (vi < vec_hi && n * BN + col + 8 <= N) ? row * N + col : -1;
#pragma unroll
            for (int s = 0; s < W; ++s)
                if (s < world && off[u] >= 0)
                    // L2 read: the partials were written by peers while this kernel ran
                    v[u][s] = __ldcg(tsrc + s * slot_vecs + vi);
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            if (off[u] < 0) continue;
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
            for (int s = 0; s < W; ++s) {
                if (s < world) {
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u][s]);
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
            *reinterpret_cast<uint4*>(tdst + off[u]) = o;
        }
    }
}

// W = upper bound of g.world this instantiation serves (2, 4 or 8); it only sizes the reducers'
// register arrays.
template <int W, int PAIR>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ GemmMaps maps, const GemmArgs g) {
    constexpr int STAGES = Cfg<PAIR>::STAGES;
    constexpr int STAGE_BYTES = Cfg<PAIR>::STAGE_BYTES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
    // position inside the pair and the pair's place in the grid
    const int crank = PAIR == 2 ? static_cast<int>(cluster_ctarank()) : 0;
    const int unit = blockIdx.x / PAIR;     // which tile walker this CTA belongs to
    const int nunits = gridDim.x / PAIR;

    const uint32_t ring = smem_base;
    const uint32_t epi = smem_base + STAGES * STAGE_BYTES;
    uint8_t* ctrl = smem + STAGES * STAGE_BYTES + EPI_BYTES;
    const uint32_t ctrl_u = epi + EPI_BYTES;
    // control block: 8-byte mbarriers, then the TMEM base address and the abort flag
    const uint32_t bar_full = ctrl_u;                 // STAGES: operands landed (a pair: both CTAs', on the leader)
    const uint32_t bar_empty = ctrl_u + 8 * STAGES;   // STAGES: the MMAs are done with the stage
    const uint32_t bar_tfull = ctrl_u + 24 * STAGES;        // 2
    const uint32_t bar_tempty = ctrl_u + 24 * STAGES + 16;  // 2
    const uint32_t bar_epi = ctrl_u + 24 * STAGES + 32;     // 1
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(ctrl + 24 * STAGES + 40);
    volatile int* abort_sm = reinterpret_cast<volatile int*>(ctrl + 24 * STAGES + 48);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const WaitCtx wc{g.status, abort_sm, g.peer_wait_ns};
    const int num_tiles = g.tiles_m * g.tiles_n;
    const bool do_gemm = (g.phases & 1) != 0;
    const long long dbg_t0 = clock64();

    if (threadIdx.x == 0) {
        *abort_sm = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_tfull + 8 * a, 1);
            mbar_init(bar_tempty + 8 * a, 128 * PAIR);  // the leader hears both CTAs' epilogues
        }
        mbar_init(bar_epi, 4);
        fence_mbar_init();
        tma_prefetch_desc(&maps.a);
        tma_prefetch_desc(&maps.b);
    }
    if (warp == 1 && do_gemm) {
        tmem_alloc<PAIR>(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
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
    const uint32_t tmem_base = do_gemm ? *tmem_slot : 0u;

    if (do_gemm) {
        if (warp == 0) {
            // ------------------------------------------------ TMA producer
            if (lane == 0) {
                int s = 0;
                uint32_t ph = 0;
                bool ok = true;
                long long dbg_prod = 0;
                for (int t = unit; t < num_tiles && ok; t += nunits) {
                    int m, n;
                    tile_coords(t, g, m, n);
                    m = m * PAIR + crank;  // this CTA's 128-row tile
                    const CUtensorMap* amap = &maps.a;
                    int arow = m * BM;
                    if (g.ag_world > 1) {
                        const int src = arow / g.ag_shard_rows;
                        if (src == g.ag_rank) {
                            arow -= src * g.ag_shard_rows;  // own rows: straight from the caller's shard
                        } else {
                            // rows of a peer: wait until all pieces of this 128-row tile have landed
                            // in the local staging copy, then make them visible to the TMA unit
                            amap = &maps.a_stage;
                            const int tile_in_shard = (arow - src * g.ag_shard_rows) / BM;
                            if (!signal_wait_ge(g.ag_cnt + src * (g.ag_shard_rows / BM) + tile_in_shard, g.ag_target,
                                                wc, SITE_AG_TILE, static_cast<unsigned>(m))) {
                                ok = false;
                                break;
                            }
                            asm volatile("fence.proxy.async;" ::: "memory");
                        }
                    }
                    for (int kb = 0; kb < g.num_kb; ++kb) {
                        const long long c0 = clock64();
                        if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, wc, SITE_EMPTY, t)) {
                            ok = false;
                            break;
                        }
                        dbg_prod += clock64() - c0;
                        const uint32_t full = bar_full + 8 * s;
                        const uint32_t sa = ring + s * STAGE_BYTES;
                        if (PAIR == 2) {
                            // both CTAs' loads complete on the LEADER's barrier, which expects the
                            // bytes of both; the follower's bytes may land before the leader has
                            // announced them (the phase cannot end before the leader's arrive)
                            const uint32_t lead_full = mapa_shared(full, 0);
                            if (crank == 0) mbar_expect_tx(full, 2 * STAGE_BYTES);
                            tma_load_2d_pair(sa, amap, lead_full, kb * BK, arow);
                            // a pair splits the 256 rows of the Bt tile between its two CTAs
                            tma_load_2d_pair(sa + A_BYTES, &maps.b, lead_full, kb * BK,
                                             n * BN + crank * Cfg<PAIR>::B_ROWS);
                        } else {
                            mbar_expect_tx(full, STAGE_BYTES);
                            tma_load_2d(sa, amap, full, kb * BK, arow);
                            tma_load_2d(sa + A_BYTES, &maps.b, full, kb * BK, n * BN);
                        }
                        if (++s == STAGES) {
                            s = 0;
                            ph ^= 1;
                        }
                    }
                }
                // plain launches have no reducers: their slot carries the producer's wait for free stages
                if (g.dbg != nullptr && g.world == 1) g.dbg[blockIdx.x * DBG_SLOTS + DBG_RED_WORK] = dbg_prod;
            }
        } else if (warp == 1) {
            // ------------------------------------------------ MMA issuer
            // the follower of a pair issues no MMAs: its operands complete on the leader's barrier
            if (lane == 0 && crank == 0) {
                constexpr uint32_t idesc = umma_idesc(1, 1, BM * PAIR, BN);
                int s = 0;
                uint32_t ph = 0;
                int acc = 0;
                uint32_t acc_ph = 0;
                bool ok = true;
                long long dbg_mma_tmem = 0, dbg_mma_full = 0;
                for (int t = unit; t < num_tiles && ok; t += nunits) {
                    long long c0 = clock64();
                    if (!mbar_wait(bar_tempty + 8 * acc, acc_ph ^ 1, wc, SITE_TMEM_EMPTY, t)) break;
                    dbg_mma_tmem += clock64() - c0;
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + acc * BN;
                    for (int kb = 0; kb < g.num_kb; ++kb) {
                        c0 = clock64();
                        if (!mbar_wait(bar_full + 8 * s, ph, wc, SITE_FULL, t)) {
                            ok = false;
                            break;
                        }
                        dbg_mma_full += clock64() - c0;
                        tc_fence_after();
                        const uint32_t sa = ring + s * STAGE_BYTES;
                        const uint64_t da = umma_desc_sw128(sa);
                        const uint64_t db = umma_desc_sw128(sa + A_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            // +32 bytes along K inside the 128-byte swizzle row = +2 in the
                            // descriptor's 16-byte address units
                            umma_f16<PAIR>(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                        }
                        // the stage is free in BOTH CTAs once these MMAs have read it
                        if (PAIR == 2) umma_commit_pair(bar_empty + 8 * s, 3);
                        else umma_commit<1>(bar_empty + 8 * s);
                        if (++s == STAGES) {
                            s = 0;
                            ph ^= 1;
                        }
                    }
                    if (!ok) break;
                    if (PAIR == 2) umma_commit_pair(bar_tfull + 8 * acc, 3);
                    else umma_commit<1>(bar_tfull + 8 * acc);
                    acc ^= 1;
                    if (acc == 0) acc_ph ^= 1;
                }
                if (g.dbg != nullptr) {
                    g.dbg[blockIdx.x * DBG_SLOTS + DBG_MMA_WAIT_TMEM] = dbg_mma_tmem;
                    g.dbg[blockIdx.x * DBG_SLOTS + DBG_MMA_WAIT_FULL] = dbg_mma_full;
                }
            }
        } else if (warp < 6) {
            // ------------------------------------------------ epilogue (warps 2..5)
            const int q = warp & 3;  // TMEM lane quarter this warp may read
            const int ew = warp - 2;
            const uint32_t my_epi = epi + ew * 2 * EPI_BUF_BYTES;
            int acc = 0;
            uint32_t acc_ph = 0;
            uint32_t epi_ph = 0;
            long long dbg_acc = 0, dbg_smem = 0, dbg_landed = 0, dbg_signal = 0, dbg_drain = 0;
            for (int t = unit; t < num_tiles; t += nunits) {
                int m, n;
                tile_coords(t, g, m, n);
                m = m * PAIR + crank;  // this CTA's 128-row tile
                const int owner = (m * BM) / g.rows_per_rank;
                const int row0 = m * BM - owner * g.rows_per_rank + q * 32;  // row inside dst
                // the whole warp takes the same branch: tcgen05.ld below is warp-collective
                long long c0 = clock64();
                if (!__all_sync(0xffffffffu,
                                mbar_wait(bar_tfull + 8 * acc, acc_ph, wc, SITE_TMEM_FULL, t)))
                    break;
                dbg_acc += clock64() - c0;
                const long long c_drain = clock64();
                tc_fence_after();
                const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
#pragma unroll 1
                for (int c = 0; c < BN / 64; ++c) {
                    uint32_t r0[32], r1[32];
                    tmem_ld_32x32b_x32(t_acc + c * 64, r0);
                    tmem_ld_32x32b_x32(t_acc + c * 64 + 32, r1);
                    tmem_ld_wait(r0);
                    tmem_ld_wait(r1);
                    uint32_t p[32];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        p[i] = pack_bf16x2(__uint_as_float(r0[2 * i]), __uint_as_float(r0[2 * i + 1]));
                        p[16 + i] =
                            pack_bf16x2(__uint_as_float(r1[2 * i]), __uint_as_float(r1[2 * i + 1]));
                    }
                    const int col0 = n * BN + c * 64;
                    if (g.epi_mode == 1) {
                        const uint32_t buf = my_epi + (c & 1) * EPI_BUF_BYTES;
                        // the store issued two chunks ago has finished reading this buffer
                        c0 = clock64();
                        if (lane == 0) tma_store_wait_read<1>();
                        __syncwarp();
                        dbg_smem += clock64() - c0;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const uint32_t addr = buf + lane * 128 + ((j ^ (lane & 7)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                                         "r"(p[4 * j]), "r"(p[4 * j + 1]), "r"(p[4 * j + 2]),
                                         "r"(p[4 * j + 3])
                                         : "memory");
                        }
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            if (g.world > 1) {
                                // staging is tile-major: the tile's 64 KiB image is 16 blocks of
                                // 4 KiB (lane quarter q, column chunk c), each an exact copy of
                                // this swizzled buffer, so the peer sees one contiguous 4 KiB write
                                const int tis = ((m * BM - owner * g.rows_per_rank) / BM) * g.tiles_n + n;
                                bulk_store_1d(g.dst[owner] + static_cast<size_t>(tis) * (BM * BN) +
                                                  (q * (BN / 64) + c) * (EPI_BUF_BYTES / 2),
                                              buf, EPI_BUF_BYTES);
                            } else {
                                tma_store_2d(&maps.out[owner], buf, col0, row0);
                            }
                            tma_store_commit();
                        }
                    } else {
                        const int row = row0 + lane;
                        const bool row_ok = (m * BM + q * 32 + lane) < g.M;
                        __nv_bfloat16* dst = g.dst[owner] + static_cast<size_t>(row) * g.N + col0;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            if (row_ok && col0 + 8 * j + 8 <= g.N) {
                                *reinterpret_cast<uint4*>(dst + 8 * j) =
                                    make_uint4(p[4 * j], p[4 * j + 1], p[4 * j + 2], p[4 * j + 3]);
                            }
                        }
                    }
                }
                // accumulator drained: hand the TMEM buffer back to the (leader's) MMA warp
                tc_fence_before();
                if (PAIR == 2 && crank != 0) mbar_arrive_cluster(mapa_shared(bar_tempty + 8 * acc, 0));
                else mbar_arrive(bar_tempty + 8 * acc);
                acc ^= 1;
                if (acc == 0) acc_ph ^= 1;

                if (g.world > 1) {
                    // Tell the owner once all four warps' stores of this tile have landed. The
                    // bulk stores complete through wait_group, the warps meet on an mbarrier, and
                    // ONE system-scope release store publishes the flag: no other fence is issued
                    // (system-scope fences next to NVLink traffic cost tens of microseconds each).
                    dbg_drain += clock64() - c_drain;
                    c0 = clock64();
                    if (lane == 0) tma_store_wait_all<0>();
                    __syncwarp();
                    dbg_landed += clock64() - c0;
                    c0 = clock64();
                    const int tis = ((m * BM - owner * g.rows_per_rank) / BM) * g.tiles_n + n;
                    if (!epi_signal(g, wc, bar_epi, epi_ph, ew, lane, owner, tis)) break;
                    dbg_signal += clock64() - c0;
                    epi_ph ^= 1;
                }
            }
            if (g.epi_mode == 1 && lane == 0) tma_store_wait_all<0>();
            if (g.dbg != nullptr && ew == 0 && lane == 0) {
                g.dbg[blockIdx.x * DBG_SLOTS + DBG_EPI_WAIT_ACC] = dbg_acc;
                g.dbg[blockIdx.x * DBG_SLOTS + DBG_EPI_WAIT_SMEM] = dbg_smem;
                g.dbg[blockIdx.x * DBG_SLOTS + DBG_EPI_WAIT_LANDED] = dbg_landed;
                if ((g.phases & 2) == 0 && g.world > 1) {
                    // produce-only launches have no reducers: their two slots carry the time spent
                    // draining accumulators and the time spent in fences + flag stores instead
                    g.dbg[blockIdx.x * DBG_SLOTS + DBG_RED_WAIT_FLAG] = dbg_drain;
                    g.dbg[blockIdx.x * DBG_SLOTS + DBG_RED_WORK] = dbg_signal;
                }
            }
        }
    }

    // -------------------------------------------------------- all-gather pushers (warps 6..11)
    // Every piece is AG_ROWS rows of this rank's shard = AG_ROWS * K contiguous bf16 at the source and
    // at the destination. Pieces are dealt round-robin to the pusher warps of the whole grid, nearest
    // consumer first: rank d works through the shards d, d+1, ..., so the shard of rank s is needed
    // first by s-1, then s-2, ...
    if (warp >= 6 && g.ag_world > 1 && g.ag_push) {
        const int tiles_shard = g.ag_shard_rows / BM;
        const int per_peer = tiles_shard * AG_PIECES;
        const int total = (g.ag_world - 1) * per_peer;
        const int nvec = AG_ROWS * (g.K / 8);
        const int nwarps = gridDim.x * 6;
        for (int u = blockIdx.x * 6 + (warp - 6); u < total; u += nwarps) {
            const int pi = u / per_peer;
            int d = g.ag_rank - 1 - pi;
            if (d < 0) d += g.ag_world;
            const int rem = u - pi * per_peer;
            const int rt = rem / AG_PIECES;
            const size_t row0 = static_cast<size_t>(rt) * BM + (rem - rt * AG_PIECES) * AG_ROWS;
            const uint4* src = g.ag_src + row0 * (g.K / 8);
            uint4* dst = g.ag_dst[d] + (static_cast<size_t>(g.ag_rank) * g.ag_shard_rows + row0) * (g.K / 8);
            int i = lane;
            for (; i + 224 < nvec; i += 256) {  // eight 16-byte loads per lane in flight
                uint4 v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = src[i + 32 * j];
#pragma unroll
                for (int j = 0; j < 8; ++j) dst[i + 32 * j] = v[j];
            }
            for (; i < nvec; i += 32) dst[i] = src[i];
            // the lanes' stores are ordered before lane 0's release by the warp barrier; the release
            // add is cumulative over them at system scope
            __syncwarp();
            if (lane == 0) signal_add_release_sys(g.ag_cnt_dst[d] + g.ag_rank * tiles_shard + rt, 1u);
        }
    }

    // -------------------------------------------------------- reducers (warps 6..11, world > 1)
    // The tiles whose rows this rank owns are summed by the reducer warps of the WHOLE grid, a
    // quarter of a 128-row tile (32 rows = four 4 KiB blocks of the staged image) per work item, items
    // dealt round-robin over the CTAs in the order in which the tiles are computed. A tile is summed
    // as soon as its `world` partials are there, by four CTAs at once, while the MMA warps are on later
    // tiles; after the last wave every CTA has at most one quarter tile left instead of a few CTAs
    // having a whole one.
    if (warp >= 6 && (g.phases & 2) != 0 && g.world > 1) {
        const int rt = threadIdx.x - (GEMM_THREADS - RED_THREADS);
        const size_t slot_elems = static_cast<size_t>(g.rows_per_rank) * g.tiles_n * BN;
        constexpr int QUARTER_VECS = 32 * (BN / 8);
        const int own_tiles = num_tiles / g.world;  // tile units (pairs) whose rows this rank owns
        const int items = own_tiles * PAIR * 4;
        long long dbg_flag = 0, dbg_work = 0;
        bool ok = true;
        // one work item: quarter `quarter` of the 128-row tile m (a row-tile index of the whole output)
        auto reduce_item = [&](int m, int n, int quarter) {
            long long c0 = clock64();
            const int tm = (m * BM - g.rank * g.rows_per_rank) / BM;
            const int rtile = tm * g.tiles_n + n;
            if (rt < g.world)
                signal_wait_ge(g.red_flags + static_cast<size_t>(rtile) * g.world + rt, g.epoch, wc,
                               SITE_RS_FLAG, rtile);
            named_bar_sync(2, RED_THREADS);
            if (*abort_sm) {
                ok = false;
                return;
            }
            dbg_flag += clock64() - c0;
            c0 = clock64();
            // world * UNR = 16 vectors per thread in flight
            reduce_tile<16 / W, W>(g.red_src, g.red_out, g.N, g.world, rt, tm, n, rtile, slot_elems,
                                   quarter * QUARTER_VECS, (quarter + 1) * QUARTER_VECS);
            dbg_work += clock64() - c0;
        };
        // the owners take turns in the visiting order, this rank last of each round, so the i-th own
        // tile is tile i * world + world - 1
        for (int j = blockIdx.x; j < items && ok; j += gridDim.x) {
            const int i = j / (4 * PAIR);
            int m, n;
            tile_coords(i * g.world + g.world - 1, g, m, n);
            m = m * PAIR + (j >> 2) % PAIR;
            if ((m * BM) / g.rows_per_rank != g.rank) continue;  // cannot happen in this order
            reduce_item(m, n, j & 3);
        }
        if (g.dbg != nullptr && rt == 0) {
            g.dbg[blockIdx.x * DBG_SLOTS + DBG_RED_WAIT_FLAG] = dbg_flag;
            g.dbg[blockIdx.x * DBG_SLOTS + DBG_RED_WORK] = dbg_work;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (PAIR == 2) {
        // neither CTA leaves (or frees the pair's TMEM) while the other may still signal it
        cluster_arrive();
        cluster_wait();
    }
    if (g.dbg != nullptr && threadIdx.x == 0) g.dbg[blockIdx.x * DBG_SLOTS + DBG_TOTAL] = clock64() - dbg_t0;
    if (warp == 1 && do_gemm) {
        __syncwarp();
        tc_fence_after();
        if (*abort_sm) {
            // give copies still in flight time to land before the shared memory goes away
            const uint64_t t0 = globaltimer_ns();
            while (globaltimer_ns() - t0 < 200000ull) {
            }
        }
        tmem_dealloc<PAIR>(tmem_base, TMEM_COLS);
    }
}

// --------------------------------------------------------------------------------------------
// host side

// Stall-counter buffer handed to every GEMM launch (null = off); see dk_gemm_debug_counters.
static long long* g_gemm_dbg = nullptr;

static int check_gemm_args(const void* A, const void* Bt, void* C, int M, int N, int K) {
    DK_REQUIRE(A != nullptr && Bt != nullptr && C != nullptr, "null operand");
    DK_REQUIRE(M > 0 && N > 0 && K > 0, "M, N, K must be positive");
    DK_REQUIRE(K % 8 == 0, "K must be a multiple of 8 (16-byte rows for TMA)");
    DK_REQUIRE(N % 8 == 0, "N must be a multiple of 8 (16-byte output vectors)");
    return DK_OK;
}

template <int W, int PAIR>
static int launch_gemm_w(const GemmMaps& maps, const GemmArgs& args, int grid, cudaStream_t stream) {
    static bool attr_set[64] = {false};
    int dev = 0;
    DK_CUDA_OK(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        DK_CUDA_OK(cudaFuncSetAttribute(gemm_bf16_kernel<W, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        Cfg<PAIR>::SMEM_BYTES));
        attr_set[dev & 63] = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = Cfg<PAIR>::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = PAIR;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    DK_CUDA_OK(cudaLaunchKernelEx(&cfg, gemm_bf16_kernel<W, PAIR>, maps, args));
    return DK_OK;
}

// pair != 0 selects the two-CTA kernel; `grid` counts CTAs and is then even.
static int launch_gemm(const GemmMaps& maps, const GemmArgs& args, int grid, int pair, cudaStream_t stream) {
    if (pair) {
        if (args.world <= 2) return launch_gemm_w<2, 2>(maps, args, grid, stream);
        if (args.world <= 4) return launch_gemm_w<4, 2>(maps, args, grid, stream);
        return launch_gemm_w<8, 2>(maps, args, grid, stream);
    }
    if (args.world <= 2) return launch_gemm_w<2, 1>(maps, args, grid, stream);
    if (args.world <= 4) return launch_gemm_w<4, 1>(maps, args, grid, stream);
    return launch_gemm_w<8, 1>(maps, args, grid, stream);
}

// Two-CTA tiles need whole 256-row tiles (per owner in reduce-scatter mode). Where the shape allows
// it the pair kernel is the default (it needs two thirds of the one-CTA kernel's shared-memory fill
// bandwidth per flop and has a deeper ring); dk_gemm_pair_mode(0) or DK_GEMM_PAIR=0 selects the
// one-CTA kernel.
static int group_m_setting() {
    static int v = -1;
    if (v < 0) {
        const char* e = std::getenv("DK_GEMM_GROUP_M");
        v = (e && *e) ? std::atoi(e) : GROUP_M;
        if (v < 2) v = 2;
    }
    return v;
}

static int g_pair_mode = -2;  // -2: read DK_GEMM_PAIR on first use; 0 off; 1 on (default)
static bool use_pair(int M, int rows_per_rank) {
    if (g_pair_mode == -2) {
        const char* e = std::getenv("DK_GEMM_PAIR");
        g_pair_mode = (e && *e && std::atoi(e) == 0) ? 0 : 1;
    }
    const bool possible = (M % (2 * BM) == 0) && (rows_per_rank % (2 * BM) == 0);
    return g_pair_mode == 1 && possible;
}

int gemm_bf16_impl(const void* A, const void* Bt, void* C, int M, int N, int K, int epilogue,
                   cudaStream_t stream) {
    int rc = check_gemm_args(A, Bt, C, M, N, K);
    if (rc != DK_OK) return rc;
    GemmMaps maps;
    GemmArgs g{};
    rc = make_tmap_2d(&maps.a, A, 2, K, M, static_cast<uint64_t>(K) * 2, BK, BM);
    if (rc != DK_OK) return rc;
    const int pair = use_pair(M, ((M + BM - 1) / BM) * BM) ? 2 : 1;
    rc = make_tmap_2d(&maps.b, Bt, 2, K, N, static_cast<uint64_t>(K) * 2, BK, BN / pair);
    if (rc != DK_OK) return rc;
    rc = make_tmap_2d(&maps.out[0], C, 2, N, M, static_cast<uint64_t>(N) * 2, 64, 32);
    if (rc != DK_OK) return rc;
    for (int r = 1; r < DK_MAX_RANKS; ++r) maps.out[r] = maps.out[0];
    maps.a_stage = maps.a;
    g.M = M;
    g.N = N;
    g.K = K;
    g.tiles_m = (M + BM - 1) / BM / pair;   // tiles of 128 * pair rows
    g.group_m = group_m_setting() / pair;
    g.tiles_n = (N + BN - 1) / BN;
    g.num_kb = (K + BK - 1) / BK;
    g.world = 1;
    g.rank = 0;
    g.rows_per_rank = g.tiles_m * pair * BM;  // one owner
    g.tiles_per_owner = 0;
    g.m_tile_rot = 0;
    g.epi_mode = epilogue < 0 ? 1 : epilogue;
    g.phases = 1;
    g.dst[0] = static_cast<__nv_bfloat16*>(C);
    g.epoch = 0;
    rc = device_status_ptr(&g.status);
    if (rc != DK_OK) return rc;
    g.peer_wait_ns = peer_wait_ns();
    g.dbg = g_gemm_dbg;
    int sms = 0;
    rc = sm_count(&sms);
    if (rc != DK_OK) return rc;
    const int tiles = g.tiles_m * g.tiles_n;
    const int units = sms / pair;   // tile walkers: CTAs, or pairs of CTAs
    return launch_gemm(maps, g, (tiles < units ? tiles : units) * pair, pair == 2, stream);
}

// ---- reduce-scatter ---------------------------------------------------------------------------
// Workspace layout (identical offset on every rank, inside the symmetric heap):
//   stage [2 parities][world slots][tiles of the shard][64 KiB tile image] bf16, then
//   flags [2 parities][tiles per shard][world] u32 (offset rounded up to 256 bytes)
static size_t rs_stage_bytes(int M, int N, int world) {
    const size_t n_padded = static_cast<size_t>((N + BN - 1) / BN) * BN;  // whole 128 x 256 tiles
    return static_cast<size_t>(2) * world * (M / world) * n_padded * 2;
}
static size_t rs_flag_words(int M, int N, int world) {
    const int shard_tiles = ((M / world) / BM) * ((N + BN - 1) / BN);
    return static_cast<size_t>(shard_tiles) * world;
}
static size_t rs_flags_offset(int M, int N, int world) {
    return (rs_stage_bytes(M, N, world) + 255) / 256 * 256;
}
size_t gemm_rs_workspace_bytes(int M, int N, int world) {
    if (world <= 1) return 0;
    return rs_flags_offset(M, N, world) + 2 * rs_flag_words(M, N, world) * 4;
}

int gemm_rs_impl(const void* A, const void* Bt, void* out, int M, int N, int Kloc, void* workspace,
                 const dk_view* view, unsigned seq, int phases, int epilogue, cudaStream_t stream) {
    const int world = view ? view->world : 1;
    if (world <= 1) {
        if ((phases & 1) == 0) return DK_OK;
        return gemm_bf16_impl(A, Bt, out, M, N, Kloc, epilogue, stream);
    }
    int rc = check_gemm_args(A, Bt, out, M, N, Kloc);
    if (rc != DK_OK) return rc;
    DK_REQUIRE(world <= DK_MAX_RANKS, "world must be <= 8");
    DK_REQUIRE(view->rank >= 0 && view->rank < world, "rank out of range");
    DK_REQUIRE(M % (world * BM) == 0, "M must be a multiple of world * 128");
    DK_REQUIRE(workspace != nullptr, "gemm_rs needs a workspace inside the symmetric heap");
    DK_REQUIRE(seq != 0, "sequence numbers start at 1");
    if (const int pending = device_status_pending()) return pending;
    const int rank = view->rank;
    const int mloc = M / world;
    const size_t slot_elems = static_cast<size_t>(mloc) * ((N + BN - 1) / BN) * BN;
    const unsigned parity = seq & 1u;

    GemmMaps maps;
    GemmArgs g{};
    rc = make_tmap_2d(&maps.a, A, 2, Kloc, M, static_cast<uint64_t>(Kloc) * 2, BK, BM);
    if (rc != DK_OK) return rc;
    const int pair = use_pair(M, mloc) ? 2 : 1;
    rc = make_tmap_2d(&maps.b, Bt, 2, Kloc, N, static_cast<uint64_t>(Kloc) * 2, BK, BN / pair);
    if (rc != DK_OK) return rc;
    g.M = M;
    g.N = N;
    g.K = Kloc;
    g.tiles_m = M / BM / pair;   // tiles of 128 * pair rows
    // world * group_m row-tiles are live at a time; keep that near the one-rank group
    g.group_m = group_m_setting() / pair / world;
    if (g.group_m < 1) g.group_m = 1;
    g.tiles_n = (N + BN - 1) / BN;
    g.num_kb = (Kloc + BK - 1) / BK;
    g.world = world;
    g.rank = rank;
    g.rows_per_rank = mloc;
    g.tiles_per_owner = mloc / BM / pair;
    g.m_tile_rot = 0;
    // Pushes to peers always use TMA bulk stores: with direct 16-byte stores to peer memory an
    // 8-GPU run stalled until its peer waits ran out, so that variant is not offered across GPUs.
    (void)epilogue;
    g.epi_mode = 1;
    g.phases = phases;
    g.epoch = seq;
    char* ws_local = static_cast<char*>(workspace);
    const size_t stage_par = static_cast<size_t>(parity) * world * slot_elems * 2;
    const size_t flags_off = rs_flags_offset(M, N, world) + static_cast<size_t>(parity) * rs_flag_words(M, N, world) * 4;
    for (int o = 0; o < world; ++o) {
        char* ws_o = static_cast<char*>(peer_ptr(view, ws_local, o));
        g.dst[o] = reinterpret_cast<__nv_bfloat16*>(ws_o + stage_par) + static_cast<size_t>(rank) * slot_elems;
        g.flag_dst[o] = reinterpret_cast<unsigned*>(ws_o + flags_off);
    }
    // the output maps are used by the plain GEMM only; fill them with a valid descriptor
    for (int o = 0; o < DK_MAX_RANKS; ++o) maps.out[o] = maps.a;
    maps.a_stage = maps.a;
    g.red_src = reinterpret_cast<const __nv_bfloat16*>(ws_local + stage_par);
    g.red_out = static_cast<__nv_bfloat16*>(out);
    g.red_flags = reinterpret_cast<const unsigned*>(ws_local + flags_off);
    rc = device_status_ptr(&g.status);
    if (rc != DK_OK) return rc;
    g.peer_wait_ns = peer_wait_ns();
    g.dbg = g_gemm_dbg;
    int sms = 0;
    rc = sm_count(&sms);
    if (rc != DK_OK) return rc;
    const int tiles = g.tiles_m * g.tiles_n;
    const int units = sms / pair;
    return launch_gemm(maps, g, (tiles < units ? tiles : units) * pair, pair == 2, stream);
}

// ---- all-gather + GEMM -------------------------------------------------------------------------
// Workspace layout (identical offset on every rank, inside the symmetric heap):
//   stage [2 parities][M, K] bf16: this rank's copy of the whole A (its own rows are never written:
//         they are read from the caller's shard), then
//   counters [world][tiles per shard] u32 (offset rounded up to 256 bytes): pieces received so far
//         of every 128-row tile; they only grow (AG_PIECES per call), nothing is reset.
static size_t ag_stage_bytes(int M, int K) { return static_cast<size_t>(M) * K * 2; }
static size_t ag_cnt_offset(int M, int K) { return (2 * ag_stage_bytes(M, K) + 255) / 256 * 256; }
size_t ag_gemm_workspace_bytes(int M, int K, int world) {
    if (world <= 1) return 0;
    return ag_cnt_offset(M, K) + static_cast<size_t>(M / BM) * 4;
}

// phases: bit 0 = push this rank's shard to the peers, bit 1 = the GEMM (which waits for the peers'
// pieces). seq = 1-based call number on this workspace.
int ag_gemm_impl(const void* A, const void* Bt, void* C, int M, int N, int K, void* workspace, const dk_view* view,
                 unsigned seq, int phases, cudaStream_t stream) {
    const int world = view ? view->world : 1;
    if (world <= 1) {
        if ((phases & 2) == 0) return DK_OK;
        return gemm_bf16_impl(A, Bt, C, M, N, K, -1, stream);
    }
    int rc = check_gemm_args(A, Bt, C, M, N, K);
    if (rc != DK_OK) return rc;
    DK_REQUIRE(world <= DK_MAX_RANKS, "world must be <= 8");
    DK_REQUIRE(view->rank >= 0 && view->rank < world, "rank out of range");
    DK_REQUIRE(M % (world * BM) == 0, "M must be a multiple of world * 128");
    DK_REQUIRE(workspace != nullptr, "ag_gemm needs a workspace inside the symmetric heap");
    DK_REQUIRE(seq != 0, "sequence numbers start at 1");
    if (const int pending = device_status_pending()) return pending;
    const int rank = view->rank;
    const int shard = M / world;
    GemmMaps maps;
    GemmArgs g{};
    const int pair = use_pair(M, shard) ? 2 : 1;
    char* ws_local = static_cast<char*>(workspace);
    const size_t par_off = static_cast<size_t>(seq & 1u) * ag_stage_bytes(M, K);
    rc = make_tmap_2d(&maps.a, A, 2, K, shard, static_cast<uint64_t>(K) * 2, BK, BM);
    if (rc != DK_OK) return rc;
    rc = make_tmap_2d(&maps.a_stage, ws_local + par_off, 2, K, M, static_cast<uint64_t>(K) * 2, BK, BM);
    if (rc != DK_OK) return rc;
    rc = make_tmap_2d(&maps.b, Bt, 2, K, N, static_cast<uint64_t>(K) * 2, BK, BN / pair);
    if (rc != DK_OK) return rc;
    rc = make_tmap_2d(&maps.out[0], C, 2, N, M, static_cast<uint64_t>(N) * 2, 64, 32);
    if (rc != DK_OK) return rc;
    for (int r = 1; r < DK_MAX_RANKS; ++r) maps.out[r] = maps.out[0];
    g.M = M;
    g.N = N;
    g.K = K;
    g.tiles_m = M / BM / pair;
    // raster groups never span two shards: all tiles of the rows already here come before the first
    // tile that has to wait for a peer
    g.group_m = std::min(group_m_setting() / pair, shard / BM / pair);
    if (g.group_m < 1) g.group_m = 1;
    g.tiles_n = (N + BN - 1) / BN;
    g.num_kb = (K + BK - 1) / BK;
    g.world = 1;                       // the output is local: plain epilogue, no reducers
    g.rank = 0;
    g.rows_per_rank = g.tiles_m * pair * BM;
    g.tiles_per_owner = 0;
    g.m_tile_rot = rank * (shard / BM / pair);   // own rows first, then the shards of rank+1, rank+2, ...
    g.epi_mode = 1;
    g.phases = (phases & 2) ? 1 : 0;
    g.dst[0] = static_cast<__nv_bfloat16*>(C);
    g.epoch = 0;
    g.ag_world = world;
    g.ag_rank = rank;
    g.ag_shard_rows = shard;
    g.ag_push = (phases & 1) ? 1 : 0;
    g.ag_src = static_cast<const uint4*>(A);
    for (int d = 0; d < world; ++d) {
        char* ws_d = static_cast<char*>(peer_ptr(view, ws_local, d));
        g.ag_dst[d] = reinterpret_cast<uint4*>(ws_d + par_off);
        g.ag_cnt_dst[d] = reinterpret_cast<unsigned*>(ws_d + ag_cnt_offset(M, K));
    }
    g.ag_cnt = reinterpret_cast<const unsigned*>(ws_local + ag_cnt_offset(M, K));
    g.ag_target = seq * static_cast<unsigned>(AG_PIECES);
    rc = device_status_ptr(&g.status);
    if (rc != DK_OK) return rc;
    g.peer_wait_ns = peer_wait_ns();
    g.dbg = g_gemm_dbg;
    int sms = 0;
    rc = sm_count(&sms);
    if (rc != DK_OK) return rc;
    const int tiles = g.tiles_m * g.tiles_n;
    const int units = sms / pair;
    // a launch that pushes uses the whole machine's pusher warps even when there are few tiles
    const int ctas = (phases & 1) ? units : (tiles < units ? tiles : units);
    return launch_gemm(maps, g, ctas * pair, pair == 2, stream);
}

}  // namespace dk

extern "C" size_t dk_ag_gemm_workspace_bytes(int M, int K, int world) {
    if (M <= 0 || K <= 0 || world < 1 || world > DK_MAX_RANKS || M % (world * dk::BM) != 0) return 0;
    return dk::ag_gemm_workspace_bytes(M, K, world);
}

extern "C" int dk_ag_gemm_workspace_init(void* workspace, size_t bytes, const dk_view* view, void* stream) {
    if (view == nullptr || view->world <= 1) return DK_OK;
    DK_REQUIRE(workspace != nullptr && bytes > 0, "null workspace");
    DK_REQUIRE(dk::in_heap(view, workspace, bytes), "workspace must lie inside the symmetric heap");
    DK_CUDA_OK(cudaMemsetAsync(workspace, 0, bytes, static_cast<cudaStream_t>(stream)));
    DK_CUDA_OK(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    dk_heap* h = static_cast<dk_heap*>(view->heap);
    if (h != nullptr) {
        {
            std::lock_guard<std::mutex> lk(h->mu);
            h->rs_seq[workspace] = 0;
        }
        return dk_heap_barrier(h);
    }
    return DK_OK;
}

extern "C" int dk_ag_gemm_phase(const void* A, const void* Bt, void* C, int M, int N, int K, void* workspace,
                                const dk_view* view, unsigned seq, int phases, void* stream) {
    DK_REQUIRE(phases >= 1 && phases <= 3, "phases must be 1 (push), 2 (GEMM) or 3 (both)");
    return dk::ag_gemm_impl(A, Bt, C, M, N, K, workspace, view, seq, phases, static_cast<cudaStream_t>(stream));
}

extern "C" int dk_ag_gemm(const void* A, const void* Bt, void* C, int M, int N, int K, void* workspace,
                          const dk_view* view, void* stream) {
    unsigned seq = 1;
    if (view != nullptr && view->world > 1) {
        dk_heap* h = static_cast<dk_heap*>(view->heap);
        DK_REQUIRE(h != nullptr, "view has no heap handle; use dk_ag_gemm_phase with explicit sequence numbers");
        DK_REQUIRE(workspace != nullptr && dk::in_heap(view, workspace, dk::ag_gemm_workspace_bytes(M, K, view->world)),
                   "workspace must lie inside the symmetric heap");
        if (const int pending = dk::device_status_pending()) return pending;
        std::lock_guard<std::mutex> lk(h->mu);
        auto it = h->rs_seq.find(workspace);
        DK_REQUIRE(it != h->rs_seq.end(), "workspace was not initialised with dk_ag_gemm_workspace_init");
        seq = ++it->second;
    }
    return dk::ag_gemm_impl(A, Bt, C, M, N, K, workspace, view, seq, 3, static_cast<cudaStream_t>(stream));
}

extern "C" int dk_ag_gemm_workspace_get(const dk_view* view, int M, int K, void* stream, void** out) {
    DK_REQUIRE(out != nullptr, "null result pointer");
    *out = nullptr;
    if (view == nullptr || view->world <= 1) return DK_OK;
    dk_heap* h = static_cast<dk_heap*>(view->heap);
    DK_REQUIRE(h != nullptr, "view has no heap handle");
    DK_REQUIRE(M > 0 && K > 0 && M % (view->world * dk::BM) == 0, "M must be a positive multiple of world * 128");
    {
        std::lock_guard<std::mutex> lk(h->mu);
        auto it = h->ag_ws.find({M, K});
        if (it != h->ag_ws.end()) {
            *out = it->second;
            return DK_OK;
        }
    }
    const size_t bytes = dk::ag_gemm_workspace_bytes(M, K, view->world);
    void* ws = dk_heap_alloc(h, bytes, 1024);
    if (ws == nullptr) {
        dk::set_last_error("symmetric heap exhausted: an all-gather workspace of " + std::to_string(bytes) +
                           " bytes does not fit");
        return DK_ERR_NOMEM;
    }
    const int rc = dk_ag_gemm_workspace_init(ws, bytes, view, stream);
    if (rc != DK_OK) return rc;
    std::lock_guard<std::mutex> lk(h->mu);
    h->ag_ws[{M, K}] = ws;
    dk::log_msg(1, "rank " + std::to_string(view->rank) + ": all-gather workspace for M=" + std::to_string(M) +
                       " K=" + std::to_string(K) + ", " + std::to_string(bytes >> 20) + " MiB of the heap");
    *out = ws;
    return DK_OK;
}

extern "C" int dk_gemm_pair_mode(int mode) {
    if (mode != 0 && mode != 1) {
        dk::set_last_error("argument error: mode must be 0 or 1");
        return DK_ERR_ARG;
    }
    dk::g_pair_mode = mode;
    return DK_OK;
}

extern "C" int dk_gemm_debug_counters(long long* device_buffer) {
    dk::g_gemm_dbg = device_buffer;
    return DK_OK;
}

extern "C" size_t dk_gemm_rs_workspace_bytes(int M, int N, int world) {
    if (M <= 0 || N <= 0 || world < 1 || world > DK_MAX_RANKS || M % world != 0) return 0;
    return dk::gemm_rs_workspace_bytes(M, N, world);
}

extern "C" int dk_gemm_rs_workspace_init(void* workspace, size_t bytes, const dk_view* view,
                                         void* stream) {
    if (view == nullptr || view->world <= 1) return DK_OK;
    DK_REQUIRE(workspace != nullptr && bytes > 0, "null workspace");
    DK_REQUIRE(dk::in_heap(view, workspace, bytes), "workspace must lie inside the symmetric heap");
    DK_CUDA_OK(cudaMemsetAsync(workspace, 0, bytes, static_cast<cudaStream_t>(stream)));
    DK_CUDA_OK(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    dk_heap* h = static_cast<dk_heap*>(view->heap);
    if (h != nullptr) {
        {
            std::lock_guard<std::mutex> lk(h->mu);
            h->rs_seq[workspace] = 0;
        }
        return dk_heap_barrier(h);
    }
    return DK_OK;
}

extern "C" int dk_gemm_rs_workspace_get(const dk_view* view, int M, int N, void* stream, void** out) {
    DK_REQUIRE(out != nullptr, "null result pointer");
    *out = nullptr;
    if (view == nullptr || view->world <= 1) return DK_OK;
    dk_heap* h = static_cast<dk_heap*>(view->heap);
    DK_REQUIRE(h != nullptr, "view has no heap handle");
    DK_REQUIRE(M > 0 && N > 0 && M % (view->world * dk::BM) == 0, "M must be a positive multiple of world * 128");
    {
        std::lock_guard<std::mutex> lk(h->mu);
        auto it = h->rs_ws.find({M, N});
        if (it != h->rs_ws.end()) {
            *out = it->second;
            return DK_OK;
        }
    }
    const size_t bytes = dk::gemm_rs_workspace_bytes(M, N, view->world);
    void* ws = dk_heap_alloc(h, bytes, 1024);
    if (ws == nullptr) {
        dk::set_last_error("symmetric heap exhausted: a reduce-scatter workspace of " + std::to_string(bytes) +
                           " bytes does not fit");
        return DK_ERR_NOMEM;
    }
    const int rc = dk_gemm_rs_workspace_init(ws, bytes, view, stream);
    if (rc != DK_OK) return rc;
    std::lock_guard<std::mutex> lk(h->mu);
    h->rs_ws[{M, N}] = ws;
    dk::log_msg(1, "rank " + std::to_string(view->rank) + ": reduce-scatter workspace for M=" + std::to_string(M) +
                       " N=" + std::to_string(N) + ", " + std::to_string(bytes >> 20) + " MiB of the heap");
    *out = ws;
    return DK_OK;
}

extern "C" int dk_gemm_rs_phase(const void* A, const void* Bt, void* out, int M, int N, int Kloc,
                                void* workspace, const dk_view* view, unsigned seq, int phases,
                                int epilogue, void* stream) {
    DK_REQUIRE(phases >= 1 && phases <= 3, "phases must be 1 (produce), 2 (reduce) or 3 (both)");
    DK_REQUIRE(epilogue <= 1, "epilogue must be -1, 0 or 1");
    return dk::gemm_rs_impl(A, Bt, out, M, N, Kloc, workspace, view, seq, phases, epilogue,
                            static_cast<cudaStream_t>(stream));
}

extern "C" int dk_gemm_rs(const void* A, const void* Bt, void* out, int M, int N, int Kloc,
                          void* workspace, const dk_view* view, void* stream) {
    unsigned seq = 1;
    if (view != nullptr && view->world > 1) {
        dk_heap* h = static_cast<dk_heap*>(view->heap);
        DK_REQUIRE(h != nullptr, "view has no heap handle; use dk_gemm_rs_phase with explicit sequence numbers");
        DK_REQUIRE(workspace != nullptr && dk::in_heap(view, workspace, dk::gemm_rs_workspace_bytes(M, N, view->world)),
                   "workspace must lie inside the symmetric heap");
        // before the call number advances: a refused call must not leave this rank one call ahead
        if (const int pending = dk::device_status_pending()) return pending;
        std::lock_guard<std::mutex> lk(h->mu);
        auto it = h->rs_seq.find(workspace);
        DK_REQUIRE(it != h->rs_seq.end(), "workspace was not initialised with dk_gemm_rs_workspace_init");
        seq = ++it->second;
    }
    return dk::gemm_rs_impl(A, Bt, out, M, N, Kloc, workspace, view, seq, 3, -1,
                            static_cast<cudaStream_t>(stream));
}

extern "C" int dk_gemm_bf16(const void* A, const void* Bt, void* C, int M, int N, int K,
                            const dk_view* view, int epilogue, void* stream) {
    (void)view;  // a plain GEMM writes to local memory only; the view is accepted for symmetry
    if (epilogue > 1) {
        dk::set_last_error("argument error: epilogue must be -1, 0 or 1");
        return DK_ERR_ARG;
    }
    return dk::gemm_bf16_impl(A, Bt, C, M, N, K, epilogue, static_cast<cudaStream_t>(stream));
}
