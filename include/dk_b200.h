/*
 * dk_b200 -- C ABI of the B200 (sm_100a) multi-GPU hot path.
 *
 * One shared library, libdk_b200.so. Plain pointers and sizes only; no C++ or torch types cross
 * this line. Every function returns 0 (DK_OK) on success or a DK_ERR_* code; dk_strerror() names
 * it. Buffers are borrowed: the caller keeps them alive until the stream has run the work.
 * Launches are asynchronous on the given stream (NULL = the legacy default stream, which is what
 * the reference launches on, distributed-kernels/bf16_gemm/kernel.cpp:82,249-250).
 *
 * Reference interfaces these entry points stand in for are cited at each declaration, by path
 * inside the reference project.
 */
#ifndef DK_B200_H
#define DK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DK_MAX_RANKS 8

enum {
    DK_OK = 0,
    DK_ERR_ARG = 1,        /* bad shape, alignment, null pointer, unsupported size */
    DK_ERR_CUDA = 2,       /* a CUDA runtime/driver call failed; see dk_last_error_string() */
    DK_ERR_DEVICE = 3,     /* the device holds an unread error record (a bounded wait gave up, or a kernel
                              skipped a bad index); see dk_last_device_status() */
    DK_ERR_BOOTSTRAP = 4,  /* rendezvous between ranks failed (socket, timeout, peer gone) */
    DK_ERR_NOMEM = 5,      /* symmetric heap exhausted */
    DK_ERR_UNSUPPORTED = 6 /* feature not available on this device/driver */
};

/*
 * Device view of the symmetric heap: what a kernel needs to address a peer.
 * Stands in for iris::iris_device_view (external to the reference tree; used at
 * distributed-kernels/bf16_gemm/kernel.cpp:25,39,58-59,75 and bound at
 * distributed-kernels/iris_py.cpp:113-115). base[r] is THIS process's mapping of rank r's heap;
 * the peer address of a local heap pointer p is base[r] + (p - base[rank]).
 */
typedef struct dk_view {
    int rank;
    int world;
    void* base[DK_MAX_RANKS];
    uint64_t heap_bytes;
    void* mc_base;   /* NVLS multicast mapping of the heap, NULL when not available */
    void* heap;      /* host handle (dk_heap*) that owns the collective epoch; NULL if world==1 */
} dk_view;

const char* dk_strerror(int code);
/* Text of the last CUDA/bootstrap failure on the calling thread ("" if none). */
const char* dk_last_error_string(void);
/* Version of this ABI: major*1000 + minor. */
int dk_version(void);

/*
 * Record of the first device-side error on the current device since the last call:
 * out = {code, block, site, detail}; code 0 = none, 1 = a wait inside a CTA gave up, 2 = a wait on
 * another rank's signal gave up, 3 = a kernel met an index from device memory (expert id, row,
 * offset) that points outside its buffers and skipped the access. Clears the record.
 *
 * Launches are asynchronous: DK_OK from an entry point means "launched", not "completed". While a
 * record is unread, every collective entry point (dk_allreduce, dk_gemm_rs, dk_gemm_rs_phase,
 * dk_peer_barrier*, dk_allgather, dk_moe_dispatch, dk_moe_combine_ep, dk_moe_ep_layer) returns
 * DK_ERR_DEVICE without launching and leaves the record in place: after a wait has run out the
 * ranks are out of step, and later waits on peers would give up at once and leave wrong results.
 * The reference has no counterpart (HIP errors are printed and dropped, include/pyutils/util.cuh:10-16).
 */
int dk_last_device_status(unsigned out[4]);
/*
 * Limit, in milliseconds, of device-side waits on another rank's signal (flags of the
 * reduce-scatter, all-reduce and peer barrier). Such a wait also covers the time by which a peer's
 * launch lags behind on the host, so the default is generous: 20 s, or DK_PEER_WAIT_MS from the
 * environment. When it runs out the kernel records {code 2, block, site, detail}, stops waiting and
 * returns; the context stays usable. Applies to launches made after the call.
 */
int dk_set_peer_wait_ms(int ms);
/*
 * Host-side log to stderr: 0 = silent (default), 1 = life cycle (heap created / destroyed, multicast
 * mapping, workspaces taken from the heap, collectives refused because of an unread device record),
 * 2 = also every peer mapping. DK_LOG in the environment sets the initial level. The reference has
 * only the `verbose` flag it hands to iris (distributed-kernels/iris_py.cpp:53,61).
 */
int dk_set_log_level(int level);
/*
 * Tuning knob of the grouped and block-scaled GEMMs' tile order. Inside a group (an expert) tiles run
 * band by band; a band is as many row tiles as hold `bytes` of the row operand, and inside a band row
 * tiles run fastest, then column tiles: the band's rows stay in L2 while all column tiles pass.
 * Default 32 MB (DK_WALK_BAND_MB in the environment). Results do not depend on it.
 */
int dk_set_walk_band_bytes(size_t bytes);

/* ------------------------------------------------------------------ symmetric heap */
/*
 * Stands in for iris::iris (host runtime; call sites distributed-kernels/iris_py.cpp:55-61,89,
 * 24,100,105) and iris::mpi::initialize/finalize (iris_py.cpp:55,149-154).
 *
 * dk_bootstrap_env: rank/world/local_rank from RANK/WORLD_SIZE/LOCAL_RANK, else
 * OMPI_COMM_WORLD_RANK/SIZE/LOCAL_RANK, else 0/1/0 (no MPI needed).
 */
int dk_bootstrap_env(int* rank, int* world, int* local_rank);

typedef struct dk_heap dk_heap;

/*
 * Create a heap of `bytes` per rank on the current CUDA device and map every peer's heap
 * (cuMemCreate + POSIX file-descriptor exchange over a Unix socket + cuMemMap). `rendezvous` names
 * the Unix socket (NULL: derived from MASTER_PORT / DK_JOB_ID). world == 1 needs no rendezvous.
 */
int dk_heap_create(size_t bytes, int rank, int world, const char* rendezvous, dk_heap** out);
int dk_heap_destroy(dk_heap* h);
/* Bump allocation with a free list; identical call sequences give identical offsets on every
 * rank. Returns NULL when exhausted. align must be a power of two (0 = 256). */
void* dk_heap_alloc(dk_heap* h, size_t bytes, size_t align);
int dk_heap_free(dk_heap* h, void* p);
/* Host barrier across ranks (after cudaDeviceSynchronize of the caller's choice). */
int dk_heap_barrier(dk_heap* h);
int dk_heap_view(dk_heap* h, dk_view* out);
/*
 * Collective over all ranks of the heap: create one NVLink multicast object (NVLS) over the ranks'
 * heaps and map it (cuMulticastCreate / AddDevice / BindMem + cuMemMap). Afterwards dk_view.mc_base
 * is non-null: a multimem store to mc_base + o lands at offset o of EVERY rank's heap and a
 * multimem.ld_reduce there returns the sum over ranks, both done by the NVSwitch. Every step is
 * agreed between the ranks: on DK_ERR_UNSUPPORTED (no multicast support, or a step failed on some
 * rank) no rank has the mapping and the heap works as before. DK_NVLS=1 in the environment makes
 * dk_heap_create do this by itself. Opt-in because a process that dies while its memory is bound
 * to a multicast object can disturb its peers' GPUs; dk_heap_destroy unbinds in order.
 * No reference counterpart (iris has no multicast path at its call sites).
 */
int dk_heap_enable_multicast(dk_heap* h);
/* Bytes still free (largest bump region), for tests. */
size_t dk_heap_bytes_free(dk_heap* h);

/* Host-only pieces of the bootstrap, callable without a GPU (used by the CPU tests):
 * rendezvous of `world` processes, exchange of one file descriptor each, barrier. */
typedef struct dk_comm dk_comm;
int dk_comm_create(int rank, int world, const char* rendezvous, int timeout_ms, dk_comm** out);
int dk_comm_destroy(dk_comm* c);
int dk_comm_barrier(dk_comm* c);
/* all-gather of one fd per rank: fds_out[world]; fds_out[rank] is a dup of my_fd. */
int dk_comm_allgather_fd(dk_comm* c, int my_fd, int* fds_out);
/* all-gather of a fixed-size blob per rank. */
int dk_comm_allgather(dk_comm* c, const void* mine, size_t bytes, void* all_out);

/* ------------------------------------------------------------------ GEMM */
/*
 * C[M,N] = A[M,K] * Bt[N,K]^T, bf16 in, fp32 accumulate (tcgen05/TMEM), bf16 out (round to
 * nearest even). Row-major, contiguous. K % 8 == 0 and N % 8 == 0.
 * Replaces dispatch_micro / micro_tk (distributed-kernels/bf16_gemm/kernel.cpp:89-251).
 * view may be NULL (single GPU). epilogue: 0 = direct vector stores, 1 = TMA bulk stores, -1 = default.
 */
int dk_gemm_bf16(const void* A, const void* Bt, void* C, int M, int N, int K,
                 const dk_view* view, int epilogue, void* stream);

/*
 * Row-parallel (K-sharded) GEMM fused with reduce-scatter, no NCCL:
 *   out[M/P, N] (this rank's rows) = sum over ranks r of A_r[M, K/P] * Bt_r[N, K/P]^T
 * Every rank calls it with its own K-shard. Partial tiles are pushed as bf16 into the owner's
 * staging slot over NVLink and summed there in fp32 in rank order. M % (world*128) == 0.
 * The reference has no reduce-scatter (its kernel stores to its own rank only,
 * distributed-kernels/bf16_gemm/kernel.cpp:39,58-59; `row_offset` is accepted and unused, :80);
 * this is the tensor-parallel down-projection (GEMM + reduce-scatter), behind the same calling convention.
 *
 * `workspace` is dk_gemm_rs_workspace_bytes(M, N, world) bytes allocated from the symmetric heap
 * at the same offset on every rank and initialised once, collectively, with
 * dk_gemm_rs_workspace_init (zeroes the flags, synchronises the stream, host barrier).
 * With world == 1 the call is a plain GEMM and workspace may be NULL.
 */
size_t dk_gemm_rs_workspace_bytes(int M, int N, int world);
int dk_gemm_rs_workspace_init(void* workspace, size_t bytes, const dk_view* view, void* stream);
/*
 * The heap's own workspace for an (M, N) reduce-scatter: allocated from the heap and initialised on
 * first use (a collective: every rank makes the same calls in the same order), then returned again
 * for the same (M, N). It belongs to the heap and goes away with it. *out is NULL for world == 1.
 */
int dk_gemm_rs_workspace_get(const dk_view* view, int M, int N, void* stream, void** out);
int dk_gemm_rs(const void* A, const void* Bt, void* out, int M, int N, int Kloc, void* workspace,
               const dk_view* view, void* stream);
/*
 * The same in explicit phases, for callers that schedule them separately and for running all
 * ranks of a job on one GPU: phases bit 0 = compute and push partial tiles, bit 1 = wait for the
 * peers' tiles and reduce this rank's rows. `seq` is the 1-based call number on this workspace
 * (identical on every rank); the view needs no heap handle here.
 */
int dk_gemm_rs_phase(const void* A, const void* Bt, void* out, int M, int N, int Kloc,
                     void* workspace, const dk_view* view, unsigned seq, int phases, int epilogue,
                     void* stream);
/* (`epilogue` is honoured for world == 1 only: pushes to peers always use TMA bulk stores.) */

/*
 * Column-parallel GEMM fused with the all-gather of its activations, no NCCL: the projection that
 * precedes the row-parallel one of dk_gemm_rs in a tensor-parallel MLP.
 *   C[M, N] (all rows, this rank's N columns) = concat over ranks r of A_r[M/P, K]  *  Bt[N, K]^T
 * Every rank calls it with its own row shard A_r and its own weight columns Bt. Inside ONE kernel,
 * the warps a plain GEMM leaves idle push the shard to every peer's staging copy of A (16-byte peer
 * stores, a per-tile counter at the destination), while the MMA warps start on the rank's own rows
 * and take the other shards in the order rank+1, rank+2, ... as their tiles complete; TMA only ever
 * loads from this GPU's own memory. M % (world*128) == 0. The reference has no counterpart (it has
 * no collective); calling convention and operand layouts are those of dispatch_micro.
 *
 * `workspace`: dk_ag_gemm_workspace_bytes(M, K, world) bytes from the symmetric heap at the same
 * offset on every rank, initialised once, collectively, with dk_ag_gemm_workspace_init (or taken
 * from the heap with dk_ag_gemm_workspace_get, which does both on first use and keeps it with the
 * heap). With world == 1 the call is a plain GEMM and workspace may be NULL. dk_ag_gemm_phase runs
 * the push (bit 0) and the GEMM (bit 1) as separate launches with an explicit 1-based call number,
 * for running all ranks of a job on one GPU.
 */
size_t dk_ag_gemm_workspace_bytes(int M, int K, int world);
int dk_ag_gemm_workspace_init(void* workspace, size_t bytes, const dk_view* view, void* stream);
int dk_ag_gemm_workspace_get(const dk_view* view, int M, int K, void* stream, void** out);
int dk_ag_gemm(const void* A_shard, const void* Bt, void* C, int M, int N, int K, void* workspace,
               const dk_view* view, void* stream);
int dk_ag_gemm_phase(const void* A_shard, const void* Bt, void* C, int M, int N, int K, void* workspace,
                     const dk_view* view, unsigned seq, int phases, void* stream);

/*
 * Mode 1 (the default; DK_GEMM_PAIR=0 in the environment selects 0) makes dk_gemm_bf16 / dk_gemm_rs
 * use clusters of two CTAs per 256x256 tile (tcgen05.mma.cta_group::2: each CTA stages its 128
 * rows of A and half of the Bt tile in a six-stage ring, both CTAs' TMA loads complete on the
 * leader's mbarrier) whenever M (and the rows per rank) are multiples of 256; other shapes, and
 * mode 0, use the one-CTA kernel (128x256 tiles, four stages). Results are identical. No reference
 * counterpart.
 */
int dk_gemm_pair_mode(int mode);
/*
 * Stall accounting for the GEMM kernels, for tuning. device_buffer holds 8 int64 per CTA (148 CTAs
 * at most): clock ticks the MMA warp waited for a free accumulator / for operands, the epilogue
 * waited for an accumulator / for its staging buffer / for its stores to land, the reducers waited
 * for flags / spent summing, and the CTA's total. NULL switches it off (the default).
 */
int dk_gemm_debug_counters(long long* device_buffer);
/* The same for the fp8 grouped GEMM (MMA waits, promotion waits, per-tile epilogue, total). */
int dk_moe_gemm_debug_counters(long long* device_buffer);

/* ------------------------------------------------------------------ all-reduce */
/*
 * out = sum over ranks of x, n bf16 elements (n % 8 == 0), fp32 accumulation in rank order, so
 * every rank ends with bit-identical results. x must lie inside the symmetric heap at the same
 * offset on every rank. algo: -1 auto by message size (DK_ALLREDUCE_ONESHOT_MAX_BYTES overrides
 * the crossover), 0 one-shot (every rank reads all inputs; out may be any local buffer, not x),
 * 1 two-shot (reduce a slice, push it to every rank; out must lie inside the heap, may alias x;
 * n % (8*world) == 0), 2 NVLS (rank r reduces slice r inside the NVSwitch with multimem.ld_reduce
 * and broadcasts it with multimem.st; same conditions as two-shot, plus the heap's multicast
 * mapping, see dk_heap_enable_multicast, else DK_ERR_UNSUPPORTED; the switch's summation order is
 * unspecified but every element is reduced once and broadcast, so ranks still agree bit for bit).
 * Auto picks NVLS when the mapping exists, the conditions hold and world >= 4, where it measured
 * fastest at every size (DK_ALLREDUCE_NVLS_AUTO=0 keeps auto to the first two). world == 1 copies x to out. The reference has no counterpart: it contains no collective.
 */
int dk_allreduce(const void* x, void* out, size_t n, int algo, const dk_view* view, void* stream);
/*
 * All ranks of a job inside ONE cooperative launch on one GPU (blockIdx.y = rank): views[q],
 * x[q], out[q] describe rank q, whose "heap" is a region of this GPU's memory. `epoch` is the
 * 1-based call number shared by all ranks. For single-GPU testing of the multi-rank protocol.
 */
int dk_allreduce_all_ranks(int world, const dk_view* views, const void* const* x, void* const* out,
                           size_t n, int algo, unsigned epoch, void* stream);

/* ------------------------------------------------------------------ MoE: routing, layout, fp8 */
/*
 * None of the MoE entry points has a counterpart in the reference (it contains no MoE code); the
 * fp8 pieces follow the pattern of its block-scaled fixtures
 * (tests/unit/cdna4/warp/register/tile/mma_scaled.cu:200-258) with 128x128 fp32 scale blocks.
 *
 * dk_moe_route: top-k of logits[T,E] (fp32, E <= 256, k <= 8) on the raw logits, ties to the lower
 * expert index, slots in descending logit order; topk_w = softmax over all experts, gathered and
 * renormalised to sum to one.
 */
int dk_moe_route(const float* logits, int T, int E, int k, int* topk_idx, float* topk_w, void* stream);
/*
 * dk_moe_permute: group the T*k (token, slot) pairs by expert, pairs of one expert in (token,
 * slot) order, every expert padded to a multiple of `pad` rows. Experts are cut into segments of
 * `experts_per_segment` (= E for one GPU; = E / world for expert parallelism, one segment per
 * destination rank) and row numbering restarts in every segment.
 *   row_of_pair [T*k]                      row of the pair inside its segment
 *   pair_of_row [E/seg][seg_row_capacity]  inverse map, -1 on padding rows
 *   offsets     [E/seg][seg+1]             first row of each expert inside its segment
 *   counts      [E]                        pairs per expert
 * scratch: dk_moe_permute_scratch_bytes(T, k, E) bytes of device memory.
 * dk_moe_rows_capacity(T, k, E, pad): rows that always suffice for one segment.
 */
size_t dk_moe_permute_scratch_bytes(int T, int k, int E);
size_t dk_moe_rows_capacity(int T, int k, int E, int pad);
int dk_moe_permute(const int* topk_idx, int T, int k, int E, int pad, int experts_per_segment,
                   int* row_of_pair, int* pair_of_row, int seg_row_capacity, int* offsets,
                   int* counts, void* scratch, size_t scratch_bytes, void* stream);
/*
 * dk_moe_permute_static: dk_moe_permute for callers that must not allocate and have no scratch
 * buffer of their own to hand in -- code running where device allocation is off limits (inside a
 * region that forbids cudaMalloc, or a host runtime that was given a fixed set of buffers and no
 * allocator). It has no counterpart in the reference. Same arguments and results as
 * dk_moe_permute minus the scratch pair: the scratch is a fixed array compiled into the library,
 * dk_moe_permute_static_max_bytes() = 256 KiB per GPU, held from library load to process exit.
 * Routings that need more (dk_moe_permute_scratch_bytes(T, k, E) above that, i.e. more than
 * 65536 / E chunks of 1024 pairs) are rejected with DK_ERR_ARG and a message naming both sizes.
 * The call makes no cudaMalloc/cudaFree and uses no allocating library routine; inputs and outputs
 * are the caller's. The first call on each device looks up the array's device address (that device
 * must be current); make that first call before any stream capture starts. All calls on one GPU
 * share the one array, which keeps the previous call's contents (harmless: every entry a call reads
 * is written by that call first); two calls whose kernels overlap on the GPU, e.g. on different
 * streams, race on it and must be serialised by the caller.
 */
size_t dk_moe_permute_static_max_bytes(void);
int dk_moe_permute_static(const int* topk_idx, int T, int k, int E, int pad, int experts_per_segment,
                          int* row_of_pair, int* pair_of_row, int seg_row_capacity, int* offsets,
                          int* counts, void* stream);
/*
 * dk_quant_block128: x[*,C] bf16 -> q[R,C] e4m3 bytes + s[R/128, C/128] fp32, per 128x128 block
 * s = amax/448 (1 if the block is all zero), q = round-to-nearest-even(clamp(x/s, +-448)).
 * map_mode 0: row r of x. 1: row row_map[r]/k of x (gather of tokens into permuted rows), zeros
 * where row_map[r] < 0. 2: row r of x where row_map[r] >= 0, zeros elsewhere.
 */
int dk_quant_block128(const void* x, int R, int C, const int* row_map, int map_mode, int k, void* q,
                      float* s, void* stream);
/* out[t,:] = sum_j topk_w[t,j] * y[row_of_pair[t,j], :] in fp32, bf16 out. H % 8 == 0. */
int dk_moe_combine(const void* y, const int* row_of_pair, const float* topk_w, int T, int k, int H,
                   void* out, void* stream);

/*
 * dk_moe_grouped_gemm_fp8: per expert e, rows [offsets[e], offsets[e+1]) of X (multiples of 128,
 * read on the device) times that expert's weight, e4m3 operands with 128x128 fp32 block scales
 * (xs [R/128, K/128]; ws [E, rows/128, K/128]), fp32 accumulation with per-128-K promotion.
 *   gated = 1: wq is [E, 2N, K] (N gate rows, then N up rows); out = e4m3 bytes [R, N] of
 *              silu(gate) * up, requantised per 128x128 block, out_scales [R/128, N/128]. N % 128 == 0.
 *   gated = 0: wq is [E, N, K]; out = bf16 [R, N]; out_scales unused. N % 256 == 0.
 * Rows at or beyond offsets[E] are not written.
 */
int dk_moe_grouped_gemm_fp8(const void* xq, const float* xs, const void* wq, const float* ws,
                            const int* offsets, int E, int R, int N, int K, int gated, void* out,
                            float* out_scales, void* stream);

/* ------------------------------------------------------------------ MXFP8 (1x32 e8m0 block scales) */
/*
 * The block-scaled fp8 format the reference ships: e4m3 elements with one e8m0 (power-of-two) scale
 * per 32 consecutive elements of K. Here the tensor core applies the scales itself
 * (tcgen05.mma.kind::mxf8f6f4.block_scale reads them from tensor memory).
 *
 * Scale "atoms": the layout the tensor core wants. For every 128 rows x 128 elements of K one
 * 512-byte atom, byte r0*16 + r1*4 + g = scale of row r0 + 32*r1 (inside the 128-row block) for
 * the 32-element group g; atoms are ordered [row block][K block]. dk_mx_sf_bytes(R, K) is the size
 * of the atom array for an [R, K] operand (R rounded up to 128 rows).
 *
 * dk_mx_quant: x [R, K] (bf16, or fp32 when x_is_f32) -> q e4m3 bytes [R, K], the scales row-major
 * s_rows [R, K/32] (may be NULL) and as atoms. scale = clamp(floor(log2(amax)) + 127, 0, 254), 0 for
 * an all-zero block; q = e4m3(x * 2^(127 - scale)), round to nearest even. K % 128 == 0.
 * Replaces the reference's host quantiser, compute_e8m0 and its loop
 * (kernels/cdna4/gemm/mxfp8/MXFP8_8wave/8_wave_NT.cu:286-327,
 * tests/unit/cdna4/warp/register/tile/mma_scaled.cu:200-232); the atoms replace its per-iteration
 * packed scale words (mma_scaled.cu:249-264).
 *
 * dk_gemm_mxfp8: C[M, N] = dequant(A) dequant(B)^T with A [M, K], B [N, K] e4m3 bytes and their
 * scale atoms; fp32 accumulation in tensor memory; C bf16 (out_f32 = 0) or fp32 (out_f32 = 1).
 * K % 128 == 0, N % 8 == 0. Replaces the reference's MXFP8 GEMM kernel (8_wave_NT.cu:432-496,
 * scaled MFMA at :39-44) and the register-tile op its fixture tests (mma_scaled.cu:107-198).
 */
size_t dk_mx_sf_bytes(int R, int K);
int dk_mx_quant(const void* x, int x_is_f32, int R, int K, void* q, void* s_rows, void* sf_atoms,
                void* stream);
int dk_gemm_mxfp8(const void* aq, const void* sfa, const void* bq, const void* sfb, void* C, int M, int N,
                  int K, int out_f32, void* stream);
/*
 * The MoE path on the same instruction, for 128x128 block scales that are powers of two (a
 * second quantisation mode beside the fp32 scales of dk_quant_block128 / dk_moe_grouped_gemm_fp8;
 * no reference counterpart, as for the other MoE entry points).
 *
 * "Block atoms": with one scale per 128x128 block the four scale bytes the tensor core holds per
 * row carry four consecutive K blocks instead of four 32-element groups. Per 128 rows and 512
 * elements of K one 512-byte atom: byte r*4 + g (r = 0..127 any row slot, g = 0..3) = scale byte of
 * block (row block, 4j + g); atoms ordered [row block][ceil(K/512)]. Bytes of K blocks that do not
 * exist are never read.
 *
 * dk_quant_block128_pow2: as dk_quant_block128 with s = 2^ceil(log2(amax/448)) (1 for an all-zero
 * block); besides q it writes s (fp32, may be NULL), e8 = log2(s) + 127 as bytes [R/128, C/128] (may
 * be NULL) and the block atoms [R/128][ceil(C/512)][512].
 *
 * dk_moe_grouped_gemm_mxfp8: as dk_moe_grouped_gemm_fp8 with block atoms in place of the fp32
 * scales: x_atoms [R/128][ceil(K/512)][512], w_atoms [E * rows/128][ceil(K/512)][512]. gated = 1
 * writes e4m3 bytes [R, N] of silu(gate) * up requantised per 128x128 block with a power-of-two
 * scale, out_e8 [R/128, N/128] and out_atoms [R/128][ceil(N/512)][512]; gated = 0 writes bf16 [R, N].
 */
/*
 * Which form of the block-scaled kernel runs: 1 = clusters of two CTAs per 256-row tile (tcgen05
 * cta_group::2: half the shared-memory fill per flop, a six-stage ring), 0 = one CTA per 128-row
 * tile, -1 (the default) = pairs for dk_gemm_mxfp8 and one CTA for dk_moe_grouped_gemm_mxfp8 (many
 * small experts leave half a pair idle). DK_MX_PAIR=0/1 in the environment does the same. Results
 * are identical. No reference counterpart.
 */
int dk_mx_pair_mode(int mode);
int dk_quant_block128_pow2(const void* x, int R, int C, const int* row_map, int map_mode, int k, void* q,
                           float* s, void* e8, void* sf_atoms, void* stream);
int dk_moe_grouped_gemm_mxfp8(const void* xq, const void* x_atoms, const void* wq, const void* w_atoms,
                              const int* offsets, int E, int R, int N, int K, int gated, void* out,
                              void* out_e8, void* out_atoms, void* stream);

/* ------------------------------------------------------------------ expert-parallel exchange */
/*
 * No counterpart in the reference (it has no all-to-all and no expert parallelism).
 * Token t lives on rank t / T_loc; expert e on rank e / experts_per_rank. All of these are
 * collective: every rank calls them in the same order.
 *
 * dk_peer_barrier: device-side barrier across the ranks of the view, ordered on `stream` (a
 * one-block kernel: release-store of the heap's epoch into every peer's flag, bounded wait for
 * theirs). Work enqueued before it on every rank is complete and visible after it on every rank.
 * dk_allgather: all[r*bytes .. (r+1)*bytes) = rank r's `mine`, on every rank. `all` lies inside the
 * heap (same offset everywhere); bytes % 16 == 0. Barriers before and after are included.
 */
int dk_peer_barrier(const dk_view* view, void* stream);
/* The same with an explicit 1-based epoch, for views that carry no heap handle. */
int dk_peer_barrier_epoch(const dk_view* view, unsigned epoch, void* stream);
int dk_allgather(const void* mine, size_t bytes, void* all, const dk_view* view, void* stream);
/*
 * dk_moe_dispatch: for each local token t and slot j, copy x[t, :] (H bf16) into row
 * row_of_pair[t,j] of the receive buffer `xrecv` of rank topk_idx[t,j] / experts_per_rank (peer
 * stores). row_of_pair is this rank's slice of the global permutation computed with one segment
 * per rank (dk_moe_permute, experts_per_segment = experts_per_rank). xrecv lies inside the heap.
 * sync != 0 brackets the copy with peer barriers (peers done with the old contents / all rows
 * landed); sync == 0 leaves ordering to the caller.
 * dk_moe_combine_ep: out[t,:] = sum_j topk_w[t,j] * y_of_rank(dest(t,j))[row_of_pair[t,j], :]
 * with peer loads; y lies inside the heap; fp32 accumulation, bf16 out.
 */
int dk_moe_dispatch(const void* x, const int* topk_idx, const int* row_of_pair, int T_loc, int k, int H,
                    int experts_per_rank, void* xrecv, const dk_view* view, int sync, void* stream);
int dk_moe_combine_ep(const void* y, const int* topk_idx, const int* row_of_pair, const float* topk_w,
                      int T_loc, int k, int H, int experts_per_rank, void* out, const dk_view* view,
                      int sync, void* stream);

/*
 * dk_moe_ep_layer: one fp8 MoE layer, expert-parallel over the ranks of the view, as ONE host call
 * that allocates nothing: routing, exchange of the routing table, permutation, dispatch, block
 * quantisation, gate/up + SiLU*mul + requantise, down, combine. No counterpart in the reference.
 *
 *  - Token t lives on rank t / T_loc, expert e on rank e / (E / world).
 *  - Dispatch sends each token ONCE to every rank that holds at least one of its experts (not once
 *    per expert); the receiving rank replicates it into its experts' rows while quantising.
 *  - Combine happens on the expert side: per (token, rank) one fp32 weighted sum of that rank's
 *    expert outputs, pushed back as one bf16 vector; the home rank adds the partials in rank order.
 *  - Work is bounded by the rows that actually arrived (the experts' offsets are read on the device).
 *  - No barrier launches: producers publish a per-source flag when their last CTA is done, consumers
 *    wait (bounded, see dk_set_peer_wait_ms) for all sources before they read.
 *
 * scale_mode 0: 128x128 blocks with fp32 scales (w13s [E/P, 2F/128, H/128], w2s [E/P, H/128, F/128]
 * fp32; dk_moe_grouped_gemm_fp8). scale_mode 1: the same blocks with power-of-two scales applied by
 * the tensor core (w13s, w2s are block atoms as dk_quant_block128_pow2 writes them;
 * dk_moe_grouped_gemm_mxfp8). scale_mode 2: weights as in mode 1; every token is quantised on its
 * home rank per 128 channels with a power-of-two scale (1x128 activation scales) and crosses NVLink
 * as H e4m3 bytes + H/128 scale bytes instead of 2H bytes of bf16; the receiving rank only gathers
 * bytes into expert order (the per-row scales are what the tensor core's scale atoms hold anyway).
 * H % 256 == 0, F % 128 == 0, E <= 256, k <= 8.
 *
 * workspace: dk_moe_ep_workspace_bytes(...) bytes, 256-byte aligned; for world > 1 inside the
 * symmetric heap at the same offset on every rank. Its contents need no initialisation. Calls on
 * one workspace must not overlap on the GPU. counts_out (device, may be NULL) receives the number of
 * pairs routed to each of this rank's E / world experts.
 *
 * `epoch`: 0 takes the next epoch of the view's heap (every rank calls in the same order); views
 * without a heap handle pass the 1-based call number. DK_EPOCH_DEVICE keeps the call number in device
 * memory instead (a word of this rank's control block, advanced by the call's last launch, with flags
 * of its own): nothing a launch is given then changes from call to call, so after one eager call the
 * work can be captured into a CUDA graph and replayed, every rank replaying the same number of
 * times; device-numbered and host-numbered calls can be mixed on one heap. A replay does not pass
 * through this library, so read dk_last_device_status() after replays. `phases` selects what is enqueued: 1 routing +
 * exchange, 2 permutation + dispatch, 4 experts + combine push, 8 final sum; 15 = the layer. Running
 * all ranks of a job on one GPU means phase by phase over the ranks (no launch then waits for a
 * later one).
 */
#define DK_EPOCH_DEVICE 0xFFFFFFFFu
typedef struct dk_moe_ep_args {
    int T_loc, k, E, H, F;
    int scale_mode;
    const void* x;        /* [T_loc, H] bf16 */
    const float* logits;  /* [T_loc, E] fp32 */
    const void* w13q;     /* [E/P, 2F, H] e4m3: gate rows, then up rows */
    const void* w13s;
    const void* w2q;      /* [E/P, H, F] e4m3 */
    const void* w2s;
    void* out;            /* [T_loc, H] bf16 */
    void* workspace;
    int* counts_out;
    void* ev_gemm_begin;  /* optional cudaEvent_t handles recorded on the stream just before and just */
    void* ev_gemm_end;    /* after the two grouped GEMMs (for timing them inside the layer); NULL: none */
} dk_moe_ep_args;
size_t dk_moe_ep_workspace_bytes(int T_loc, int k, int E, int H, int F, int world);
int dk_moe_ep_layer(const dk_moe_ep_args* args, const dk_view* view, unsigned epoch, int phases, void* stream);

/* ------------------------------------------------------------------ device helpers */
/* For hosts that link this library but not the CUDA runtime (the pybind11 modules). */
int dk_device_set(int device);
int dk_device_get(int* device);
int dk_device_count(int* count);
int dk_device_synchronize(void);

#ifdef __cplusplus
}
#endif
#endif /* DK_B200_H */
