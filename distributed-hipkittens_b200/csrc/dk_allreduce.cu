// Tensor-parallel all-reduce of bf16 activations over peer memory (NVLink / NVSwitch), no NCCL.
//
// The reference has no all-reduce (no collective of any kind exists under distributed-kernels/,
// include/ or kernels/); this is the operation the named hot path adds, built on the same symmetric
// heap and the same device-view convention as its GEMM (distributed-kernels/bf16_gemm/kernel.cpp:75).
//
// Three algorithms. The first two sum in fp32 in rank order, so every rank ends with identical bits:
//   one-shot  every rank reads all `world` inputs and writes the sum locally. (world-1) x S bytes
//             come in over NVLink; one exchange. For small messages (decode).
//   two-shot  rank r reduces slice r (reading the peers' slice r) and pushes the bf16 result into
//             every rank's output. 2 (world-1)/world x S bytes per direction. For large messages.
//
//   NVLS      rank r reduces slice r with multimem.ld_reduce (the NVSwitch fetches the slice from
//             every GPU and adds in fp32) and broadcasts the result with multimem.st (the switch
//             writes it into every rank's output). About S bytes per direction per GPU, for every
//             world size. Needs the heap's multicast mapping (dk_view.mc_base). The order of the
//             switch's sum is not specified, but each element is reduced once and then broadcast,
//             so all ranks still hold identical bits.
//
// Synchronisation is per block: block b of every rank handles the same elements, so block b only
// has to meet the peers' block b. Flags live in the control block at the start of each rank's heap,
// take the value of the heap's collective epoch (they only grow, nothing is reset), are written
// with st.release.sys and read with ld.acquire.sys, and every wait is bounded.
//
// All ranks of a job can also be run inside ONE cooperative launch on one GPU (blockIdx.y = rank):
// that is how the single-GPU tests drive the multi-rank path, since separate launches that wait for
// one another on one device are not guaranteed to be co-resident.
#include "dk_heap.h"
#include "dk_host.h"
#include "dk_ptx.cuh"

#include <cstdlib>

namespace dk {

constexpr int AR_THREADS = 512;
constexpr int AR_MAX_BLOCKS = 512;  // flag capacity in the control block

struct ARRank {
    const uint4* x[DK_MAX_RANKS];   // input of rank r as seen from this rank
    uint4* out[DK_MAX_RANKS];       // output of rank r as seen from this rank (two-shot pushes)
    unsigned* ctrl[DK_MAX_RANKS];   // control block of rank r
    const uint4* mc_x;              // NVLS: input and output through the multicast mapping
    uint4* mc_out;
    int rank;
};
struct ARJob {
    ARRank r[DK_MAX_RANKS];  // real launch: only r[0]; emulated launch: one per blockIdx.y
    int world;
    int algo;                // 0 one-shot, 1 two-shot, 2 NVLS
    unsigned epoch;
    size_t nvec;             // 16-byte vectors (8 bf16) per rank input
    unsigned* status;
    unsigned long long peer_wait_ns;
};

enum : unsigned { SITE_AR_START = 16, SITE_AR_END = 17 };

__device__ __forceinline__ void add8(float (&acc)[8], const uint4& u) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float (&acc)[8]) {
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    return o;
}

// Meet block `b` of every peer: tell each peer this rank has reached `epoch`, then wait for theirs.
template <bool RELEASE>
__device__ __forceinline__ bool block_meet(const ARRank& me, int world, size_t flag_base, int b,
                                           unsigned epoch, const WaitCtx& wc, unsigned site) {
    __syncthreads();
    if (threadIdx.x < world) {
        const int r = threadIdx.x;
        // the release store itself orders everything this block did before the __syncthreads above
        // (cumulativity); a separate system fence next to NVLink traffic costs tens of microseconds
        unsigned* flag = me.ctrl[r] + flag_base + static_cast<size_t>(b) * DK_MAX_RANKS + me.rank;
        if (RELEASE) signal_store_release_sys(flag, epoch);
        else signal_store_relaxed_sys(flag, epoch);
        signal_wait_ge(me.ctrl[me.rank] + flag_base + static_cast<size_t>(b) * DK_MAX_RANKS + r, epoch, wc, site, r);
    }
    __syncthreads();
    return *wc.abort_sm == 0;
}

__global__ void __launch_bounds__(AR_THREADS) allreduce_kernel(const __grid_constant__ ARJob job) {
    __shared__ int abort_sm;
    const ARRank& me = job.r[blockIdx.y];
    const int world = job.world;
    const int b = blockIdx.x;
    if (threadIdx.x == 0) abort_sm = 0;
    const WaitCtx wc{job.status, &abort_sm, job.peer_wait_ns};

    // every peer has entered the kernel, so its input (written by earlier work on its stream) is
    // complete; this block has published nothing yet, so the arrival flag needs no release
    if (!block_meet<false>(me, world, DK_CTRL_AR_START, b, job.epoch, wc, SITE_AR_START)) return;

    const size_t stride = static_cast<size_t>(gridDim.x) * AR_THREADS;
    if (job.algo == 0) {
        for (size_t i = static_cast<size_t>(b) * AR_THREADS + threadIdx.x; i < job.nvec; i += stride) {
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            uint4 v[DK_MAX_RANKS];
#pragma unroll
            for (int r = 0; r < DK_MAX_RANKS; ++r)
                if (r < world) v[r] = __ldcg(me.x[r] + i);
#pragma unroll
            for (int r = 0; r < DK_MAX_RANKS; ++r)
                if (r < world) add8(acc, v[r]);
            me.out[me.rank][i] = pack8(acc);
        }
    } else if (job.algo == 2) {
        const size_t slice = job.nvec / world;
        const size_t lo = slice * me.rank;
        size_t j = static_cast<size_t>(b) * AR_THREADS + threadIdx.x;
        // four independent switch reductions in flight per thread
        for (; j + 3 * stride < slice; j += 4 * stride) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = multimem_ld_reduce_add_bf16x8(me.mc_x + lo + j + u * stride);
#pragma unroll
            for (int u = 0; u < 4; ++u) multimem_st_bf16x8(me.mc_out + lo + j + u * stride, v[u]);
        }
        for (; j < slice; j += stride)
            multimem_st_bf16x8(me.mc_out + lo + j, multimem_ld_reduce_add_bf16x8(me.mc_x + lo + j));
    } else {
        const size_t slice = job.nvec / world;
        const size_t lo = slice * me.rank;
        for (size_t j = static_cast<size_t>(b) * AR_THREADS + threadIdx.x; j < slice; j += stride) {
            const size_t i = lo + j;
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            uint4 v[DK_MAX_RANKS];
#pragma unroll
            for (int r = 0; r < DK_MAX_RANKS; ++r)
                if (r < world) v[r] = __ldcg(me.x[r] + i);
#pragma unroll
            for (int r = 0; r < DK_MAX_RANKS; ++r)
                if (r < world) add8(acc, v[r]);
            const uint4 o = pack8(acc);
#pragma unroll
            for (int r = 0; r < DK_MAX_RANKS; ++r)
                if (r < world) me.out[r][i] = o;
        }
    }

    // one-shot: peers are done reading this rank's input; two-shot: the peers' pushes have landed
    block_meet<true>(me, world, DK_CTRL_AR_END, b, job.epoch, wc, SITE_AR_END);
}

static size_t oneshot_max_bytes(int world) {
    if (const char* e = std::getenv("DK_ALLREDUCE_ONESHOT_MAX_BYTES")) return std::strtoull(e, nullptr, 10);
    return world <= 2 ? (4u << 20) : world <= 4 ? (1u << 20) : (512u << 10);
}

// Whether algo -1 may pick NVLS when the mapping exists (DK_ALLREDUCE_NVLS_AUTO=0 turns that off).
static bool nvls_auto() {
    const char* e = std::getenv("DK_ALLREDUCE_NVLS_AUTO");
    return !(e && *e && std::atoi(e) == 0);
}

// Grid size, as measured on B200s: one 16-byte vector per thread while the message is small (a
// 1 MiB message on 2 GPUs takes 14 us with 128 blocks against 20 us with 32), at most two blocks
// per SM for the peer-load algorithms. NVLS saturates the switch with few requesters and slows
// down with more (8 GPUs, 128 MiB: 294 us with 16 blocks, 301 with 64, 347 with 296; 16 MiB: 49 us
// with 16 blocks, 59 with 64), so it gets at most 16 blocks (32 below four ranks).
static int pick_blocks(size_t work_vecs, int sms, int ranks_in_launch, int algo, int world) {
    // DK_ALLREDUCE_BLOCKS pins the grid (tuning; every rank must use the same value)
    if (const char* e = std::getenv("DK_ALLREDUCE_BLOCKS")) {
        const int v = std::atoi(e);
        if (v >= 1 && v <= AR_MAX_BLOCKS) return v;
    }
    const size_t per_block = algo == 2 ? AR_THREADS * 4 : AR_THREADS;
    size_t nb = (work_vecs + per_block - 1) / per_block;
    size_t cap = algo == 2 ? (world >= 4 ? 16 : 32) : static_cast<size_t>(sms) * 2 / ranks_in_launch;
    if (cap > AR_MAX_BLOCKS) cap = AR_MAX_BLOCKS;
    if (nb > cap) nb = cap;
    if (nb < 1) nb = 1;
    return static_cast<int>(nb);
}

// nvls_ok: the heap has a multicast mapping (real multi-GPU launches only).
static int resolve_algo(int algo, size_t n, int world, bool nvls_ok, int* out) {
    DK_REQUIRE(algo >= -1 && algo <= 2, "algo must be -1 (auto), 0 (one-shot), 1 (two-shot) or 2 (NVLS)");
    const bool two_ok = (n % (static_cast<size_t>(8) * world)) == 0;
    if (algo == 2) {
        if (!nvls_ok) {
            set_last_error("NVLS all-reduce needs the heap's NVLink multicast mapping, which this job does not "
                           "have (no multicast support, DK_NVLS=0, or the set-up failed on some rank)");
            return DK_ERR_UNSUPPORTED;
        }
        DK_REQUIRE(two_ok, "NVLS needs n to be a multiple of 8 * world elements");
    }
    if (algo == 1) DK_REQUIRE(two_ok, "two-shot needs n to be a multiple of 8 * world elements");
    if (algo == -1) {
        // With four or more ranks NVLS moves the fewest bytes and measured fastest at every size
        // (8 GPUs: 1 MiB 14.7 us against 17.9 two-shot, 128 MiB 294 us against 370). With two
        // ranks it moves 1.5x the bytes of two-shot and is never the better choice.
        if (nvls_ok && two_ok && world >= 4 && nvls_auto()) algo = 2;
        else algo = (two_ok && n * 2 > oneshot_max_bytes(world)) ? 1 : 0;
    }
    *out = algo;
    return DK_OK;
}

}  // namespace dk

extern "C" int dk_allreduce(const void* x, void* out, size_t n, int algo, const dk_view* view,
                            void* stream) {
    using namespace dk;
    DK_REQUIRE(x != nullptr && out != nullptr, "null buffer");
    DK_REQUIRE(n > 0 && n % 8 == 0, "n must be a positive multiple of 8 bf16 elements");
    DK_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
               "buffers must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (view == nullptr || view->world <= 1) {
        if (x != out) DK_CUDA_OK(cudaMemcpyAsync(out, x, n * 2, cudaMemcpyDeviceToDevice, st));
        return DK_OK;
    }
    const int world = view->world;
    DK_REQUIRE(world <= DK_MAX_RANKS && view->rank >= 0 && view->rank < world, "bad view");
    DK_REQUIRE(view->heap != nullptr, "view has no heap handle");
    DK_REQUIRE(in_heap(view, x, n * 2), "the all-reduce input must lie inside the symmetric heap");
    if (const int pending = device_status_pending()) return pending;
    int a = 0;
    // auto may pick NVLS only if `out` can be written through the multicast mapping; an explicit
    // request with `out` outside the heap is reported as such below
    const bool mc = view->mc_base != nullptr;
    int rc = resolve_algo(algo, n, world, algo == 2 ? mc : (mc && in_heap(view, out, n * 2)), &a);
    if (rc != DK_OK) return rc;
    if (a >= 1) DK_REQUIRE(in_heap(view, out, n * 2), "two-shot and NVLS write into the peers' outputs: out must lie inside the symmetric heap");
    if (a == 0) DK_REQUIRE(x != out, "one-shot cannot run in place: peers still read x while out is written");

    ARJob job{};
    job.world = world;
    job.algo = a;
    job.nvec = n / 8;
    job.epoch = heap_next_epoch(static_cast<dk_heap*>(view->heap));
    rc = device_status_ptr(&job.status);
    if (rc != DK_OK) return rc;
    job.peer_wait_ns = peer_wait_ns();
    ARRank& me = job.r[0];
    me.rank = view->rank;
    for (int r = 0; r < world; ++r) {
        me.x[r] = static_cast<const uint4*>(peer_ptr(view, x, r));
        me.out[r] = a == 1 ? static_cast<uint4*>(peer_ptr(view, out, r)) : static_cast<uint4*>(out);
        me.ctrl[r] = ctrl_words(view, r);
    }
    if (a == 2) {
        const char* base = static_cast<const char*>(view->base[view->rank]);
        char* mc = static_cast<char*>(view->mc_base);
        me.mc_x = reinterpret_cast<const uint4*>(mc + (static_cast<const char*>(x) - base));
        me.mc_out = reinterpret_cast<uint4*>(mc + (static_cast<const char*>(out) - base));
    }
    int sms = 0;
    rc = sm_count(&sms);
    if (rc != DK_OK) return rc;
    const int nb = pick_blocks(a >= 1 ? job.nvec / world : job.nvec, sms, 1, a, world);
    allreduce_kernel<<<dim3(nb, 1), AR_THREADS, 0, st>>>(job);
    DK_CUDA_OK(cudaGetLastError());
    return DK_OK;
}

extern "C" int dk_allreduce_all_ranks(int world, const dk_view* views, const void* const* x,
                                      void* const* out, size_t n, int algo, unsigned epoch,
                                      void* stream) {
    using namespace dk;
    DK_REQUIRE(world >= 2 && world <= DK_MAX_RANKS, "world must be 2..8");
    DK_REQUIRE(views != nullptr && x != nullptr && out != nullptr, "null argument");
    DK_REQUIRE(n > 0 && n % 8 == 0, "n must be a positive multiple of 8 bf16 elements");
    DK_REQUIRE(epoch != 0, "epochs start at 1");
    int a = 0;
    int rc = resolve_algo(algo, n, world, false, &a);  // ranks emulated on one GPU have no switch between them
    if (rc != DK_OK) return rc;
    ARJob job{};
    job.world = world;
    job.algo = a;
    job.nvec = n / 8;
    job.epoch = epoch;
    rc = device_status_ptr(&job.status);
    if (rc != DK_OK) return rc;
    job.peer_wait_ns = peer_wait_ns();
    for (int q = 0; q < world; ++q) {
        const dk_view* v = &views[q];
        DK_REQUIRE(v->rank == q && v->world == world, "views must be ordered by rank");
        DK_REQUIRE(in_heap(v, x[q], n * 2) && in_heap(v, out[q], n * 2), "buffers must lie inside each rank's heap");
        ARRank& me = job.r[q];
        me.rank = q;
        for (int r = 0; r < world; ++r) {
            me.x[r] = static_cast<const uint4*>(peer_ptr(v, x[q], r));
            me.out[r] = a == 1 ? static_cast<uint4*>(peer_ptr(v, out[q], r)) : static_cast<uint4*>(out[q]);
            me.ctrl[r] = ctrl_words(v, r);
        }
    }
    int sms = 0;
    rc = sm_count(&sms);
    if (rc != DK_OK) return rc;
    const int nb = pick_blocks(a == 1 ? job.nvec / world : job.nvec, sms, world, a, world);
    // all ranks' blocks wait for one another: they must be co-resident, hence a cooperative launch
    void* args[] = {&job};
    DK_CUDA_OK(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(allreduce_kernel), dim3(nb, world),
                                           dim3(AR_THREADS), args, 0, static_cast<cudaStream_t>(stream)));
    return DK_OK;
}
