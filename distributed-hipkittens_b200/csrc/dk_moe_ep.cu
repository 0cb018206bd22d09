// Expert-parallel exchange over peer memory: device-side barrier, all-gather, dispatch, combine.
//
// The reference has no expert parallelism and no all-to-all; these are built on the same
// symmetric-heap convention as its GEMM (a device view that addresses the same offset on any
// rank, distributed-kernels/bf16_gemm/kernel.cpp:25,39,58-59). No NCCL.
//
// Layout: token t lives on rank t / T_loc, expert e on rank e / experts_per_rank. Every rank
// all-gathers the routing table (T*k int32, small), runs the same deterministic permutation with
// one segment per destination rank, and so knows the row every pair occupies at its destination:
//   dispatch  pushes each local token's hidden vector (H bf16) into row_of_pair of the destination
//             rank's receive buffer with 16-byte peer stores
//   combine   pulls, for each local token, its k expert outputs from the ranks that computed them
//             with 16-byte peer loads and forms sum_j w_j * y_j in fp32
// Each is bracketed by a peer barrier: a one-block kernel in which thread r release-stores the
// heap's epoch into rank r's flag and waits (bounded) for rank r's. Stream order makes the barrier
// cover the kernels launched before it.
#include "dk_heap.h"
#include "dk_host.h"
#include "dk_ptx.cuh"

namespace dk {

enum : unsigned { SITE_PEER_BARRIER = 48, SITE_AG = 49 };

struct BarrierArgs {
    unsigned* ctrl[DK_MAX_RANKS];
    int rank, world;
    unsigned epoch;
    unsigned* status;
    unsigned long long peer_wait_ns;
};

__global__ void __launch_bounds__(32) peer_barrier_kernel(const BarrierArgs a) {
    __shared__ int abort_sm;
    if (threadIdx.x == 0) abort_sm = 0;
    __syncwarp();
    const WaitCtx wc{a.status, &abort_sm, a.peer_wait_ns};
    if (threadIdx.x < a.world) {
        const int r = threadIdx.x;
        signal_store_release_sys(a.ctrl[r] + DK_CTRL_MOE + a.rank, a.epoch);
        signal_wait_ge(a.ctrl[a.rank] + DK_CTRL_MOE + r, a.epoch, wc, SITE_PEER_BARRIER, r);
    }
}

// out_r[rank * nvec + i] = mine[i] for every rank r
struct GatherArgs {
    const uint4* mine;
    uint4* out[DK_MAX_RANKS];
    int rank, world;
    size_t nvec;
};
__global__ void __launch_bounds__(256) allgather_push_kernel(const GatherArgs a) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < a.nvec; i += stride) {
        const uint4 v = a.mine[i];
#pragma unroll
        for (int r = 0; r < DK_MAX_RANKS; ++r)
            if (r < a.world) a.out[r][static_cast<size_t>(a.rank) * a.nvec + i] = v;
    }
}

struct DispatchArgs {
    const uint4* x;        // [T_loc, H/8]
    const int* topk_idx;   // [T_loc, k]
    const int* row_of_pair;  // [T_loc, k] row inside the destination rank's receive buffer
    uint4* recv[DK_MAX_RANKS];  // receive buffer of rank r as seen from here, [rows, H/8]
    int T_loc, k, hvec, experts_per_rank, world;
    unsigned* status;
};
enum : unsigned { SITE_EP_DEST = 82 };
__global__ void __launch_bounds__(256) moe_dispatch_kernel(const DispatchArgs a) {
    const int t = blockIdx.x;
    __shared__ int dst_s[8], row_s[8];
    if (threadIdx.x < a.k) {
        const int e = a.topk_idx[static_cast<size_t>(t) * a.k + threadIdx.x];
        int d = e >= 0 ? e / a.experts_per_rank : -1;
        int row = a.row_of_pair[static_cast<size_t>(t) * a.k + threadIdx.x];
        if (d < 0 || d >= a.world) {  // an expert no rank of this job holds: the pair is not sent
            record_bad_index(a.status, SITE_EP_DEST, static_cast<unsigned>(t * a.k + threadIdx.x));
            row = -1;
            d = 0;
        }
        dst_s[threadIdx.x] = d;
        row_s[threadIdx.x] = row;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < a.hvec; c += blockDim.x) {
        const uint4 v = a.x[static_cast<size_t>(t) * a.hvec + c];
        for (int j = 0; j < a.k; ++j)
            if (row_s[j] >= 0) a.recv[dst_s[j]][static_cast<size_t>(row_s[j]) * a.hvec + c] = v;
    }
}

struct CombineEpArgs {
    const uint4* y[DK_MAX_RANKS];  // expert outputs of rank r as seen from here, [rows, H/8]
    const int* topk_idx;
    const int* row_of_pair;
    const float* w;
    uint4* out;  // [T_loc, H/8]
    int T_loc, k, hvec, experts_per_rank, world;
    unsigned* status;
};
__global__ void __launch_bounds__(256) moe_combine_ep_kernel(const CombineEpArgs a) {
    const int t = blockIdx.x;
    __shared__ int dst_s[8], row_s[8];
    __shared__ float w_s[8];
    if (threadIdx.x < a.k) {
        const int e = a.topk_idx[static_cast<size_t>(t) * a.k + threadIdx.x];
        int d = e >= 0 ? e / a.experts_per_rank : -1;
        int row = a.row_of_pair[static_cast<size_t>(t) * a.k + threadIdx.x];
        if (d < 0 || d >= a.world) {
            record_bad_index(a.status, SITE_EP_DEST, static_cast<unsigned>(t * a.k + threadIdx.x));
            row = -1;
            d = 0;
        }
        dst_s[threadIdx.x] = d;
        row_s[threadIdx.x] = row;
        w_s[threadIdx.x] = a.w[static_cast<size_t>(t) * a.k + threadIdx.x];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < a.hvec; c += blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (j < a.k) v[j] = row_s[j] >= 0 ? __ldcg(a.y[dst_s[j]] + static_cast<size_t>(row_s[j]) * a.hvec + c)
                                              : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (j < a.k) {
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[j]);
                const float wj = w_s[j];
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
        a.out[static_cast<size_t>(t) * a.hvec + c] = o;
    }
}

static int launch_peer_barrier(const dk_view* view, cudaStream_t st, unsigned explicit_epoch = 0) {
    if (view == nullptr || view->world <= 1) return DK_OK;
    DK_REQUIRE(view->heap != nullptr || explicit_epoch != 0, "view has no heap handle");
    // before the epoch advances: a refused call must not leave this rank one epoch ahead
    if (const int pending = device_status_pending()) return pending;
    BarrierArgs a{};
    a.rank = view->rank;
    a.world = view->world;
    a.epoch = explicit_epoch ? explicit_epoch : heap_next_epoch(static_cast<dk_heap*>(view->heap));
    for (int r = 0; r < view->world; ++r) a.ctrl[r] = ctrl_words(view, r);
    int rc = device_status_ptr(&a.status);
    if (rc != DK_OK) return rc;
    a.peer_wait_ns = peer_wait_ns();
    peer_barrier_kernel<<<1, 32, 0, st>>>(a);
    DK_CUDA_OK(cudaGetLastError());
    return DK_OK;
}

static int check_ep(const dk_view* view, int T_loc, int k, int H, int experts_per_rank) {
    DK_REQUIRE(view != nullptr && view->world >= 1 && view->world <= DK_MAX_RANKS, "bad view");
    DK_REQUIRE(T_loc >= 0 && k >= 1 && k <= 8, "k must be 1..8");
    DK_REQUIRE(H > 0 && H % 8 == 0, "H must be a multiple of 8");
    DK_REQUIRE(experts_per_rank >= 1, "experts_per_rank must be positive");
    return DK_OK;
}

}  // namespace dk

extern "C" {

int dk_peer_barrier(const dk_view* view, void* stream) {
    return dk::launch_peer_barrier(view, static_cast<cudaStream_t>(stream));
}

int dk_peer_barrier_epoch(const dk_view* view, unsigned epoch, void* stream) {
    DK_REQUIRE(epoch != 0, "epochs start at 1");
    return dk::launch_peer_barrier(view, static_cast<cudaStream_t>(stream), epoch);
}

int dk_allgather(const void* mine, size_t bytes, void* all, const dk_view* view, void* stream) {
    using namespace dk;
    DK_REQUIRE(mine != nullptr && all != nullptr && view != nullptr, "null argument");
    DK_REQUIRE(bytes > 0 && bytes % 16 == 0, "bytes must be a positive multiple of 16");
    DK_REQUIRE((reinterpret_cast<uintptr_t>(mine) & 15) == 0 && (reinterpret_cast<uintptr_t>(all) & 15) == 0,
               "buffers must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int world = view->world;
    if (world > 1) DK_REQUIRE(in_heap(view, all, bytes * world), "the gathered buffer must lie inside the symmetric heap");
    GatherArgs a{};
    a.mine = static_cast<const uint4*>(mine);
    a.rank = view->rank;
    a.world = world;
    a.nvec = bytes / 16;
    for (int r = 0; r < world; ++r)
        a.out[r] = static_cast<uint4*>(world > 1 ? peer_ptr(view, all, r) : all);
    // the peers must be done with the previous contents of `all` before it is overwritten
    int rc = launch_peer_barrier(view, st);
    if (rc != DK_OK) return rc;
    size_t nb = (a.nvec + 255) / 256;
    if (nb > 592) nb = 592;
    allgather_push_kernel<<<static_cast<int>(nb), 256, 0, st>>>(a);
    DK_CUDA_OK(cudaGetLastError());
    return launch_peer_barrier(view, st);
}

int dk_moe_dispatch(const void* x, const int* topk_idx, const int* row_of_pair, int T_loc, int k, int H,
                    int experts_per_rank, void* xrecv, const dk_view* view, int sync, void* stream) {
    using namespace dk;
    int rc = check_ep(view, T_loc, k, H, experts_per_rank);
    if (rc != DK_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    DK_REQUIRE(xrecv != nullptr, "null receive buffer");
    if (view->world > 1)
        DK_REQUIRE(in_heap(view, xrecv, 16), "the receive buffer must lie inside the symmetric heap");
    // every rank has finished reading the previous contents of its receive buffer
    if (sync) {
        rc = launch_peer_barrier(view, st);
        if (rc != DK_OK) return rc;
    }
    if (T_loc > 0) {
        DK_REQUIRE(x && topk_idx && row_of_pair, "null buffer");
        DispatchArgs a{};
        a.x = static_cast<const uint4*>(x);
        a.topk_idx = topk_idx;
        a.row_of_pair = row_of_pair;
        a.T_loc = T_loc;
        a.k = k;
        a.hvec = H / 8;
        a.experts_per_rank = experts_per_rank;
        a.world = view->world;
        rc = device_status_ptr(&a.status);
        if (rc != DK_OK) return rc;
        for (int r = 0; r < view->world; ++r)
            a.recv[r] = static_cast<uint4*>(view->world > 1 ? peer_ptr(view, xrecv, r) : xrecv);
        moe_dispatch_kernel<<<T_loc, 256, 0, st>>>(a);
        DK_CUDA_OK(cudaGetLastError());
    }
    // every rank's rows have landed here
    if (sync) return launch_peer_barrier(view, st);
    return DK_OK;
}

int dk_moe_combine_ep(const void* y, const int* topk_idx, const int* row_of_pair, const float* topk_w,
                      int T_loc, int k, int H, int experts_per_rank, void* out, const dk_view* view,
                      int sync, void* stream) {
    using namespace dk;
    int rc = check_ep(view, T_loc, k, H, experts_per_rank);
    if (rc != DK_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    DK_REQUIRE(y != nullptr, "null expert output buffer");
    if (view->world > 1)
        DK_REQUIRE(in_heap(view, y, 16), "the expert outputs must lie inside the symmetric heap");
    // every rank's expert outputs are complete
    if (sync) {
        rc = launch_peer_barrier(view, st);
        if (rc != DK_OK) return rc;
    }
    if (T_loc > 0) {
        DK_REQUIRE(topk_idx && row_of_pair && topk_w && out, "null buffer");
        CombineEpArgs a{};
        a.topk_idx = topk_idx;
        a.row_of_pair = row_of_pair;
        a.w = topk_w;
        a.out = static_cast<uint4*>(out);
        a.T_loc = T_loc;
        a.k = k;
        a.hvec = H / 8;
        a.experts_per_rank = experts_per_rank;
        a.world = view->world;
        rc = device_status_ptr(&a.status);
        if (rc != DK_OK) return rc;
        for (int r = 0; r < view->world; ++r)
            a.y[r] = static_cast<const uint4*>(view->world > 1 ? peer_ptr(view, y, r) : y);
        moe_combine_ep_kernel<<<T_loc, 256, 0, st>>>(a);
        DK_CUDA_OK(cudaGetLastError());
    }
    // every rank is done reading this rank's expert outputs
    if (sync) return launch_peer_barrier(view, st);
    return DK_OK;
}

}  // extern "C"
