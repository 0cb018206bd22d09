// Internal interface between the MoE translation units (dk_moe.cu, dk_moe_layer.cu): kernel
// launchers with the hooks the expert-parallel layer needs, and the two device-side halves of its
// rank-to-rank synchronisation.
//
// The expert-parallel layer has no separate barrier launches. A kernel that PRODUCES data in peer
// memory ends with ep_signal_done: every CTA fences and counts itself, the last one release-stores
// the call's epoch into flag [phase][this rank] of every rank. A kernel that CONSUMES such data
// starts with ep_wait_sources: thread r of every CTA waits (bounded) until flag [phase][r] has
// reached the epoch, for every source rank r. The reference has nothing of the kind (it has no
// exchange between ranks at all).
//
// The epoch is a host-side call number, or (epoch_ptr) one more than a word in this rank's device
// memory that the call itself advances when all of its kernels are through: the enqueued work then
// carries no host-side counter and can be replayed from a CUDA graph.
#pragma once
#include "dk_heap.h"
#include "dk_host.h"
#include "dk_ptx.cuh"

namespace dk {

enum : unsigned { SITE_EP_WAIT = 90 };

struct EpSignal {
    unsigned* counter;                 // CTAs of this launch that are done (local memory); null: no signal
    unsigned* flag[DK_MAX_RANKS];      // at rank r: flags[phase][this rank]
    int world;
    unsigned epoch;
    const unsigned* epoch_ptr;         // not null: the call number is *epoch_ptr + 1 (device-resident)
};

struct EpWait {
    const unsigned* flags;  // local flags[phase][source rank]; null: nothing to wait for
    int world;
    unsigned epoch;
    unsigned* status;
    unsigned long long limit_ns;
    const unsigned* epoch_ptr;  // as in EpSignal
};

// Called by every thread of the CTA once its stores have been issued.
__device__ __forceinline__ void ep_signal_done(const EpSignal& s) {
    if (s.counter == nullptr) return;
    __syncthreads();
    if (threadIdx.x == 0) {
        // this CTA's stores (peer stores among them) are ordered before its count ...
        __threadfence_system();
        const unsigned done = atomicAdd(s.counter, 1u) + 1u;
        if (done == gridDim.x * gridDim.y) {
            // ... and all counts before the flags: the last CTA publishes for the whole launch
            __threadfence_system();
            *s.counter = 0u;  // ready for the next launch on this stream
            const unsigned epoch = s.epoch_ptr != nullptr ? *s.epoch_ptr + 1u : s.epoch;
            for (int r = 0; r < s.world; ++r) signal_store_release_sys(s.flag[r], epoch);
        }
    }
}

// Called by every thread of the CTA before it reads what the sources wrote. False: a wait gave up
// (recorded); the caller leaves without touching the data.
__device__ __forceinline__ bool ep_wait_sources(const EpWait& w) {
    if (w.flags == nullptr) return true;
    __shared__ int ep_abort;
    if (threadIdx.x == 0) ep_abort = 0;
    __syncthreads();
    if (threadIdx.x < static_cast<unsigned>(w.world)) {
        const WaitCtx wc{w.status, &ep_abort, w.limit_ns};
        const unsigned epoch = w.epoch_ptr != nullptr ? *w.epoch_ptr + 1u : w.epoch;
        signal_wait_ge(w.flags + threadIdx.x, epoch, wc, SITE_EP_WAIT, threadIdx.x);
    }
    __syncthreads();
    return ep_abort == 0;
}

// Where moe_route writes: the same (idx, w) rows into n_out destinations (the local result, or the
// slice of every rank's gathered routing table), at row row_base + t.
struct RouteOut {
    int* idx[DK_MAX_RANKS];
    float* w[DK_MAX_RANKS];
    int n_out;
    int row_base;
};
int moe_route_launch(const float* logits, int T, int E, int k, const RouteOut& out, const EpSignal& sig,
                     cudaStream_t st);

int moe_permute_launch(const int* topk_idx, int T, int k, int E, int pad, int seg, int* row_of_pair,
                       int* pair_of_row, int seg_row_capacity, int* offsets, int* counts, int* scratch,
                       const EpWait& wait, cudaStream_t st);

// 128x128 block quantiser. map_mode 0..2 as dk_quant_block128; 3: row r of the output takes row
// map2[map[r] / k] of x (zeros where map[r] < 0 or that entry is negative). row_limit (device, may be
// null): rows at or beyond *row_limit are not produced. pow2: power-of-two scales + e8 + block atoms.
int quant_block128_launch(const void* x, int R, int C, const int* map, int map_mode, int k, const int* map2,
                          const int* row_limit, void* q, float* s, void* e8, void* atoms, bool pow2,
                          const EpWait& wait, cudaStream_t st);

}  // namespace dk
