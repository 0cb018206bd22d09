// Internal view of the symmetric heap shared by the translation units of libdk_b200.
#pragma once
#include <cuda.h>

#include <map>
#include <mutex>
#include <utility>

#include "../../include/dk_b200.h"

// The first DK_CTRL_BYTES of every rank's heap are the control block: 4-byte signal counters
// written by peers with release stores and read with acquire loads. They start at zero and only
// ever take the value of a collective's epoch, so they are never reset.
constexpr size_t DK_CTRL_BYTES = 1u << 20;
// control block layout, in 4-byte words
constexpr size_t DK_CTRL_AR_START = 0;         // all-reduce start flags  [512 blocks][8 ranks]
constexpr size_t DK_CTRL_AR_END = 4096;        // all-reduce end flags    [512 blocks][8 ranks]
constexpr size_t DK_CTRL_MOE = 8192;           // MoE dispatch/combine    [2][512][8]
constexpr size_t DK_CTRL_WORDS = DK_CTRL_BYTES / 4;

struct dk_comm;

struct dk_heap {
    int rank = 0;
    int world = 1;
    int device = 0;
    size_t bytes = 0;  // per rank, rounded up to the allocation granularity
    CUdeviceptr window = 0;  // world * bytes of reserved address space; rank r at window + r*bytes
    CUmemGenericAllocationHandle handles[DK_MAX_RANKS] = {};
    bool have[DK_MAX_RANKS] = {};    // handles[r] holds a reference
    bool mapped[DK_MAX_RANKS] = {};  // rank r's segment is mapped into the window
    // NVLink multicast object over all ranks' heaps (NVLS); zero when not set up
    CUmemGenericAllocationHandle mc_handle = 0;
    bool mc_have = false, mc_bound = false, mc_mapped = false;
    CUdevice mc_dev = 0;
    size_t mc_gran = 0;         // multicast granule the heap size was rounded to (0: no multicast)
    CUdeviceptr mc_window = 0;  // `bytes` of address space: offset o = offset o of EVERY rank's heap
    dk_comm* comm = nullptr;
    unsigned epoch = 0;
    std::mutex mu;
    std::map<size_t, size_t> free_blocks;  // offset -> size, coalesced
    std::map<size_t, size_t> used_blocks;  // offset -> size
    std::map<void*, unsigned> rs_seq;      // per GEMM+RS workspace: calls made so far
    std::map<std::pair<int, int>, void*> rs_ws;  // workspaces the heap owns, by (M, N); they die with it
    std::map<std::pair<int, int>, void*> ag_ws;  // the same for all-gather + GEMM, by (M, K)
};

namespace dk {
// Next collective epoch of this heap (all ranks call collectives in the same order).
inline unsigned heap_next_epoch(dk_heap* h) { return ++h->epoch; }
inline unsigned* ctrl_words(const dk_view* v, int r) { return static_cast<unsigned*>(v->base[r]); }
// Translate a pointer into this rank's heap to the same offset of rank r's heap.
inline void* peer_ptr(const dk_view* v, const void* local, int r) {
    const char* b = static_cast<const char*>(v->base[v->rank]);
    return static_cast<char*>(v->base[r]) + (static_cast<const char*>(local) - b);
}
inline bool in_heap(const dk_view* v, const void* p, size_t bytes) {
    const char* b = static_cast<const char*>(v->base[v->rank]);
    const char* q = static_cast<const char*>(p);
    return q >= b + DK_CTRL_BYTES && q + bytes <= b + v->heap_bytes;
}
}  // namespace dk
