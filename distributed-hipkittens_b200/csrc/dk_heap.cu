// Symmetric heap over the CUDA virtual-memory-management API.
//
// Stands in for iris::iris, the host runtime behind the reference's iris_py
// (call sites distributed-kernels/iris_py.cpp:55-61 ctor, :89 allocate<char>, :24 deallocate,
// :100 barrier, :105 get_device_view). The iris source is not part of the reference tree; its
// contract is taken from those call sites: every rank owns `heap_size` bytes, the same allocation
// sequence yields the same offset on every rank, and a device handle lets a kernel address the
// same offset on any rank.
//
// Each rank cuMemCreate()s one physical allocation exportable as a POSIX file descriptor, the
// descriptors are all-gathered over the Unix-socket bootstrap, and every rank maps all `world`
// allocations back to back into one reserved address window: rank r's heap is at
// window + r * bytes. Peer traffic is then plain loads/stores (or TMA) on those addresses, routed
// over NVLink/NVSwitch by the memory system.
#include "dk_heap.h"

#include <fcntl.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "dk_host.h"

extern "C" {
int dk_comm_create(int, int, const char*, int, dk_comm**);
int dk_comm_destroy(dk_comm*);
int dk_comm_barrier(dk_comm*);
int dk_comm_allgather_fd(dk_comm*, int, int*);
int dk_comm_allgather(dk_comm*, const void*, size_t, void*);
}

namespace {

size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Take the multicast mapping down again (each step only if it was made).
void multicast_teardown(dk_heap* h, const dk::DriverApi* api) {
    if (h->mc_mapped) {
        api->cuMemUnmap(h->mc_window, h->bytes);
        h->mc_mapped = false;
    }
    if (h->mc_window) {
        api->cuMemAddressFree(h->mc_window, h->bytes);
        h->mc_window = 0;
    }
    if (h->mc_bound) {
        api->cuMulticastUnbind(h->mc_handle, h->mc_dev, 0, h->bytes);
        h->mc_bound = false;
    }
    if (h->mc_have) {
        api->cuMemRelease(h->mc_handle);
        h->mc_have = false;
    }
}

// True when every rank reports `mine` (one all-gather; also a barrier).
bool all_ranks_ok(dk_heap* h, bool mine) {
    int v = mine ? 1 : 0;
    int all[DK_MAX_RANKS] = {0};
    if (dk_comm_allgather(h->comm, &v, sizeof(v), all) != DK_OK) return false;
    for (int r = 0; r < h->world; ++r)
        if (!all[r]) return false;
    return true;
}

// DK_NVLS=1 makes dk_heap_create set the multicast mapping up by itself.
bool multicast_at_create() {
    const char* e = std::getenv("DK_NVLS");
    return e && *e && std::atoi(e) == 1;
}

// One NVLink multicast object over all ranks' heaps: rank 0 creates it and hands its descriptor
// round, every rank adds its device, then (all added) binds its own allocation at offset 0 and maps
// the object. A store to mc_window + o then lands at offset o of EVERY rank's heap and a
// multimem.ld_reduce there returns the sum over ranks, both performed by the switch. Every step
// is agreed between the ranks, so a failure anywhere leaves all of them without the mapping
// (dk_view.mc_base null) and the heap otherwise intact.
void multicast_setup(dk_heap* h, const dk::DriverApi* api) {
    bool ok = api->mc_ok && h->mc_gran != 0 && h->bytes % h->mc_gran == 0;
    if (!all_ranks_ok(h, ok)) return;

    CUmulticastObjectProp mp{};
    mp.numDevices = static_cast<unsigned>(h->world);
    mp.size = h->bytes;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    int my_fd = -1;
    if (h->rank == 0) {
        ok = api->cuMulticastCreate(&h->mc_handle, &mp) == CUDA_SUCCESS;
        h->mc_have = ok;
        if (ok)
            ok = api->cuMemExportToShareableHandle(&my_fd, h->mc_handle,
                                                   CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) == CUDA_SUCCESS;
    }
    if (my_fd < 0) my_fd = open("/dev/null", O_RDONLY);  // the exchange wants a descriptor from everyone
    if (my_fd < 0) ok = false;
    if (!all_ranks_ok(h, ok)) {
        if (my_fd >= 0) close(my_fd);
        multicast_teardown(h, api);
        return;
    }
    int fds[DK_MAX_RANKS];
    for (int& f : fds) f = -1;
    ok = dk_comm_allgather_fd(h->comm, my_fd, fds) == DK_OK;
    close(my_fd);
    if (ok && h->rank != 0) {
        ok = api->cuMemImportFromShareableHandle(&h->mc_handle,
                                                 reinterpret_cast<void*>(static_cast<uintptr_t>(fds[0])),
                                                 CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) == CUDA_SUCCESS;
        h->mc_have = ok;
    }
    for (int& f : fds)
        if (f >= 0) close(f);
    if (ok) ok = api->cuDeviceGet(&h->mc_dev, h->device) == CUDA_SUCCESS;
    if (ok) ok = api->cuMulticastAddDevice(h->mc_handle, h->mc_dev) == CUDA_SUCCESS;
    // memory may be bound only once ALL devices have been added: the agreement is the barrier
    if (!all_ranks_ok(h, ok)) {
        multicast_teardown(h, api);
        return;
    }
    ok = api->cuMulticastBindMem(h->mc_handle, 0, h->handles[h->rank], 0, h->bytes, 0) == CUDA_SUCCESS;
    h->mc_bound = ok;
    if (ok) ok = api->cuMemAddressReserve(&h->mc_window, h->bytes, h->mc_gran, 0, 0) == CUDA_SUCCESS;
    if (ok) {
        ok = api->cuMemMap(h->mc_window, h->bytes, 0, h->mc_handle, 0) == CUDA_SUCCESS;
        h->mc_mapped = ok;
    }
    if (ok) {
        CUmemAccessDesc acc{};
        acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        acc.location.id = h->device;
        acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        ok = api->cuMemSetAccess(h->mc_window, h->bytes, &acc, 1) == CUDA_SUCCESS;
    }
    if (!all_ranks_ok(h, ok)) multicast_teardown(h, api);
}

int unmap_all(dk_heap* h, const dk::DriverApi* api) {
    multicast_teardown(h, api);
    for (int r = 0; r < h->world; ++r) {
        if (h->mapped[r]) {
            api->cuMemUnmap(h->window + static_cast<size_t>(r) * h->bytes, h->bytes);
            h->mapped[r] = false;
        }
        if (h->have[r]) {
            api->cuMemRelease(h->handles[r]);
            h->have[r] = false;
        }
    }
    if (h->window) {
        api->cuMemAddressFree(h->window, h->bytes * h->world);
        h->window = 0;
    }
    return DK_OK;
}

}  // namespace

extern "C" {

int dk_heap_create(size_t bytes, int rank, int world, const char* rendezvous, dk_heap** out) {
    using namespace dk;
    DK_REQUIRE(out != nullptr, "out is null");
    DK_REQUIRE(world >= 1 && world <= DK_MAX_RANKS, "world must be 1..8");
    DK_REQUIRE(rank >= 0 && rank < world, "rank out of range");
    DK_REQUIRE(bytes > 0, "heap size must be positive");
    *out = nullptr;
    DK_CUDA_OK(cudaFree(nullptr));  // make sure the primary context exists
    const DriverApi* api;
    int rc = driver_api(&api);
    if (rc != DK_OK) return rc;

    dk_heap* h = new dk_heap;
    h->rank = rank;
    h->world = world;
    DK_CUDA_OK(cudaGetDevice(&h->device));

    CUmemAllocationProp prop{};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = h->device;
    prop.requestedHandleTypes =
        world > 1 ? CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR : CU_MEM_HANDLE_TYPE_NONE;
    size_t gran = 0;
    CUresult cr = api->cuMemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
    if (cr != CUDA_SUCCESS || gran == 0) {
        set_last_error("cuMemGetAllocationGranularity failed: CUresult " + std::to_string((int)cr));
        delete h;
        return DK_ERR_CUDA;
    }
    // With NVLink multicast available the heap is also a whole number of multicast granules, so
    // that it can be bound to a multicast object as one piece.
    if (world > 1 && api->mc_ok) {
        CUdevice cudev;
        int supported = 0;
        if (api->cuDeviceGet(&cudev, h->device) == CUDA_SUCCESS &&
            api->cuDeviceGetAttribute(&supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cudev) == CUDA_SUCCESS &&
            supported) {
            CUmulticastObjectProp mp{};
            mp.numDevices = static_cast<unsigned>(world);
            mp.size = round_up(bytes + DK_CTRL_BYTES, gran);
            mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
            size_t g_rec = 0, g_min = 0;
            if (api->cuMulticastGetGranularity(&g_min, &mp, CU_MULTICAST_GRANULARITY_MINIMUM) == CUDA_SUCCESS &&
                api->cuMulticastGetGranularity(&g_rec, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS &&
                g_min != 0) {
                // the recommended granule unless it would inflate small heaps beyond reason
                h->mc_gran = (g_rec != 0 && g_rec <= (64u << 20)) ? g_rec : g_min;
            }
        }
    }
    if (h->mc_gran > gran) gran = round_up(h->mc_gran, gran);
    h->bytes = round_up(bytes + DK_CTRL_BYTES, gran);

    if (world > 1) {
        rc = dk_comm_create(rank, world, rendezvous, 0, &h->comm);
        if (rc != DK_OK) {
            delete h;
            return rc;
        }
    }

    auto bail = [&](int code, const std::string& what, CUresult r) {
        if (r != CUDA_SUCCESS) set_last_error(what + ": CUresult " + std::to_string((int)r));
        unmap_all(h, api);
        if (h->comm) dk_comm_destroy(h->comm);
        delete h;
        return code;
    };

    cr = api->cuMemAddressReserve(&h->window, h->bytes * world, gran, 0, 0);
    if (cr != CUDA_SUCCESS) return bail(DK_ERR_CUDA, "cuMemAddressReserve", cr);

    cr = api->cuMemCreate(&h->handles[rank], h->bytes, &prop, 0);
    if (cr != CUDA_SUCCESS) return bail(DK_ERR_CUDA, "cuMemCreate", cr);
    h->have[rank] = true;

    std::vector<int> fds(world, -1);
    auto close_fds = [&] {
        for (int& fd : fds) {
            if (fd >= 0) close(fd);
            fd = -1;
        }
    };
    if (world > 1) {
        int my_fd = -1;
        cr = api->cuMemExportToShareableHandle(&my_fd, h->handles[rank],
                                               CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
        if (cr != CUDA_SUCCESS) return bail(DK_ERR_CUDA, "cuMemExportToShareableHandle", cr);
        rc = dk_comm_allgather_fd(h->comm, my_fd, fds.data());
        close(my_fd);
        if (rc != DK_OK) {
            close_fds();
            return bail(rc, "", CUDA_SUCCESS);
        }
    }

    CUmemAccessDesc acc{};
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = h->device;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    for (int r = 0; r < world; ++r) {
        if (r != rank) {
            cr = api->cuMemImportFromShareableHandle(
                &h->handles[r], reinterpret_cast<void*>(static_cast<uintptr_t>(fds[r])),
                CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
            if (cr != CUDA_SUCCESS) {
                close_fds();
                return bail(DK_ERR_CUDA, "cuMemImportFromShareableHandle(rank " + std::to_string(r) + ")", cr);
            }
            h->have[r] = true;
        }
        const CUdeviceptr at = h->window + static_cast<size_t>(r) * h->bytes;
        cr = api->cuMemMap(at, h->bytes, 0, h->handles[r], 0);
        if (cr != CUDA_SUCCESS) {
            close_fds();
            return bail(DK_ERR_CUDA, "cuMemMap(rank " + std::to_string(r) + ")", cr);
        }
        h->mapped[r] = true;
        if (log_level() >= 2) {
            char line[96];
            snprintf(line, sizeof line, "rank %d: heap of rank %d mapped at %#llx", rank, r, (unsigned long long)at);
            log_msg(2, line);
        }
        cr = api->cuMemSetAccess(at, h->bytes, &acc, 1);
        if (cr != CUDA_SUCCESS) {
            close_fds();
            return bail(DK_ERR_CUDA, "cuMemSetAccess(rank " + std::to_string(r) + ")", cr);
        }
    }
    close_fds();

    // flags start at zero; user memory too, so that a first epoch never sees garbage
    cudaError_t ce = cudaMemset(reinterpret_cast<void*>(h->window + static_cast<size_t>(rank) * h->bytes), 0, h->bytes);
    if (ce == cudaSuccess) ce = cudaDeviceSynchronize();
    if (ce != cudaSuccess) {
        set_last_error(std::string("zeroing the heap: ") + cudaGetErrorString(ce));
        return bail(DK_ERR_CUDA, "", CUDA_SUCCESS);
    }
    h->free_blocks[DK_CTRL_BYTES] = h->bytes - DK_CTRL_BYTES;
    if (h->comm && multicast_at_create()) multicast_setup(h, api);
    if (h->comm) {
        rc = dk_comm_barrier(h->comm);
        if (rc != DK_OK) return bail(rc, "", CUDA_SUCCESS);
    }
    *out = h;
    log_msg(1, "rank " + std::to_string(rank) + " of " + std::to_string(world) + ": symmetric heap of " +
                   std::to_string(h->bytes >> 20) + " MiB per rank on device " + std::to_string(h->device) +
                   (h->mc_mapped ? ", multicast mapped" : ""));
    return DK_OK;
}

int dk_heap_destroy(dk_heap* h) {
    if (h == nullptr) return DK_OK;
    dk::log_msg(1, "rank " + std::to_string(h->rank) + ": symmetric heap released");
    const dk::DriverApi* api;
    int rc = dk::driver_api(&api);
    if (rc != DK_OK) return rc;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(h->device);
    cudaDeviceSynchronize();
    // nobody may unmap while a peer could still be writing: meet first (best effort)
    if (h->comm) dk_comm_barrier(h->comm);
    unmap_all(h, api);
    if (h->comm) dk_comm_destroy(h->comm);
    cudaSetDevice(prev);
    delete h;
    return DK_OK;
}

int dk_heap_enable_multicast(dk_heap* h) {
    using namespace dk;
    DK_REQUIRE(h != nullptr, "heap is null");
    if (h->mc_mapped) return DK_OK;
    if (h->comm == nullptr) {
        set_last_error("NVLink multicast needs a job of at least two ranks");
        return DK_ERR_UNSUPPORTED;
    }
    const DriverApi* api;
    int rc = driver_api(&api);
    if (rc != DK_OK) return rc;
    int prev = 0;
    DK_CUDA_OK(cudaGetDevice(&prev));
    DK_CUDA_OK(cudaSetDevice(h->device));
    multicast_setup(h, api);
    cudaSetDevice(prev);
    log_msg(1, "rank " + std::to_string(h->rank) + (h->mc_mapped ? ": multicast mapping set up" : ": no multicast mapping"));
    if (!h->mc_mapped) {
        set_last_error("NVLink multicast mapping not available (no multicast support on some rank, or a set-up "
                       "step failed there); the heap works without it");
        return DK_ERR_UNSUPPORTED;
    }
    return DK_OK;
}

void* dk_heap_alloc(dk_heap* h, size_t bytes, size_t align) {
    if (h == nullptr) return nullptr;
    if (align == 0) align = 256;
    if ((align & (align - 1)) != 0) return nullptr;
    if (bytes == 0) bytes = 1;
    bytes = round_up(bytes, 256);
    std::lock_guard<std::mutex> lk(h->mu);
    // first fit in address order: deterministic, hence identical on every rank
    for (auto it = h->free_blocks.begin(); it != h->free_blocks.end(); ++it) {
        const size_t off = it->first, sz = it->second;
        const size_t a = round_up(off, align);
        if (a + bytes > off + sz) continue;
        h->free_blocks.erase(it);
        if (a > off) h->free_blocks[off] = a - off;
        if (a + bytes < off + sz) h->free_blocks[a + bytes] = off + sz - (a + bytes);
        h->used_blocks[a] = bytes;
        return reinterpret_cast<void*>(h->window + static_cast<size_t>(h->rank) * h->bytes + a);
    }
    dk::set_last_error("symmetric heap exhausted");
    return nullptr;
}

int dk_heap_free(dk_heap* h, void* p) {
    if (h == nullptr || p == nullptr) return DK_ERR_ARG;
    const size_t off = reinterpret_cast<CUdeviceptr>(p) - (h->window + static_cast<size_t>(h->rank) * h->bytes);
    std::lock_guard<std::mutex> lk(h->mu);
    auto it = h->used_blocks.find(off);
    if (it == h->used_blocks.end()) {
        dk::set_last_error("argument error: pointer was not allocated from this heap");
        return DK_ERR_ARG;
    }
    size_t start = off, size = it->second;
    h->used_blocks.erase(it);
    h->rs_seq.erase(p);
    auto next = h->free_blocks.lower_bound(start);
    if (next != h->free_blocks.end() && start + size == next->first) {
        size += next->second;
        next = h->free_blocks.erase(next);
    }
    if (next != h->free_blocks.begin()) {
        auto prev = std::prev(next);
        if (prev->first + prev->second == start) {
            start = prev->first;
            size += prev->second;
            h->free_blocks.erase(prev);
        }
    }
    h->free_blocks[start] = size;
    return DK_OK;
}

size_t dk_heap_bytes_free(dk_heap* h) {
    if (h == nullptr) return 0;
    std::lock_guard<std::mutex> lk(h->mu);
    size_t best = 0;
    for (auto& kv : h->free_blocks) best = kv.second > best ? kv.second : best;
    return best;
}

int dk_heap_barrier(dk_heap* h) {
    if (h == nullptr) return DK_ERR_ARG;
    if (h->comm == nullptr) return DK_OK;
    return dk_comm_barrier(h->comm);
}

int dk_heap_view(dk_heap* h, dk_view* out) {
    if (h == nullptr || out == nullptr) return DK_ERR_ARG;
    std::memset(out, 0, sizeof(*out));
    out->rank = h->rank;
    out->world = h->world;
    for (int r = 0; r < h->world; ++r)
        out->base[r] = reinterpret_cast<void*>(h->window + static_cast<size_t>(r) * h->bytes);
    out->heap_bytes = h->bytes;
    out->mc_base = h->mc_mapped ? reinterpret_cast<void*>(h->mc_window) : nullptr;
    out->heap = h;
    return DK_OK;
}

}  // extern "C"
