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

#include <unistd.h>

#include <cstring>
#include <vector>

#include "dk_host.h"

extern "C" {
int dk_comm_create(int, int, const char*, int, dk_comm**);
int dk_comm_destroy(dk_comm*);
int dk_comm_barrier(dk_comm*);
int dk_comm_allgather_fd(dk_comm*, int, int*);
}

namespace {

size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int unmap_all(dk_heap* h, const dk::DriverApi* api) {
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
    if (h->comm) {
        rc = dk_comm_barrier(h->comm);
        if (rc != DK_OK) return bail(rc, "", CUDA_SUCCESS);
    }
    *out = h;
    return DK_OK;
}

int dk_heap_destroy(dk_heap* h) {
    if (h == nullptr) return DK_OK;
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
    out->mc_base = nullptr;
    out->heap = h;
    return DK_OK;
}

}  // extern "C"
