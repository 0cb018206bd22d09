// Host-side common code of libdk_b200: error text, driver entry points, tensor-map encoding,
// the device status record.
#include "dk_host.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace dk {

static thread_local std::string g_last_error;

void set_last_error(const std::string& s) { g_last_error = s; }

static long long g_band_bytes = 0;
int walk_band_tiles(int tile_rows, int K) {
    if (g_band_bytes == 0) {
        const char* e = std::getenv("DK_WALK_BAND_MB");
        const long long mb = (e && *e) ? std::atoll(e) : 32;
        g_band_bytes = (mb > 0 ? mb : 32) << 20;
    }
    const long long t = g_band_bytes / (static_cast<long long>(tile_rows) * K);
    return t < 1 ? 1 : (t > (1 << 20) ? (1 << 20) : static_cast<int>(t));
}

static int g_log_level = -1;
int log_level() {
    if (g_log_level < 0) {
        const char* e = std::getenv("DK_LOG");
        g_log_level = (e && *e) ? std::atoi(e) : 0;
        if (g_log_level < 0) g_log_level = 0;
    }
    return g_log_level;
}
void log_msg(int level, const std::string& s) {
    if (level <= log_level()) fprintf(stderr, "[dk_b200] %s\n", s.c_str());
}

static DriverApi g_api;
static std::once_flag g_api_once;
static int g_api_rc = DK_ERR_CUDA;

template <typename F>
static bool resolve(const char* name, F* fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
        (void)cudaGetLastError();
        set_last_error(std::string("cudaGetDriverEntryPoint failed for ") + name);
        return false;
    }
    *fn = reinterpret_cast<F>(p);
    return true;
}

int driver_api(const DriverApi** api) {
    std::call_once(g_api_once, [] {
        bool ok = true;
        ok = ok && resolve("cuTensorMapEncodeTiled", &g_api.cuTensorMapEncodeTiled);
        ok = ok && resolve("cuMemCreate", &g_api.cuMemCreate);
        ok = ok && resolve("cuMemRelease", &g_api.cuMemRelease);
        ok = ok && resolve("cuMemAddressReserve", &g_api.cuMemAddressReserve);
        ok = ok && resolve("cuMemAddressFree", &g_api.cuMemAddressFree);
        ok = ok && resolve("cuMemMap", &g_api.cuMemMap);
        ok = ok && resolve("cuMemUnmap", &g_api.cuMemUnmap);
        ok = ok && resolve("cuMemSetAccess", &g_api.cuMemSetAccess);
        ok = ok && resolve("cuMemGetAllocationGranularity", &g_api.cuMemGetAllocationGranularity);
        ok = ok && resolve("cuMemExportToShareableHandle", &g_api.cuMemExportToShareableHandle);
        ok = ok && resolve("cuMemImportFromShareableHandle", &g_api.cuMemImportFromShareableHandle);
        g_api.ok = ok;
        g_api_rc = ok ? DK_OK : DK_ERR_CUDA;
        bool mc = ok;
        mc = mc && resolve("cuDeviceGet", &g_api.cuDeviceGet);
        mc = mc && resolve("cuDeviceGetAttribute", &g_api.cuDeviceGetAttribute);
        mc = mc && resolve("cuMulticastCreate", &g_api.cuMulticastCreate);
        mc = mc && resolve("cuMulticastAddDevice", &g_api.cuMulticastAddDevice);
        mc = mc && resolve("cuMulticastBindMem", &g_api.cuMulticastBindMem);
        mc = mc && resolve("cuMulticastUnbind", &g_api.cuMulticastUnbind);
        mc = mc && resolve("cuMulticastGetGranularity", &g_api.cuMulticastGetGranularity);
        g_api.mc_ok = mc;
    });
    *api = &g_api;
    return g_api_rc;
}

int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner,
                 uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner,
                 uint32_t box_outer) {
    const DriverApi* api;
    int rc = driver_api(&api);
    if (rc != DK_OK) return rc;
    DK_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "tensor base must be 16-byte aligned");
    DK_REQUIRE((row_stride_bytes & 15) == 0, "row stride must be a multiple of 16 bytes");
    DK_REQUIRE(box_inner * elem_bytes == 128, "inner box must span 128 bytes");
    DK_REQUIRE(box_outer >= 1 && box_outer <= 256, "outer box out of range");
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapDataType dt =
        elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    DK_CU_OK(api->cuTensorMapEncodeTiled(out, dt, 2, const_cast<void*>(base), dims, strides, box,
                                         estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    return DK_OK;
}

int make_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t mid,
                 uint64_t outer, uint64_t mid_stride_bytes, uint64_t outer_stride_bytes,
                 uint32_t box_inner, uint32_t box_mid, uint32_t box_outer) {
    const DriverApi* api;
    int rc = driver_api(&api);
    if (rc != DK_OK) return rc;
    DK_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "tensor base must be 16-byte aligned");
    DK_REQUIRE((mid_stride_bytes & 15) == 0 && (outer_stride_bytes & 15) == 0,
               "strides must be multiples of 16 bytes");
    DK_REQUIRE(box_inner * elem_bytes == 128, "inner box must span 128 bytes");
    cuuint64_t dims[3] = {inner, mid, outer};
    cuuint64_t strides[2] = {mid_stride_bytes, outer_stride_bytes};
    cuuint32_t box[3] = {box_inner, box_mid, box_outer};
    cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMapDataType dt =
        elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    DK_CU_OK(api->cuTensorMapEncodeTiled(out, dt, 3, const_cast<void*>(base), dims, strides, box,
                                         estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    return DK_OK;
}

static std::mutex g_status_mu;
static unsigned* g_status_host[64] = {nullptr};
static unsigned* g_status_dev[64] = {nullptr};

int device_status_ptr(unsigned** dev_ptr) {
    int dev = 0;
    DK_CUDA_OK(cudaGetDevice(&dev));
    DK_REQUIRE(dev >= 0 && dev < 64, "device index out of range");
    std::lock_guard<std::mutex> lk(g_status_mu);
    if (g_status_dev[dev] == nullptr) {
        unsigned* h = nullptr;
        DK_CUDA_OK(cudaHostAlloc(reinterpret_cast<void**>(&h), 4 * sizeof(unsigned),
                                 cudaHostAllocMapped | cudaHostAllocPortable));
        std::memset(h, 0, 4 * sizeof(unsigned));
        unsigned* d = nullptr;
        DK_CUDA_OK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&d), h, 0));
        g_status_host[dev] = h;
        g_status_dev[dev] = d;
    }
    *dev_ptr = g_status_dev[dev];
    return DK_OK;
}

int device_status_pending() {
    int dev = 0;
    DK_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return DK_OK;
    unsigned code = 0, block = 0, site = 0, detail = 0;
    {
        std::lock_guard<std::mutex> lk(g_status_mu);
        const volatile unsigned* h = g_status_host[dev];
        if (h == nullptr || h[0] == 0u) return DK_OK;
        code = h[0];
        block = h[1];
        site = h[2];
        detail = h[3];
    }
    log_msg(1, "collective refused: unread device record, code " + std::to_string(code) + " site " + std::to_string(site));
    set_last_error("an earlier kernel on this device recorded an error (code " + std::to_string(code) +
                   ", block " + std::to_string(block) + ", site " + std::to_string(site) + ", detail " +
                   std::to_string(detail) + ") that has not been read with dk_last_device_status; "
                   "nothing was launched");
    return DK_ERR_DEVICE;
}

static int g_sm_count[64] = {0};
int sm_count(int* out) {
    int dev = 0;
    DK_CUDA_OK(cudaGetDevice(&dev));
    DK_REQUIRE(dev >= 0 && dev < 64, "device index out of range");
    if (g_sm_count[dev] == 0) {
        int n = 0;
        DK_CUDA_OK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
        g_sm_count[dev] = n;
    }
    *out = g_sm_count[dev];
    return DK_OK;
}

static std::mutex g_wait_mu;
static long long g_peer_wait_ms = -1;
unsigned long long peer_wait_ns() {
    std::lock_guard<std::mutex> lk(g_wait_mu);
    if (g_peer_wait_ms < 0) {
        const char* e = std::getenv("DK_PEER_WAIT_MS");
        g_peer_wait_ms = (e && *e) ? std::atoll(e) : 20000;
        if (g_peer_wait_ms < 1) g_peer_wait_ms = 1;
    }
    return static_cast<unsigned long long>(g_peer_wait_ms) * 1000000ull;
}

}  // namespace dk

extern "C" {

int dk_set_walk_band_bytes(size_t bytes) {
    if (bytes == 0 || bytes > (size_t{1} << 40)) return DK_ERR_ARG;
    dk::g_band_bytes = static_cast<long long>(bytes);
    return DK_OK;
}

int dk_set_log_level(int level) {
    if (level < 0 || level > 2) return DK_ERR_ARG;
    dk::g_log_level = level;
    return DK_OK;
}

int dk_set_peer_wait_ms(int ms) {
    if (ms < 1) return DK_ERR_ARG;
    std::lock_guard<std::mutex> lk(dk::g_wait_mu);
    dk::g_peer_wait_ms = ms;
    return DK_OK;
}


const char* dk_strerror(int code) {
    switch (code) {
        case DK_OK: return "ok";
        case DK_ERR_ARG: return "invalid argument";
        case DK_ERR_CUDA: return "CUDA call failed";
        case DK_ERR_DEVICE: return "device-side error record pending (a bounded wait gave up, or a bad index was skipped)";
        case DK_ERR_BOOTSTRAP: return "rank rendezvous failed";
        case DK_ERR_NOMEM: return "symmetric heap exhausted";
        case DK_ERR_UNSUPPORTED: return "not supported on this device";
        default: return "unknown error";
    }
}

const char* dk_last_error_string(void) { return dk::g_last_error.c_str(); }

int dk_version(void) { return 1000; }

int dk_last_device_status(unsigned out[4]) {
    if (out == nullptr) return DK_ERR_ARG;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        (void)cudaGetLastError();
        out[0] = out[1] = out[2] = out[3] = 0;
        return DK_ERR_CUDA;
    }
    std::lock_guard<std::mutex> lk(dk::g_status_mu);
    unsigned* h = (dev >= 0 && dev < 64) ? dk::g_status_host[dev] : nullptr;
    if (h == nullptr) {
        out[0] = out[1] = out[2] = out[3] = 0;
        return DK_OK;
    }
    for (int i = 0; i < 4; ++i) out[i] = reinterpret_cast<volatile unsigned*>(h)[i];
    for (int i = 3; i >= 0; --i) reinterpret_cast<volatile unsigned*>(h)[i] = 0;
    return DK_OK;
}

int dk_device_set(int device) {
    DK_CUDA_OK(cudaSetDevice(device));
    return DK_OK;
}
int dk_device_get(int* device) {
    DK_REQUIRE(device != nullptr, "null");
    DK_CUDA_OK(cudaGetDevice(device));
    return DK_OK;
}
int dk_device_count(int* count) {
    DK_REQUIRE(count != nullptr, "null");
    DK_CUDA_OK(cudaGetDeviceCount(count));
    return DK_OK;
}
int dk_device_synchronize(void) {
    DK_CUDA_OK(cudaDeviceSynchronize());
    return DK_OK;
}

}  // extern "C"
