// Host-side helpers shared by the C-ABI translation units: error strings, lazily resolved driver
// entry points (so that the library has no link-time dependency on libcuda and loads on a machine
// without a GPU), the per-device status record that bounded device waits write to.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <string>

#include "../../include/dk_b200.h"

namespace dk {

void set_last_error(const std::string& s);

// Host-side log to stderr, "[dk_b200] ...". Level 1: life cycle (heap created / destroyed, multicast
// mapping, workspaces taken from the heap, calls refused because of an unread device record);
// level 2: every peer mapping and rendezvous step. Shown when level <= DK_LOG (environment, default
// 0) or the value set with dk_set_log_level.
// Row tiles per band of the grouped GEMMs' tile walk: as many tiles of `tile_rows` x K bytes of the
// row operand as fit into the band size (32 MB, a quarter of L2, unless DK_WALK_BAND_MB or
// dk_set_walk_band_bytes says otherwise). At least 1.
int walk_band_tiles(int tile_rows, int K);

int log_level();
void log_msg(int level, const std::string& s);

#define DK_CUDA_OK(expr)                                                                      \
    do {                                                                                      \
        cudaError_t _e = (expr);                                                              \
        if (_e != cudaSuccess) {                                                              \
            ::dk::set_last_error(std::string(#expr) + ": " + cudaGetErrorString(_e));         \
            return DK_ERR_CUDA;                                                               \
        }                                                                                     \
    } while (0)

#define DK_CU_OK(expr)                                                                        \
    do {                                                                                      \
        CUresult _r = (expr);                                                                 \
        if (_r != CUDA_SUCCESS) {                                                             \
            ::dk::set_last_error(std::string(#expr) + ": CUresult " + std::to_string((int)_r)); \
            return DK_ERR_CUDA;                                                               \
        }                                                                                     \
    } while (0)

#define DK_REQUIRE(cond, msg)                                                                 \
    do {                                                                                      \
        if (!(cond)) {                                                                        \
            ::dk::set_last_error(std::string("argument error: ") + (msg));                    \
            return DK_ERR_ARG;                                                                \
        }                                                                                     \
    } while (0)

// Driver API entry points resolved through cudaGetDriverEntryPoint on first use.
struct DriverApi {
    bool ok = false;
    CUresult (*cuTensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                       const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                       const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                       CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
    CUresult (*cuMemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*,
                            unsigned long long) = nullptr;
    CUresult (*cuMemRelease)(CUmemGenericAllocationHandle) = nullptr;
    CUresult (*cuMemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr,
                                    unsigned long long) = nullptr;
    CUresult (*cuMemAddressFree)(CUdeviceptr, size_t) = nullptr;
    CUresult (*cuMemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle,
                         unsigned long long) = nullptr;
    CUresult (*cuMemUnmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*cuMemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
    CUresult (*cuMemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*,
                                              CUmemAllocationGranularity_flags) = nullptr;
    CUresult (*cuMemExportToShareableHandle)(void*, CUmemGenericAllocationHandle,
                                             CUmemAllocationHandleType,
                                             unsigned long long) = nullptr;
    CUresult (*cuMemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*,
                                               CUmemAllocationHandleType) = nullptr;
    // NVLink multicast objects (NVLS). Optional: mc_ok is false when the driver lacks them.
    bool mc_ok = false;
    CUresult (*cuDeviceGet)(CUdevice*, int) = nullptr;
    CUresult (*cuDeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
    CUresult (*cuMulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
    CUresult (*cuMulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
    CUresult (*cuMulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle,
                                   size_t, size_t, unsigned long long) = nullptr;
    CUresult (*cuMulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
    CUresult (*cuMulticastGetGranularity)(size_t*, const CUmulticastObjectProp*,
                                          CUmulticastGranularity_flags) = nullptr;
};
// Returns DK_OK and fills *api, or DK_ERR_CUDA when no driver is present.
int driver_api(const DriverApi** api);

// 2-D row-major tensor map: dims {inner, outer} elements, box {box_inner, box_outer}, 128-byte
// swizzle. elem_bytes 1 (uint8 / e4m3) or 2 (bf16).
int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner,
                 uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);
// 3-D: dims {inner, mid, outer}.
int make_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t mid,
                 uint64_t outer, uint64_t mid_stride_bytes, uint64_t outer_stride_bytes,
                 uint32_t box_inner, uint32_t box_mid, uint32_t box_outer);

// 4 words of host-mapped memory per device for the bounded-wait error record.
int device_status_ptr(unsigned** dev_ptr);
// DK_ERR_DEVICE while the current device holds an error record the host has not read yet with
// dk_last_device_status (the record is left in place), DK_OK otherwise. Collectives call this before
// they launch: with an unread record every later wait on a peer gives up at once, so their results
// would be wrong without any other sign.
int device_status_pending();

int sm_count(int* out);

// Limit of device-side waits on a signal from another rank, in nanoseconds
// (DK_PEER_WAIT_MS, default 20 s).
unsigned long long peer_wait_ns();

}  // namespace dk
