// Thin access layer to CUDA for host code.
//
// The library links the static CUDA runtime (which loads the driver lazily), so the same binary loads and runs its
// CPU-only paths on a machine without a GPU driver. Virtual-memory-management entry points (cuMem*, cuMulticast*) are
// driver API; they are fetched once through cudaGetDriverEntryPoint instead of linking libcuda. This replaces the
// reference's dlopen shims for vendor SDKs (src/hybm/csrc/under_api/dl_api.cpp:22-47, dl_hal_api.h:48-71 for the VMM
// family, dl_cuda_api.cpp:50-82 for its CUDA memcpy shim).
#pragma once
#include <cuda.h>
#include <cuda_runtime_api.h>

#include <string>

namespace mf {
namespace cu {

struct DriverApi {
    CUresult (*MemAddressReserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr, unsigned long long);
    CUresult (*MemAddressFree)(CUdeviceptr, size_t);
    CUresult (*MemCreate)(CUmemGenericAllocationHandle *, size_t, const CUmemAllocationProp *, unsigned long long);
    CUresult (*MemRelease)(CUmemGenericAllocationHandle);
    CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
    CUresult (*MemUnmap)(CUdeviceptr, size_t);
    CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t);
    CUresult (*MemExportToShareableHandle)(void *, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
    CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle *, void *, CUmemAllocationHandleType);
    CUresult (*MemGetAllocationGranularity)(size_t *, const CUmemAllocationProp *, CUmemAllocationGranularity_flags);
    CUresult (*MemRetainAllocationHandle)(CUmemGenericAllocationHandle *, void *);
    CUresult (*MemGetAddressRange)(CUdeviceptr *, size_t *, CUdeviceptr);
    CUresult (*MulticastCreate)(CUmemGenericAllocationHandle *, const CUmulticastObjectProp *);
    CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
    CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
    CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
    CUresult (*MulticastGetGranularity)(size_t *, const CUmulticastObjectProp *, CUmulticastGranularity_flags);
    CUresult (*DeviceGet)(CUdevice *, int);
    CUresult (*DeviceGetAttribute)(int *, CUdevice_attribute, CUdevice);
    CUresult (*GetErrorString)(CUresult, const char **);
    CUresult (*DriverGetVersion)(int *);
};

// Number of visible CUDA devices; 0 on a machine without a GPU or driver. Cached.
int DeviceCount();
inline bool Available() { return DeviceCount() > 0; }
// Driver VMM table; nullptr when no GPU is present or an entry point is missing.
const DriverApi *Driver();
std::string ErrStr(CUresult r);
std::string ErrStr(cudaError_t e);

struct DeviceCaps {
    int device{-1};
    bool vmm{false};
    bool posixFdHandle{false};
    bool fabricHandle{false};
    bool multicast{false};
    bool hostNumaVmm{false};
    bool hostPtrForRegistered{false};
    int numaNode{-1};
    int smCount{0};
    int driverVersion{0};
    int runtimeVersion{0};
};
// Capability probe of one device (reference: driver version / GVA ABI probe, src/hybm/csrc/hybm_driver.cpp:19-123).
int ProbeDevice(int device, DeviceCaps *out);

// Per-thread non-blocking stream for `device` (created on first use, lives until process exit).
// Reference: HybmStreamManager::GetThreadAclStream (src/hybm/csrc/ts_engine/hybm_stream_manager.cpp:24-57).
cudaStream_t ThreadStream(int device);

}  // namespace cu
}  // namespace mf

#define MF_CU_CHECK_RET(call, ret)                                                   \
    do {                                                                             \
        CUresult mf_cu_r_ = (call);                                                  \
        if (mf_cu_r_ != CUDA_SUCCESS) {                                              \
            MF_ERROR(#call << " failed: " << ::mf::cu::ErrStr(mf_cu_r_));            \
            return (ret);                                                            \
        }                                                                            \
    } while (0)

#define MF_CUDA_CHECK_RET(call, ret)                                                 \
    do {                                                                             \
        cudaError_t mf_cuda_e_ = (call);                                             \
        if (mf_cuda_e_ != cudaSuccess) {                                             \
            MF_ERROR(#call << " failed: " << ::mf::cu::ErrStr(mf_cuda_e_));          \
            return (ret);                                                            \
        }                                                                            \
    } while (0)
