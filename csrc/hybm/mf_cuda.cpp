#include "mf_cuda.h"

#include <mutex>
#include <unordered_map>

#include "../util/mf_log.h"

namespace mf {
namespace cu {

int DeviceCount()
{
    static int count = []() {
        int n = 0;
        cudaError_t e = cudaGetDeviceCount(&n);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();  // clear the sticky "no device / insufficient driver" error
            return 0;
        }
        return n;
    }();
    return count;
}

template <typename F>
static bool Fetch(const char *name, F *out)
{
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult st = cudaDriverEntryPointSymbolNotFound;
    cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &st);
    if (e != cudaSuccess || st != cudaDriverEntryPointSuccess || fn == nullptr) {
        (void)cudaGetLastError();
        MF_WARN("cuda: driver entry point " << name << " is not available");
        return false;
    }
    *out = reinterpret_cast<F>(fn);
    return true;
}

const DriverApi *Driver()
{
    static DriverApi api{};
    static bool ok = []() {
        if (DeviceCount() <= 0) {
            return false;
        }
        bool all = true;
        all &= Fetch("cuMemAddressReserve", &api.MemAddressReserve);
        all &= Fetch("cuMemAddressFree", &api.MemAddressFree);
        all &= Fetch("cuMemCreate", &api.MemCreate);
        all &= Fetch("cuMemRelease", &api.MemRelease);
        all &= Fetch("cuMemMap", &api.MemMap);
        all &= Fetch("cuMemUnmap", &api.MemUnmap);
        all &= Fetch("cuMemSetAccess", &api.MemSetAccess);
        all &= Fetch("cuMemExportToShareableHandle", &api.MemExportToShareableHandle);
        all &= Fetch("cuMemImportFromShareableHandle", &api.MemImportFromShareableHandle);
        all &= Fetch("cuMemGetAllocationGranularity", &api.MemGetAllocationGranularity);
        all &= Fetch("cuMemRetainAllocationHandle", &api.MemRetainAllocationHandle);
        all &= Fetch("cuMemGetAddressRange", &api.MemGetAddressRange);
        all &= Fetch("cuDeviceGet", &api.DeviceGet);
        all &= Fetch("cuDeviceGetAttribute", &api.DeviceGetAttribute);
        all &= Fetch("cuGetErrorString", &api.GetErrorString);
        all &= Fetch("cuDriverGetVersion", &api.DriverGetVersion);
        // Multicast (NVLS) is optional: absent on drivers without it.
        Fetch("cuMulticastCreate", &api.MulticastCreate);
        Fetch("cuMulticastAddDevice", &api.MulticastAddDevice);
        Fetch("cuMulticastBindMem", &api.MulticastBindMem);
        Fetch("cuMulticastUnbind", &api.MulticastUnbind);
        Fetch("cuMulticastGetGranularity", &api.MulticastGetGranularity);
        return all;
    }();
    return ok ? &api : nullptr;
}

std::string ErrStr(CUresult r)
{
    const DriverApi *d = Driver();
    const char *s = nullptr;
    if (d != nullptr && d->GetErrorString(r, &s) == CUDA_SUCCESS && s != nullptr) {
        return std::string(s) + " (CUresult " + std::to_string((int)r) + ")";
    }
    return "CUresult " + std::to_string((int)r);
}

std::string ErrStr(cudaError_t e) { return std::string(cudaGetErrorString(e)) + " (cudaError " + std::to_string((int)e) + ")"; }

int ProbeDevice(int device, DeviceCaps *out)
{
    const DriverApi *d = Driver();
    if (d == nullptr || device < 0 || device >= DeviceCount()) {
        return -1;
    }
    CUdevice dev;
    if (d->DeviceGet(&dev, device) != CUDA_SUCCESS) {
        return -1;
    }
    auto attr = [&](CUdevice_attribute a) {
        int v = 0;
        if (d->DeviceGetAttribute(&v, a, dev) != CUDA_SUCCESS) {
            v = 0;
        }
        return v;
    };
    out->device = device;
    out->vmm = attr(CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED) != 0;
    out->posixFdHandle = attr(CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED) != 0;
    out->fabricHandle = attr(CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_FABRIC_SUPPORTED) != 0;
    out->multicast = attr(CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED) != 0 && d->MulticastCreate != nullptr;
    out->hostNumaVmm = attr(CU_DEVICE_ATTRIBUTE_HOST_NUMA_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED) != 0;
    out->hostPtrForRegistered = attr(CU_DEVICE_ATTRIBUTE_CAN_USE_HOST_POINTER_FOR_REGISTERED_MEM) != 0;
    out->numaNode = attr(CU_DEVICE_ATTRIBUTE_HOST_NUMA_ID);
    out->smCount = attr(CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT);
    d->DriverGetVersion(&out->driverVersion);
    cudaRuntimeGetVersion(&out->runtimeVersion);
    return 0;
}

cudaStream_t ThreadStream(int device)
{
    thread_local std::unordered_map<int, cudaStream_t> streams;
    auto it = streams.find(device);
    if (it != streams.end()) {
        return it->second;
    }
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != device) {
        cudaSetDevice(device);
    }
    cudaStream_t s = nullptr;
    int lo = 0, hi = 0;
    cudaDeviceGetStreamPriorityRange(&lo, &hi);
    if (cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, hi) != cudaSuccess) {
        (void)cudaGetLastError();
        s = nullptr;  // fall back to the legacy default stream
    }
    streams[device] = s;
    return s;
}

}  // namespace cu
}  // namespace mf
