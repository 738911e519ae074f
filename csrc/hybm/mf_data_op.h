// Data operators: the engines that actually move bytes for xcopy, and the façade that picks one per call.
//
// Interface after the reference's DataOperator (src/hybm/csrc/data_operation/hybm_data_operator.h:22-101). Engines:
//   KernelDataOp      LD/ST copy kernels (mf_xcopy.cu) — every leg both of whose ends a GPU kernel can dereference: local
//                     HBM, peer HBM over NVLink, pinned host pool. Batches are one launch with a completion word.
//                     Role of HostDataOpSDMA + the copy_extend kernels (data_operation/host/hybm_data_op_sdma.cpp).
//   CopyEngineDataOp  cudaMemcpyAsync — legs that touch ordinary (unpinned) local host memory, and large host-pool legs.
//                     Unlike the reference's LH↔G path (hybm_data_op_sdma.cpp:171-221) no temporary device buffer is
//                     allocated per copy.
//   CpuDataOp         memcpy — host↔host legs and everything on CPU-only ranks (role of HostDataOpRDMA for the DRAM
//                     pool on one host, data_operation/host/hybm_data_op_host_rdma.cpp).
//   ComposeDataOp     orders the engines permitted by the (tag → op type → tag) rule for the two ranks and falls through
//                     to the next one on failure (data_operation/host/hybm_compose_data_op.cpp:84-175).
#pragma once
#include <atomic>
#include <memory>
#include <mutex>
#include <vector>

#include "mf_hybm_types.h"

namespace mf {
namespace hybm {

struct ExtOptions {
    uint32_t srcRank{0};
    uint32_t dstRank{0};
    void *stream{nullptr};  // user stream (cudaStream_t) or nullptr for the calling thread's own stream
    uint32_t flags{0};
    bool srcDeviceVisible{true};  // false: the source is pageable host memory a kernel cannot read
    bool dstDeviceVisible{true};
    bool srcRemote{false};  // the source is pool memory of a rank on another host (not mapped here)
    bool dstRemote{false};
};

class DataOperator {
public:
    virtual ~DataOperator() = default;
    virtual uint32_t Type() const = 0;  // one DataOpType bit
    virtual const char *Name() const = 0;
    virtual int Initialize() { return BM_OK; }
    // True if this engine can serve the direction with these options at all.
    virtual bool Supports(CopyDirection dir, const ExtOptions &opt) const = 0;
    virtual int DataCopy(const CopyParams &p, CopyDirection dir, const ExtOptions &opt) = 0;
    virtual int BatchDataCopy(const BatchCopyParams &p, CopyDirection dir, const ExtOptions &opt) = 0;
    // Waits for the calling thread's asynchronous copies.
    virtual int Wait() { return BM_OK; }
};

std::shared_ptr<DataOperator> MakeKernelDataOp(int device);
std::shared_ptr<DataOperator> MakeCopyEngineDataOp(int device);
std::shared_ptr<DataOperator> MakeCpuDataOp();

// Bounded wait for everything queued on `stream` (nullptr = calling thread's stream of `device`): polls an event for at
// most timeoutMs, then reports BM_TIMEOUT (reference: 1e6 × 1 µs polls → BM_TIMEOUT, src/hybm/csrc/ts_engine/hybm_stream.cpp:358-389).
int BoundedStreamSync(int device, void *stream, uint32_t timeoutMs);
uint32_t DefaultSyncTimeoutMs();

class TagInfo;

// Process-wide counters of which engine served how many calls and elements (observability, and the seam tests use to check
// that an address a kernel cannot read never reached the kernel engine).
struct DataOpStats {
    uint64_t kernelCalls, kernelElems, copyEngineCalls, copyEngineElems, cpuCalls, cpuElems, batchGroupsLast, remoteCalls, remoteElems;
};
DataOpStats GetDataOpStats();
void NoteBatchGroups(uint32_t groups);
void NoteRemoteCopy(uint64_t elems);  // copies carried by the host transport (pool memory on another host)

class ComposeDataOp : public DataOperator {
public:
    ComposeDataOp(int device, uint32_t allowedOps, std::shared_ptr<TagInfo> tags);
    uint32_t Type() const override { return 0; }
    const char *Name() const override { return "compose"; }
    int Initialize() override;
    bool Supports(CopyDirection, const ExtOptions &) const override { return true; }
    int DataCopy(const CopyParams &p, CopyDirection dir, const ExtOptions &opt) override;
    int BatchDataCopy(const BatchCopyParams &p, CopyDirection dir, const ExtOptions &opt) override;
    int Wait() override;
    // Engines in the order they would be tried for this call (exposed for tests).
    std::vector<std::shared_ptr<DataOperator>> Candidates(CopyDirection dir, const ExtOptions &opt, uint64_t bytes, bool batch) const;
    // Test seam: replace the engine list.
    void SetEngines(std::vector<std::shared_ptr<DataOperator>> engines) { engines_ = std::move(engines); }

private:
    int device_;
    uint32_t allowed_;
    std::shared_ptr<TagInfo> tags_;
    std::vector<std::shared_ptr<DataOperator>> engines_;
};

}  // namespace hybm
}  // namespace mf
