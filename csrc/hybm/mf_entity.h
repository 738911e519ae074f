// MemEntity: one pooled-memory object of one rank — owns the segments (HBM, DRAM, user-registered), the tag rules and
// the data operator, and implements reserve / alloc / export / import / map / copy on top of them.
// Reference: MemEntityDefault (src/hybm/csrc/entity/hybm_entity_default.cpp:88-114 init, :121-154 reserve, :172-264
// alloc/register, :303-449 export, :451-587 import, :650-714 mmap/remove, :737-809 copy/wait, :870-902 device meta,
// :995-1017 locating the owner rank of an address) and MemEntityFactory (entity/hybm_entity_factory.h:20-56).
#pragma once
#include <map>
#include <memory>
#include <mutex>
#include <shared_mutex>
#include <vector>

#include "mf_data_op.h"
#include "mf_hybm_types.h"
#include "mf_segment.h"
#include "mf_tag_info.h"
#include "../transport/mf_compose_transport.h"

namespace mf {
namespace hybm {

class MemEntity {
public:
    MemEntity(uint32_t id, const Options &opt);
    ~MemEntity();
    int Initialize();
    uint32_t Id() const { return id_; }
    const Options &Opt() const { return opt_; }

    // hints: 0 = first fit. On BM_ERROR the caller may retry with later hints (address negotiation between ranks).
    int ReserveMemorySpace(uint64_t hbmHint = 0, uint64_t dramHint = 0);
    int UnreserveMemorySpace();
    uint64_t MemoryPtr(uint32_t memType) const;
    uint64_t WindowSize(uint32_t memType) const;

    int AllocLocalMemory(uint64_t size, uint32_t memType, uint32_t flags, uint64_t *sliceHandle);
    int RegisterLocalMemory(uint64_t addr, uint64_t size, uint32_t flags, uint64_t *sliceHandle);
    int FreeLocalMemory(uint64_t sliceHandle);
    int SliceVa(uint64_t sliceHandle, uint64_t *va, uint64_t *size);

    int Export(uint64_t sliceHandle, uint32_t flags, ExchangeInfo *out);
    int Import(const ExchangeInfo *infos, uint32_t count, void **addresses, uint32_t flags);
    int Mmap();
    int Unmap();
    int RemoveImported(uint32_t rank);
    // Role of a peer (learned from its entity export, or told by the layer above). A SENDER maps the memory of RECEIVERs and of
    // PEERs only, a RECEIVER that of SENDERs and PEERs: slices of a rank with the same one-sided role are recorded nowhere and
    // never mapped (reference: the sender/receiver-only connections of transport/device/bipartite_ranks_qp_manager.cpp).
    void SetPeerRole(uint32_t rank, Role role);
    bool RolePermits(uint32_t rank);
    // The per-peer link table (role, host, state, slices) kept by the device transport of this entity.
    transport::PeerLinkManager &Links() { return devTp_->Links(); }
    // Cross-host mode only (FLAG_CROSS_HOST / MF_CROSS_HOST=1): the router over the device links and the TCP host transport
    // that serves this rank's pool memory to ranks on other hosts and reaches theirs. nullptr otherwise.
    std::shared_ptr<transport::ComposeTransport> Transport() const { return tp_; }
    // True if `rank` lives on another host (its memory was imported as remote).
    bool IsRemoteRank(uint32_t rank) { return devTp_->Links().StateOf(rank) == transport::LINK_REMOTE; }
    // One-sided copy between local memory and registered USER memory of a rank on another host (`remote` is an address of
    // that rank's own address space). write: local → remote. Device-side locals are staged. Blocking.
    int RemoteUserCopy(uint32_t rank, uint64_t local, uint64_t remote, uint64_t size, bool write, void *stream);
    int SetExtraContext(const void *ctx, uint32_t size);
    // Bit mask of DataOpType usable towards `rank`.
    uint32_t ReachTypes(uint32_t rank);

    int CopyData(const CopyParams &p, CopyDirection dir, void *stream, uint32_t flags);
    int BatchCopyData(const BatchCopyParams &p, CopyDirection dir, void *stream, uint32_t flags);
    int Wait();

    bool AddressInEntity(uint64_t addr, uint64_t len);
    // Owner rank of a pooled address; RANK_MAX if the address is not pooled in this entity.
    uint32_t RankOfAddress(uint64_t addr);
    PtrClass Classify(uint64_t addr, bool *deviceVisible);
    const DeviceMeta *DeviceMetaPtr() const { return devMeta_; }
    DeviceMeta HostMeta() const { return hostMeta_; }
    // Publishes the signal area and (optionally) the NVLS multicast alias to device code.
    int SetMetaExtras(uint64_t signalBase, uint64_t multicastBase)
    {
        hostMeta_.signalBase = signalBase;
        hostMeta_.multicastBase = multicastBase;
        return UpdateDeviceMeta();
    }
    // MF_DEBUG_* bits for device code (bit 0: kernels validate their heap arguments).
    int SetDebugFlags(uint64_t flags)
    {
        hostMeta_.debugFlags = flags;
        return UpdateDeviceMeta();
    }
    std::shared_ptr<MemSegment> Segment(uint32_t memType) const;
    std::shared_ptr<ComposeDataOp> DataOp() const { return dataOp_; }

private:
    int UpdateDeviceMeta();
    int ResolveDirection(uint64_t src, uint64_t dst, CopyDirection *dir, ExtOptions *opt);
    std::shared_ptr<MemSegment> SegmentOfSlice(uint64_t handle, MemSlice *slice);

    uint32_t id_;
    Options opt_;
    std::shared_ptr<MemSegment> hbm_;
    std::shared_ptr<MemSegment> dram_;
    std::shared_ptr<MemSegment> user_;
    std::shared_ptr<TagInfo> tags_;
    std::shared_ptr<ComposeDataOp> dataOp_;
    DeviceMeta hostMeta_{};
    DeviceMeta *devMeta_{nullptr};
    void *devCtx_{nullptr};
    // Copies hold this shared; unmapping a peer takes it exclusively, so a range is never pulled from under a copy.
    std::shared_mutex mapMu_;
    bool reserved_{false};
    // Pool memory of ranks on other hosts: known (so that addresses classify and bounds-check) but never mapped.
    struct RemoteSlice {
        uint32_t rank;
        uint64_t gva;
        uint64_t size;
        bool pooled;  // false: registered user memory, whose address is only meaningful on its owner (not in the VA manager)
    };
    int OpenCrossHost();
    int ServeSlice(std::string *blob);
    int ImportRemoteSlice(const SliceExport &e);
    int RemoteCopy(uint64_t src, uint64_t dst, uint64_t size, const ExtOptions &opt);
    bool IsDeviceAddress(uint64_t addr);
    std::shared_ptr<transport::DevicePeerTransport> devTp_;
    std::shared_ptr<transport::ComposeTransport> tp_;
    std::mutex remoteMu_;
    std::vector<RemoteSlice> remoteSlices_;
    transport::PrepareOptions pendingRanks_;  // records learned by Import, handed to the transport by Mmap
    std::mutex bounceMu_;
    void *bounce_{nullptr};  // pinned staging buffer for device-side locals of cross-host copies
};

class EntityFactory {
public:
    static EntityFactory &Instance();
    std::shared_ptr<MemEntity> Create(uint32_t id, const Options &opt, int *rc);
    std::shared_ptr<MemEntity> Find(uint32_t id);
    std::shared_ptr<MemEntity> FindByPtr(const void *p);
    void Destroy(uint32_t id);
    void DestroyAll();

private:
    std::mutex mu_;
    std::map<uint32_t, std::shared_ptr<MemEntity>> entities_;
};

// Library lifecycle (reference: hybm_init/hybm_uninit, src/hybm/csrc/hybm_entry.cpp:76-167): reference-counted, one
// device per process.
int HybmInit(int deviceId, uint64_t flags);
void HybmUninit();
bool HybmInited();
int HybmDevice();

}  // namespace hybm
}  // namespace mf
