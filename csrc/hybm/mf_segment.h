// Memory segments: one object per (entity, memory type) that reserves the GVA window, backs the local rank's slice
// with physical memory, exports it, and maps the peers' slices at identical addresses.
//
// Mirrors the reference's MemSegment family (abstract class src/hybm/csrc/mm/hybm_mem_segment.h:41-162, factory
// hybm_mem_segment.cpp:59-100). Three implementations:
//   DeviceVmmSegment  HBM through the CUDA driver VMM API — the analogue of HybmVmmBasedSegment
//                     (mm/hybm_vmm_based_segment.cpp:39-75 reserve, :184-260 alloc, :330-380 export, :409-545 import+map)
//   HostShmSegment    host DRAM through memfd/user shm fd + mmap at the GVA, pinned for the GPU with cudaHostRegister
//                     when a GPU is present — covers HybmConnBasedSegment (mm/hybm_conn_based_segment.cpp:40-338) and the
//                     host-NUMA flavour of the VMM segment; it is also the whole data plane of CPU-only ranks
//   UserMemSegment    no pool: arbitrary user device buffers registered, exported and opened by peers under a local
//                     alias — HybmDevUserLegacySegment (mm/hybm_dev_user_legacy_segment.cpp:56-455)
// Layout inside a window: rank r owns [base + r*window, base + (r+1)*window); local slices are bump-allocated from the
// start of the owner's sub-window (hybm_vmm_based_segment.cpp:196-218). A rank may contribute zero bytes.
#pragma once
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "mf_hybm_types.h"
#include "mf_va_manager.h"

namespace mf {
namespace hybm {

enum SegmentType : uint32_t { SEG_DEVICE_VMM = 1, SEG_HOST_SHM = 2, SEG_USER_MEM = 3 };
enum HandleKind : uint32_t { HK_NONE = 0, HK_FD_CHANNEL = 1, HK_CUDA_IPC = 2, HK_FD_VMM_RETAINED = 3, HK_FD_HOST = 4 };

constexpr uint32_t SLICE_EXPORT_MAGIC = 0x4D465345u;   // "MFSE"
constexpr uint32_t ENTITY_EXPORT_MAGIC = 0x4D464545u;  // "MFEE"

#pragma pack(push, 8)
struct SliceExport {
    uint32_t magic;
    uint32_t segType;
    uint32_t memType;
    uint32_t rank;
    uint32_t entityId;
    uint32_t handleKind;
    uint32_t pid;
    int32_t devId;
    uint64_t gva;         // address the slice has in its owner (and, for pooled segments, in everybody)
    uint64_t size;
    uint64_t windowBase;  // owner's idea of the window base: importers verify it equals theirs
    uint64_t windowSize;
    uint64_t fdToken;
    uint64_t fileOffset;  // offset of the slice inside the shared file / allocation
    char fdName[48];
    char hostId[40];      // boot id: peers on another host cannot map and must not try
    uint8_t ipcHandle[64];
    // Filled by the entity when it serves its memory over the host transport (cross-host mode): where to ask and the
    // key of the region. Empty nic = not served over the wire.
    char tpNic[64];
    uint64_t tpToken;
    uint32_t tpAccess;
    uint32_t tpFlags;
};
struct EntityExport {
    uint32_t magic;
    uint32_t entityId;
    uint32_t rank;
    uint32_t role;
    int32_t devId;
    uint32_t pid;
    char tag[32];
    char hostId[40];
};
#pragma pack(pop)
static_assert(sizeof(SliceExport) <= EXCHANGE_DESC_MAX, "slice export fits the exchange blob");

std::string HostIdentity();  // kernel boot id (falls back to the host name); MF_HOST_IDENTITY overrides it (tests emulate several hosts)

struct SegmentOptions {
    SegmentType type{SEG_HOST_SHM};
    uint32_t entityId{0};
    uint32_t rankId{0};
    uint32_t rankCount{1};
    int32_t devId{-1};
    uint64_t windowSize{0};  // per-rank VA window
    uint32_t flags{0};
    int shmFd{-1};
    Role role{ROLE_PEER};
};

class MemSegment {
public:
    static std::shared_ptr<MemSegment> Create(const SegmentOptions &opt);
    virtual ~MemSegment() = default;

    // Reserves rankCount*windowSize of VA. hint 0 = first free window known to the VaManager. On success *base is the
    // window start. BM_ERROR if that exact range cannot be had (callers renegotiate with a later hint).
    virtual int ReserveMemorySpace(uint64_t hint, uint64_t *base) = 0;
    virtual int UnreserveMemorySpace() = 0;
    virtual int AllocLocalMemory(uint64_t size, uint32_t flags, MemSlice *out) = 0;
    virtual int RegisterMemory(uint64_t addr, uint64_t size, MemSlice *out) = 0;
    virtual int ReleaseSlice(const MemSlice &slice) = 0;
    virtual int Export(const MemSlice &slice, std::string *blob) = 0;
    // Records peers' slices (own rank's entries are skipped). Idempotent.
    virtual int Import(const std::vector<std::string> &blobs, std::vector<uint64_t> *localAddrs) = 0;
    // Maps everything imported and not yet mapped.
    virtual int Mmap() = 0;
    virtual int RemoveImported(const std::vector<uint32_t> &ranks) = 0;
    virtual int Unmap() = 0;
    // User-memory segments only: declares [addr, addr+size) as host memory backed by the shareable file `fd` (duplicated),
    // so that later registrations inside it can be exported to peers.
    virtual int AdoptHostBlock(uint64_t /*addr*/, uint64_t /*size*/, int /*fd*/) { return BM_NOT_SUPPORTED; }
    virtual int DropHostBlock(uint64_t /*addr*/) { return BM_NOT_SUPPORTED; }
    virtual uint32_t MemTypeBit() const = 0;
    // True if GPU kernels on the local device can dereference addresses of this segment.
    virtual bool DeviceAccessible() const = 0;

    // Bytes of address space actually reserved for the window: padded to whole GiB. The CUDA driver honours a requested
    // address only for reservations that do not share its internal VA blocks with neighbours, so windows are kept at
    // least 1 GiB long and 1 GiB aligned (address space is free; physical memory is only what the slices map).
    uint64_t ReservedBytes() const
    {
        const uint64_t need = opt_.windowSize * opt_.rankCount;
        return need <= WINDOW_ALIGN ? WINDOW_ALIGN : (need + WINDOW_ALIGN - 1) / WINDOW_ALIGN * WINDOW_ALIGN;
    }
    uint64_t Base() const { return base_; }
    uint64_t WindowSize() const { return opt_.windowSize; }
    uint64_t LocalAllocated() const { return localUsed_; }
    const SegmentOptions &Opt() const { return opt_; }
    bool InWindow(uint64_t addr, uint64_t len) const
    {
        return base_ != 0 && addr >= base_ && addr + len <= base_ + opt_.windowSize * opt_.rankCount && addr + len >= addr;
    }
    // Owner rank of a pooled address by arithmetic.
    uint32_t RankOf(uint64_t addr) const { return (uint32_t)((addr - base_) / opt_.windowSize); }
    bool FindSlice(uint16_t index, MemSlice *out);

protected:
    explicit MemSegment(const SegmentOptions &opt) : opt_(opt) {}
    SegmentOptions opt_;
    uint64_t base_{0};
    uint64_t localUsed_{0};
    uint16_t nextSlice_{1};
    std::mutex mu_;
    std::map<uint16_t, MemSlice> slices_;
};

}  // namespace hybm
}  // namespace mf
