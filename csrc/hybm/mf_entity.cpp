#include "mf_entity.h"

#include <cstdlib>
#include <cstring>
#include <pthread.h>
#include <unistd.h>

#include "../util/mf_log.h"
#include "../util/mf_tracer.h"
#include "mf_cuda.h"
#include "mf_fd_channel.h"

namespace mf {
namespace hybm {

// ---------------------------------------------------------------------------------------------- lifecycle

static std::mutex g_initMu;
static int g_initCount = 0;
static int g_device = -1;

static void AtForkChild()
{
    // The child owns no threads of the parent: forget the descriptor server and the init count so it can start afresh.
    FdChannel::Instance().ResetAfterFork();
    new (&g_initMu) std::mutex();
    g_initCount = 0;
    g_device = -1;
}

int HybmInit(int deviceId, uint64_t /*flags*/)
{
    std::lock_guard<std::mutex> g(g_initMu);
    if (g_initCount > 0) {
        MF_CHECK_RET(deviceId == g_device, BM_INVALID_PARAM,
                     "hybm: already initialised with device " << g_device << ", cannot switch to " << deviceId);
        g_initCount++;
        return BM_OK;
    }
    static bool forkHook = false;
    if (!forkHook) {
        pthread_atfork(nullptr, nullptr, AtForkChild);
        forkHook = true;
    }
    if (deviceId >= 0) {
        MF_CHECK_RET(cu::Available(), BM_NOT_SUPPORTED, "hybm: device " << deviceId << " requested but no CUDA device is visible");
        MF_CHECK_RET(deviceId < cu::DeviceCount(), BM_INVALID_PARAM, "hybm: device id " << deviceId << " out of range");
        cu::DeviceCaps caps;
        MF_CHECK_RET(cu::ProbeDevice(deviceId, &caps) == 0, BM_ERROR, "hybm: cannot probe device " << deviceId);
        MF_CHECK_RET(caps.vmm && caps.posixFdHandle, BM_NOT_SUPPORTED,
                     "hybm: device " << deviceId << " lacks virtual memory management or POSIX-fd handle export");
        MF_CUDA_CHECK_RET(cudaSetDevice(deviceId), BM_ERROR);
        MF_CUDA_CHECK_RET(cudaFree(nullptr), BM_ERROR);
        MF_INFO("hybm: device " << deviceId << " sms=" << caps.smCount << " driver=" << caps.driverVersion << " runtime=" << caps.runtimeVersion
                                << " multicast=" << caps.multicast << " fabric=" << caps.fabricHandle << " numa=" << caps.numaNode);
    }
    const char *trace = std::getenv("MF_TRACE_DIR");
    if (trace != nullptr) {
        Tracer::Instance().Init(trace);
    }
    g_device = deviceId;
    g_initCount = 1;
    return BM_OK;
}

void HybmUninit()
{
    std::lock_guard<std::mutex> g(g_initMu);
    if (g_initCount == 0) {
        return;
    }
    if (--g_initCount == 0) {
        EntityFactory::Instance().DestroyAll();
        g_device = -1;
    }
}

bool HybmInited()
{
    std::lock_guard<std::mutex> g(g_initMu);
    return g_initCount > 0;
}

int HybmDevice() { return g_device; }

// ---------------------------------------------------------------------------------------------- entity

MemEntity::MemEntity(uint32_t id, const Options &opt) : id_(id), opt_(opt) {}

MemEntity::~MemEntity()
{
    Unmap();
    UnreserveMemorySpace();
    if (devMeta_ != nullptr) {
        cudaFree(devMeta_);
    }
    if (devCtx_ != nullptr) {
        cudaFree(devCtx_);
    }
    if (tp_) {
        tp_->Host()->CloseDevice();
    }
    if (bounce_ != nullptr) {
        cudaFreeHost(bounce_);
    }
    VaManager::Instance().RemoveEntity(id_);
}

int MemEntity::Initialize()
{
    MF_CHECK_RET(opt_.rankCount > 0 && opt_.rankCount <= RANK_MAX && opt_.rankId < opt_.rankCount, BM_INVALID_PARAM,
                 "entity: invalid rank " << opt_.rankId << "/" << opt_.rankCount);
    MF_CHECK_RET(opt_.maxHBMSize % GRANULE == 0 && opt_.maxDRAMSize % GRANULE == 0, BM_INVALID_PARAM,
                 "entity: pool sizes must be multiples of 2 MiB");
    tags_ = std::make_shared<TagInfo>();
    int rc = tags_->Init(opt_.rankId, opt_.tag, opt_.tagOpInfo);
    if (rc != BM_OK) {
        return rc;
    }
    // Link table. Mapping and copying are done by this entity's own import / copy paths, so the device transport gets no
    // hooks: it is the record of what those paths did.
    devTp_ = std::make_shared<transport::DevicePeerTransport>();
    transport::Options to;
    to.rankId = opt_.rankId;
    to.rankCount = opt_.rankCount;
    to.role = opt_.role;
    devTp_->OpenDevice(to);
    devTp_->Links().SetSelf(opt_.rankId, opt_.role, HostIdentity());
    const char *cross = getenv("MF_CROSS_HOST");
    if ((opt_.flags & FLAG_CROSS_HOST) != 0 || (cross != nullptr && cross[0] == '1')) {
        rc = OpenCrossHost();
        if (rc != BM_OK) {
            return rc;
        }
    }
    SegmentOptions so;
    so.entityId = id_;
    so.rankId = opt_.rankId;
    so.rankCount = opt_.rankCount;
    so.devId = opt_.devId;
    so.flags = opt_.flags;
    so.role = opt_.role;
    if (opt_.scene == SCENE_TRANS) {
        so.type = SEG_USER_MEM;
        user_ = MemSegment::Create(so);
        MF_CHECK_RET(user_ != nullptr, BM_NEW_OBJECT_FAILED, "entity: cannot create the user-memory segment");
    } else if ((opt_.memType & MEM_TYPE_DEVICE) && opt_.maxHBMSize > 0) {
        so.type = SEG_DEVICE_VMM;
        so.windowSize = opt_.deviceVASpace != 0 ? opt_.deviceVASpace : opt_.maxHBMSize;
        hbm_ = MemSegment::Create(so);
        MF_CHECK_RET(hbm_ != nullptr, BM_NEW_OBJECT_FAILED, "entity: cannot create the HBM segment");
    }
    if ((opt_.memType & MEM_TYPE_HOST) && opt_.maxDRAMSize > 0) {
        so.type = SEG_HOST_SHM;
        so.windowSize = opt_.hostVASpace != 0 ? opt_.hostVASpace : opt_.maxDRAMSize;
        so.shmFd = opt_.dramShmFd;
        dram_ = MemSegment::Create(so);
        MF_CHECK_RET(dram_ != nullptr, BM_NEW_OBJECT_FAILED, "entity: cannot create the DRAM segment");
    }
    if (opt_.bmType == INIT_HOST || opt_.scene != SCENE_SHM) {
        dataOp_ = std::make_shared<ComposeDataOp>(opt_.devId, opt_.dataOpType, tags_);
        rc = dataOp_->Initialize();
        if (rc != BM_OK) {
            return rc;
        }
    } else {
        // Kernel-initiated entities still get a host data operator: it costs nothing and lets tests stage data.
        dataOp_ = std::make_shared<ComposeDataOp>(opt_.devId, OP_KERNEL_LDST | OP_COPY_ENGINE, tags_);
        dataOp_->Initialize();
    }
    hostMeta_.entityId = id_;
    hostMeta_.rankId = opt_.rankId;
    hostMeta_.rankCount = opt_.rankCount;
    if (opt_.devId >= 0 && cu::Available()) {
        MF_CUDA_CHECK_RET(cudaSetDevice(opt_.devId), BM_ERROR);
        MF_CUDA_CHECK_RET(cudaMalloc((void **)&devMeta_, sizeof(DeviceMeta)), BM_MALLOC_FAILED);
        MF_CUDA_CHECK_RET(cudaMalloc(&devCtx_, EXTRA_CONTEXT_MAX), BM_MALLOC_FAILED);
        hostMeta_.extraContextAddr = (uint64_t)devCtx_;
        rc = UpdateDeviceMeta();
    }
    return rc;
}

int MemEntity::OpenCrossHost()
{
    auto host = std::make_shared<transport::HostTcpTransport>();
    transport::Options to;
    to.rankId = opt_.rankId;
    to.rankCount = opt_.rankCount;
    to.role = opt_.role;
    // Address peers on other hosts use to reach this rank: MF_HOST_NIC ("ip" or "ip:port"), else the first non-loopback
    // IPv4 address of the host, else loopback. Port 0 = any free port.
    std::string nic;
    const char *env = getenv("MF_HOST_NIC");
    if (env != nullptr && env[0] != '\0') {
        nic = env;
        if (nic.find(':') == std::string::npos) {
            nic += ":0";
        }
    } else {
        auto ips = net::LocalIpv4List();
        nic = (ips.empty() ? std::string("127.0.0.1") : ips[0]) + ":0";
    }
    to.nic = nic;
    to.tls = net::GetStoreTlsOptions();  // the data links between hosts use the PKI configured for the control plane
    int rc = host->OpenDevice(to);
    MF_CHECK_RET(rc == BM_OK, rc, "entity: cannot open the host transport on " << nic);
    if (opt_.devId >= 0 && cu::Available()) {
        const int dev = opt_.devId;
        host->SetDeviceCopier([dev](void *dst, const void *src, size_t n) {
            if (cudaSetDevice(dev) != cudaSuccess || cudaMemcpy(dst, src, n, cudaMemcpyDefault) != cudaSuccess) {
                (void)cudaGetLastError();
                return -1;
            }
            return 0;
        });
    }
    tp_ = std::make_shared<transport::ComposeTransport>(devTp_, host);
    tp_->SetSelf(opt_.rankId);
    MF_INFO("entity " << id_ << ": cross-host mode, pool memory served at " << host->GetNic());
    return BM_OK;
}

// Registers the exported slice with the host transport and writes its address and key into the export blob.
int MemEntity::ServeSlice(std::string *blob)
{
    SliceExport e;
    if (!tp_ || blob->size() != sizeof(e)) {
        return BM_OK;
    }
    std::memcpy(&e, blob->data(), sizeof(e));
    if (e.size == 0) {
        return BM_OK;
    }
    auto host = tp_->Host();
    if (!host->QueryHasRegistered(e.gva, e.size)) {
        transport::MemoryRegion mr;
        mr.addr = e.gva;
        mr.size = e.size;
        mr.flags = e.memType == MEM_TYPE_DEVICE ? transport::MR_FLAG_HBM : transport::MR_FLAG_DRAM;
        int rc = host->RegisterMemoryRegion(mr);
        MF_CHECK_RET(rc == BM_OK, rc, "entity: cannot serve slice 0x" << std::hex << e.gva << std::dec << " over the host transport");
    }
    transport::MemoryKey k;
    MF_CHECK_RET(host->QueryMemoryKey(e.gva, &k) == BM_OK, BM_ERROR, "entity: no key for a slice just registered");
    std::memset(e.tpNic, 0, sizeof(e.tpNic));
    std::strncpy(e.tpNic, host->GetNic().c_str(), sizeof(e.tpNic) - 1);
    e.tpToken = k.token;
    e.tpAccess = k.access;
    e.tpFlags = k.flags;
    blob->assign((const char *)&e, sizeof(e));
    return BM_OK;
}

int MemEntity::ImportRemoteSlice(const SliceExport &e)
{
    MF_CHECK_RET(tp_ != nullptr, BM_NOT_SUPPORTED,
                 "entity: rank " << e.rank << " is on another host; cross-host mode (MF_CROSS_HOST=1) is off on this rank");
    MF_CHECK_RET(e.tpNic[0] != '\0' && e.tpToken != 0, BM_NOT_SUPPORTED,
                 "entity: rank " << e.rank << " is on another host and does not serve its memory (cross-host mode is off there)");
    const bool pooled = e.segType == SEG_DEVICE_VMM || e.segType == SEG_HOST_SHM;
    if (pooled) {
        auto seg = e.segType == SEG_DEVICE_VMM ? hbm_ : dram_;
        MF_CHECK_RET(seg != nullptr && seg->InWindow(e.gva, e.size) && seg->RankOf(e.gva) == e.rank, BM_INVALID_PARAM,
                     "entity: slice of rank " << e.rank << " does not lie in that rank's window here (the ranks reserved different windows)");
    }
    std::lock_guard<std::mutex> g(remoteMu_);
    for (const auto &r : remoteSlices_) {
        if (r.gva == e.gva && r.rank == e.rank) {
            return BM_OK;  // idempotent
        }
    }
    if (pooled) {
        // Pool addresses are global: the range is entered in the VA manager so that copies classify and bounds-check it.
        // Registered user memory is addressed in its owner's address space and is only ever named together with its rank.
        AllocatedRange a;
        a.gva = e.gva;
        a.size = e.size;
        a.memType = e.memType;
        a.ownerRank = e.rank;
        a.entityId = id_;
        a.imported = true;
        a.remote = true;
        VaManager::Instance().AddAllocated(a);
    }
    remoteSlices_.push_back(RemoteSlice{e.rank, e.gva, e.size, pooled});
    transport::RankInfo &info = pendingRanks_.ranks[e.rank];
    char nic[sizeof(e.tpNic) + 1] = {0};
    std::memcpy(nic, e.tpNic, sizeof(e.tpNic));
    info.nic = nic;
    info.sameHost = false;
    transport::MemoryKey k;
    k.token = e.tpToken;
    k.addr = e.gva;
    k.size = e.size;
    k.access = e.tpAccess;
    k.flags = e.tpFlags;
    info.keys.push_back(k);
    devTp_->Links().NoteSlice(e.rank, e.size, true);
    return BM_OK;
}

bool MemEntity::IsDeviceAddress(uint64_t addr)
{
    bool vis = false;
    PtrClass pc = Classify(addr, &vis);
    return pc == PC_GLOBAL_DEVICE || pc == PC_LOCAL_DEVICE;
}

// A copy whose pool side lives on another host: carried by the host transport. A host-side local goes straight over the
// wire; a device-side local is staged through a pinned bounce buffer; remote-to-remote is staged through it twice.
int MemEntity::RemoteCopy(uint64_t src, uint64_t dst, uint64_t size, const ExtOptions &opt)
{
    MF_CHECK_RET(tp_ != nullptr, BM_NOT_SUPPORTED, "copy: pool memory on another host needs cross-host mode");
    constexpr uint64_t kBounce = 8ull << 20;
    auto host = tp_->Host();
    NoteRemoteCopy(1);
    const bool srcDev = !opt.srcRemote && IsDeviceAddress(src), dstDev = !opt.dstRemote && IsDeviceAddress(dst);
    if (!(opt.srcRemote && opt.dstRemote) && !srcDev && !dstDev) {
        return opt.dstRemote ? host->WriteRemote(opt.dstRank, src, dst, size) : host->ReadRemote(opt.srcRank, dst, src, size);
    }
    std::lock_guard<std::mutex> g(bounceMu_);
    const bool cuda = opt_.devId >= 0 && cu::Available();
    if (bounce_ == nullptr) {
        if (cuda) {
            MF_CUDA_CHECK_RET(cudaMallocHost(&bounce_, kBounce), BM_MALLOC_FAILED);
        } else {
            bounce_ = nullptr;
        }
    }
    std::vector<char> plain;
    char *stage = (char *)bounce_;
    if (stage == nullptr) {
        plain.resize(kBounce);
        stage = plain.data();
    }
    if ((srcDev || dstDev) && opt.stream != nullptr) {
        MF_CUDA_CHECK_RET(cudaStreamSynchronize((cudaStream_t)opt.stream), BM_ERROR);  // what the stream wrote is what we read
    }
    for (uint64_t off = 0; off < size; off += kBounce) {
        const uint64_t n = std::min(kBounce, size - off);
        int rc = BM_OK;
        if (opt.srcRemote) {
            rc = host->ReadRemote(opt.srcRank, (uint64_t)stage, src + off, n);
        } else if (srcDev) {
            MF_CUDA_CHECK_RET(cudaMemcpy(stage, (const void *)(src + off), n, cudaMemcpyDefault), BM_ERROR);
        } else {
            std::memcpy(stage, (const void *)(src + off), n);
        }
        if (rc != BM_OK) {
            return rc;
        }
        if (opt.dstRemote) {
            rc = host->WriteRemote(opt.dstRank, (uint64_t)stage, dst + off, n);
        } else if (dstDev) {
            MF_CUDA_CHECK_RET(cudaMemcpy((void *)(dst + off), stage, n, cudaMemcpyDefault), BM_ERROR);
        } else {
            std::memcpy((void *)(dst + off), stage, n);
        }
        if (rc != BM_OK) {
            return rc;
        }
    }
    return BM_OK;
}

int MemEntity::RemoteUserCopy(uint32_t rank, uint64_t local, uint64_t remote, uint64_t size, bool write, void *stream)
{
    MF_CHECK_RET(tp_ != nullptr, BM_NOT_SUPPORTED, "copy: memory on another host needs cross-host mode");
    MF_CHECK_RET(local != 0 && remote != 0 && size != 0, BM_INVALID_PARAM, "copy: null address or empty copy");
    ExtOptions opt;
    opt.stream = stream;
    opt.srcRank = write ? opt_.rankId : rank;
    opt.dstRank = write ? rank : opt_.rankId;
    opt.srcRemote = !write;
    opt.dstRemote = write;
    return write ? RemoteCopy(local, remote, size, opt) : RemoteCopy(remote, local, size, opt);
}

int MemEntity::UpdateDeviceMeta()
{
    if (devMeta_ == nullptr) {
        return BM_OK;
    }
    MF_CUDA_CHECK_RET(cudaMemcpy(devMeta_, &hostMeta_, sizeof(DeviceMeta), cudaMemcpyHostToDevice), BM_ERROR);
    return BM_OK;
}

int MemEntity::ReserveMemorySpace(uint64_t hbmHint, uint64_t dramHint)
{
    MF_CHECK_RET(!reserved_, BM_ERROR, "entity: memory space already reserved");
    uint64_t base = 0;
    if (hbm_) {
        int rc = hbm_->ReserveMemorySpace(hbmHint, &base);
        if (rc != BM_OK) {
            return rc;
        }
        hostMeta_.hbmBase = base;
        hostMeta_.symmetricSize = hbm_->WindowSize();
    }
    if (dram_) {
        int rc = dram_->ReserveMemorySpace(dramHint, &base);
        if (rc != BM_OK) {
            if (hbm_) {
                hbm_->UnreserveMemorySpace();
            }
            return rc;
        }
        hostMeta_.dramBase = base;
        hostMeta_.dramWindowSize = dram_->WindowSize();
    }
    reserved_ = true;
    return UpdateDeviceMeta();
}

int MemEntity::UnreserveMemorySpace()
{
    if (!reserved_) {
        return BM_OK;
    }
    if (hbm_) {
        hbm_->Unmap();
        hbm_->UnreserveMemorySpace();
    }
    if (dram_) {
        dram_->Unmap();
        dram_->UnreserveMemorySpace();
    }
    reserved_ = false;
    return BM_OK;
}

std::shared_ptr<MemSegment> MemEntity::Segment(uint32_t memType) const
{
    if (memType == MEM_TYPE_DEVICE) {
        return hbm_ ? hbm_ : user_;
    }
    return dram_;
}

uint64_t MemEntity::MemoryPtr(uint32_t memType) const
{
    auto s = memType == MEM_TYPE_DEVICE ? hbm_ : dram_;
    return s ? s->Base() : 0;
}

uint64_t MemEntity::WindowSize(uint32_t memType) const
{
    auto s = memType == MEM_TYPE_DEVICE ? hbm_ : dram_;
    return s ? s->WindowSize() : 0;
}

// Slice handles are only unique per segment: bit 1 of the handle's low nibble tags user-registered slices so that the
// three segments never collide.
static constexpr uint64_t kUserSliceTag = 1ull << 1;

int MemEntity::AllocLocalMemory(uint64_t size, uint32_t memType, uint32_t flags, uint64_t *sliceHandle)
{
    auto seg = memType == MEM_TYPE_DEVICE ? hbm_ : (memType == MEM_TYPE_HOST ? dram_ : nullptr);
    MF_CHECK_RET(seg != nullptr, BM_INVALID_PARAM, "entity: no segment of memory type " << memType);
    MF_CHECK_RET(reserved_, BM_NOT_INITIALIZED, "entity: reserve the memory space first");
    MemSlice s;
    int rc = seg->AllocLocalMemory(size, flags | (opt_.flags & FLAG_CREATE_WITH_SHM), &s);
    if (rc != BM_OK) {
        return rc;
    }
    *sliceHandle = s.ToHandle();
    return BM_OK;
}

int MemEntity::RegisterLocalMemory(uint64_t addr, uint64_t size, uint32_t /*flags*/, uint64_t *sliceHandle)
{
    if (!user_) {
        SegmentOptions so;
        so.type = SEG_USER_MEM;
        so.entityId = id_;
        so.rankId = opt_.rankId;
        so.rankCount = opt_.rankCount;
        so.devId = opt_.devId;
        user_ = MemSegment::Create(so);
        MF_CHECK_RET(user_ != nullptr, BM_NEW_OBJECT_FAILED, "entity: cannot create the user-memory segment");
    }
    MemSlice s;
    int rc = user_->RegisterMemory(addr, size, &s);
    if (rc != BM_OK) {
        return rc;
    }
    *sliceHandle = s.ToHandle() | kUserSliceTag;
    return BM_OK;
}

std::shared_ptr<MemSegment> MemEntity::SegmentOfSlice(uint64_t handle, MemSlice *slice)
{
    bool userSlice = (handle & kUserSliceTag) != 0;
    uint16_t index = 0;
    uint32_t memType = 0;
    if (!MemSlice::Decode(handle & ~kUserSliceTag, &index, &memType)) {
        return nullptr;
    }
    std::shared_ptr<MemSegment> seg = userSlice ? user_ : (memType == MEM_TYPE_DEVICE ? hbm_ : dram_);
    if (!seg || !seg->FindSlice(index, slice)) {
        return nullptr;
    }
    return seg;
}

int MemEntity::FreeLocalMemory(uint64_t sliceHandle)
{
    MemSlice s;
    auto seg = SegmentOfSlice(sliceHandle, &s);
    MF_CHECK_RET(seg != nullptr, BM_INVALID_PARAM, "entity: invalid slice handle");
    if (tp_ && tp_->Host()->QueryHasRegistered(s.vAddress, 1)) {
        tp_->Host()->UnregisterMemoryRegion(s.vAddress);  // waits for requests that are touching the slice right now
    }
    return seg->ReleaseSlice(s);
}

int MemEntity::SliceVa(uint64_t sliceHandle, uint64_t *va, uint64_t *size)
{
    MemSlice s;
    auto seg = SegmentOfSlice(sliceHandle, &s);
    MF_CHECK_RET(seg != nullptr, BM_INVALID_PARAM, "entity: invalid slice handle");
    if (va != nullptr) {
        *va = s.vAddress;
    }
    if (size != nullptr) {
        *size = s.size;
    }
    return BM_OK;
}

int MemEntity::Export(uint64_t sliceHandle, uint32_t flags, ExchangeInfo *out)
{
    MF_CHECK_RET(out != nullptr, BM_INVALID_PARAM, "entity: null exchange info");
    std::memset(out, 0, sizeof(*out));
    if (sliceHandle == 0 || (flags & FLAG_EXPORT_ENTITY)) {
        EntityExport e{};
        e.magic = ENTITY_EXPORT_MAGIC;
        e.entityId = id_;
        e.rank = opt_.rankId;
        e.role = opt_.role;
        e.devId = opt_.devId;
        e.pid = (uint32_t)getpid();
        std::strncpy(e.tag, opt_.tag, sizeof(e.tag) - 1);
        std::strncpy(e.hostId, HostIdentity().c_str(), sizeof(e.hostId) - 1);
        std::memcpy(out->desc, &e, sizeof(e));
        out->descLen = sizeof(e);
        return BM_OK;
    }
    MemSlice s;
    auto seg = SegmentOfSlice(sliceHandle, &s);
    MF_CHECK_RET(seg != nullptr, BM_INVALID_PARAM, "entity: invalid slice handle");
    std::string blob;
    int rc = seg->Export(s, &blob);
    if (rc != BM_OK) {
        return rc;
    }
    rc = ServeSlice(&blob);
    if (rc != BM_OK) {
        return rc;
    }
    MF_CHECK_RET(blob.size() <= EXCHANGE_DESC_MAX, BM_ERROR, "entity: export blob too large");
    std::memcpy(out->desc, blob.data(), blob.size());
    out->descLen = (uint32_t)blob.size();
    return BM_OK;
}

void MemEntity::SetPeerRole(uint32_t rank, Role role) { devTp_->Links().NoteIdentity(rank, role, ""); }

bool MemEntity::RolePermits(uint32_t rank) { return devTp_->Links().Permits(rank); }

int MemEntity::Import(const ExchangeInfo *infos, uint32_t count, void **addresses, uint32_t /*flags*/)
{
    MF_CHECK_RET(infos != nullptr && count > 0, BM_INVALID_PARAM, "entity: nothing to import");
    for (uint32_t i = 0; i < count; i++) {
        const ExchangeInfo &x = infos[i];
        MF_CHECK_RET(x.descLen >= 4 && x.descLen <= EXCHANGE_DESC_MAX, BM_INVALID_PARAM, "entity: malformed exchange info #" << i);
        uint32_t magic;
        std::memcpy(&magic, x.desc, 4);
        if (magic == ENTITY_EXPORT_MAGIC) {
            MF_CHECK_RET(x.descLen == sizeof(EntityExport), BM_INVALID_PARAM, "entity: malformed entity info #" << i);
            EntityExport e;
            std::memcpy(&e, x.desc, sizeof(e));
            e.tag[sizeof(e.tag) - 1] = '\0';
            int rc = tags_->AddRankTag(e.rank, e.tag);
            if (rc != BM_OK) {
                return rc;
            }
            e.hostId[sizeof(e.hostId) - 1] = '\0';
            devTp_->Links().NoteIdentity(e.rank, (Role)e.role, e.hostId);
            if (addresses != nullptr) {
                addresses[i] = nullptr;
            }
            continue;
        }
        MF_CHECK_RET(magic == SLICE_EXPORT_MAGIC && x.descLen == sizeof(SliceExport), BM_INVALID_PARAM, "entity: unknown exchange info #" << i);
        SliceExport e;
        std::memcpy(&e, x.desc, sizeof(e));
        if (!RolePermits(e.rank)) {
            MF_INFO("entity: rank " << e.rank << " has the same one-sided role as this rank; its memory is not mapped");
            if (addresses != nullptr) {
                addresses[i] = nullptr;
            }
            continue;
        }
        e.hostId[sizeof(e.hostId) - 1] = '\0';
        if (e.rank != opt_.rankId && e.size != 0 && HostIdentity() != e.hostId) {
            // Another host: nothing to map. The slice is recorded and reached through the host transport.
            int rrc = ImportRemoteSlice(e);
            if (rrc != BM_OK) {
                return rrc;
            }
            if (addresses != nullptr) {
                addresses[i] = (void *)e.gva;
            }
            continue;
        }
        std::shared_ptr<MemSegment> seg;
        if (e.segType == SEG_DEVICE_VMM) {
            seg = hbm_;
        } else if (e.segType == SEG_HOST_SHM) {
            seg = dram_;
        } else if (e.segType == SEG_USER_MEM) {
            if (!user_) {
                uint64_t dummy = 0;
                // Importing a registered buffer needs a user segment even if this side registered nothing itself.
                SegmentOptions so;
                so.type = SEG_USER_MEM;
                so.entityId = id_;
                so.rankId = opt_.rankId;
                so.rankCount = opt_.rankCount;
                so.devId = opt_.devId;
                user_ = MemSegment::Create(so);
                (void)dummy;
            }
            seg = user_;
        }
        MF_CHECK_RET(seg != nullptr, BM_INVALID_PARAM, "entity: no local segment for imported slice type " << e.segType);
        std::vector<uint64_t> local;
        std::string blob((const char *)x.desc, x.descLen);
        int rc = seg->Import({blob}, &local);
        if (rc != BM_OK) {
            return rc;
        }
        if (e.rank != opt_.rankId) {
            devTp_->Links().NoteSlice(e.rank, e.size, false);
        }
        if (addresses != nullptr) {
            addresses[i] = local.empty() ? nullptr : (void *)local[0];
        }
    }
    return BM_OK;
}

int MemEntity::Mmap()
{
    std::unique_lock<std::shared_mutex> lk(mapMu_);
    for (auto &seg : {hbm_, dram_, user_}) {
        if (seg) {
            int rc = seg->Mmap();
            if (rc != BM_OK) {
                return rc;
            }
        }
    }
    devTp_->Links().NoteMapped();
    if (tp_) {
        // "Mapping" a rank on another host is opening the link to it (under the retry policy).
        transport::PrepareOptions fresh;
        {
            std::lock_guard<std::mutex> g(remoteMu_);
            fresh.ranks.swap(pendingRanks_.ranks);
        }
        if (!fresh.ranks.empty()) {
            for (auto &kv : fresh.ranks) {
                for (const auto &l : devTp_->Links().Snapshot()) {
                    if (l.rank == kv.first) {
                        kv.second.role = l.role;
                    }
                }
            }
            int rc = tp_->Host()->UpdateRankOptions(fresh);
            MF_CHECK_RET(rc == BM_OK, rc, "entity: cannot link to the ranks on other hosts");
        }
    }
    return BM_OK;
}

int MemEntity::Unmap()
{
    std::unique_lock<std::shared_mutex> lk(mapMu_);
    for (auto &seg : {hbm_, dram_, user_}) {
        if (seg) {
            seg->Unmap();
        }
    }
    return BM_OK;
}

int MemEntity::RemoveImported(uint32_t rank)
{
    std::unique_lock<std::shared_mutex> lk(mapMu_);
    for (auto &seg : {hbm_, dram_, user_}) {
        if (seg) {
            seg->RemoveImported({rank});
        }
    }
    {
        std::lock_guard<std::mutex> g(remoteMu_);
        for (auto it = remoteSlices_.begin(); it != remoteSlices_.end();) {
            if (it->rank == rank) {
                if (it->pooled) {
                    VaManager::Instance().RemoveAllocated(it->gva);
                }
                it = remoteSlices_.erase(it);
            } else {
                ++it;
            }
        }
        pendingRanks_.ranks.erase(rank);
    }
    if (tp_) {
        tp_->Host()->RemoveRanks({rank});
    }
    devTp_->Links().NoteRemoved(rank);
    tags_->RemoveRankTag(rank);
    return BM_OK;
}

int MemEntity::SetExtraContext(const void *ctx, uint32_t size)
{
    MF_CHECK_RET(ctx != nullptr && size > 0 && size <= EXTRA_CONTEXT_MAX, BM_INVALID_PARAM, "entity: extra context must be 1..65536 bytes");
    MF_CHECK_RET(devCtx_ != nullptr, BM_NOT_SUPPORTED, "entity: no device to hold the extra context");
    MF_CUDA_CHECK_RET(cudaMemcpy(devCtx_, ctx, size, cudaMemcpyHostToDevice), BM_ERROR);
    hostMeta_.extraContextSize = size;
    return UpdateDeviceMeta();
}

uint32_t MemEntity::ReachTypes(uint32_t rank)
{
    if (rank >= opt_.rankCount) {
        return 0;
    }
    uint32_t base = 0;
    if (hbm_ || user_) {
        base |= OP_KERNEL_LDST | OP_COPY_ENGINE;
    }
    if (dram_) {
        base |= OP_HOST_RDMA;
    }
    return tags_->AllowedOps(opt_.rankId, rank, base & (opt_.dataOpType | OP_HOST_RDMA | OP_KERNEL_LDST | OP_COPY_ENGINE));
}

bool MemEntity::AddressInEntity(uint64_t addr, uint64_t len)
{
    // Window arithmetic is not enough: a rank that left (or died) leaves a hole in the window. Only ranges that are
    // backed right now — local slices, mapped peers, registered user memory — count.
    AllocatedRange a;
    return VaManager::Instance().FindAllocated(addr, len, &a) && a.entityId == id_;
}

uint32_t MemEntity::RankOfAddress(uint64_t addr)
{
    if (hbm_ && hbm_->InWindow(addr, 1)) {
        return hbm_->RankOf(addr);
    }
    if (dram_ && dram_->InWindow(addr, 1)) {
        return dram_->RankOf(addr);
    }
    AllocatedRange a;
    if (VaManager::Instance().FindAllocated(addr, 1, &a) && a.entityId == id_) {
        return a.ownerRank;
    }
    return RANK_MAX;
}

PtrClass MemEntity::Classify(uint64_t addr, bool *deviceVisible)
{
    bool vis = true;
    PtrClass pc;
    if (hbm_ && hbm_->InWindow(addr, 1)) {
        pc = PC_GLOBAL_DEVICE;
    } else if (dram_ && dram_->InWindow(addr, 1)) {
        pc = PC_GLOBAL_HOST;
        vis = dram_->DeviceAccessible() && opt_.devId >= 0 && cu::Available();
    } else {
        AllocatedRange a;
        if (VaManager::Instance().FindAllocated(addr, 1, &a)) {
            pc = a.memType == MEM_TYPE_DEVICE ? PC_GLOBAL_DEVICE : PC_GLOBAL_HOST;
            if (pc == PC_GLOBAL_HOST) {
                vis = false;
            }
        } else {
            pc = PC_LOCAL_HOST;
            vis = false;
            if (opt_.devId >= 0 && cu::Available()) {
                cudaPointerAttributes attr{};
                if (cudaPointerGetAttributes(&attr, (const void *)addr) == cudaSuccess) {
                    if (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) {
                        pc = PC_LOCAL_DEVICE;
                        vis = true;
                    } else if (attr.type == cudaMemoryTypeHost) {
                        vis = true;  // pinned or registered: kernels can read it in place
                    }
                } else {
                    (void)cudaGetLastError();
                }
            }
        }
    }
    if (deviceVisible != nullptr) {
        *deviceVisible = vis;
    }
    return pc;
}

int MemEntity::ResolveDirection(uint64_t src, uint64_t dst, CopyDirection *dir, ExtOptions *opt)
{
    bool sv = true, dv = true;
    PtrClass sc = Classify(src, &sv), dc = Classify(dst, &dv);
    if (*dir == DIR_AUTO) {
        *dir = DirectionOf(sc, dc);
        MF_CHECK_RET(*dir != DIR_BUTT, BM_INVALID_PARAM,
                     "copy: neither " << VaManager::Instance().VaToInfo(src) << " nor " << VaManager::Instance().VaToInfo(dst) << " is in the pool");
    } else {
        // The caller's direction decides what the non-pool side is; the pool side(s) must really be in this entity.
        PtrClass wantS = SrcClassOf(*dir), wantD = DstClassOf(*dir);
        if (wantS == PC_GLOBAL_HOST || wantS == PC_GLOBAL_DEVICE) {
            MF_CHECK_RET(sc == wantS, BM_INVALID_PARAM, "copy: source " << VaManager::Instance().VaToInfo(src) << " is not " << DirectionName(*dir) << "'s pool side");
        } else if (sc == PC_GLOBAL_HOST || sc == PC_GLOBAL_DEVICE) {
            // A pool address used as a "local" buffer is fine: treat it by what it really is.
            wantS = sc;
        }
        if (wantD == PC_GLOBAL_HOST || wantD == PC_GLOBAL_DEVICE) {
            MF_CHECK_RET(dc == wantD, BM_INVALID_PARAM, "copy: destination " << VaManager::Instance().VaToInfo(dst) << " is not " << DirectionName(*dir) << "'s pool side");
        } else if (dc == PC_GLOBAL_HOST || dc == PC_GLOBAL_DEVICE) {
            wantD = dc;
        }
        CopyDirection real = DirectionOf(wantS, wantD);
        if (real != DIR_BUTT) {
            *dir = real;
        }
    }
    uint32_t sr = RankOfAddress(src), dr = RankOfAddress(dst);
    opt->srcRank = sr == RANK_MAX ? opt_.rankId : sr;
    opt->dstRank = dr == RANK_MAX ? opt_.rankId : dr;
    opt->srcDeviceVisible = sv;
    opt->dstDeviceVisible = dv;
    AllocatedRange ar;
    opt->srcRemote = sr != RANK_MAX && sr != opt_.rankId && VaManager::Instance().FindAllocated(src, 1, &ar) && ar.remote;
    opt->dstRemote = dr != RANK_MAX && dr != opt_.rankId && VaManager::Instance().FindAllocated(dst, 1, &ar) && ar.remote;
    return BM_OK;
}

int MemEntity::CopyData(const CopyParams &p, CopyDirection dir, void *stream, uint32_t flags)
{
    MF_CHECK_RET(p.src != nullptr && p.dest != nullptr, BM_INVALID_PARAM, "copy: null pointer");
    MF_CHECK_RET(dataOp_ != nullptr, BM_NOT_SUPPORTED, "copy: this entity has no host data operator");
    if (p.dataSize == 0) {
        return BM_OK;
    }
    std::shared_lock<std::shared_mutex> lk(mapMu_);
    ExtOptions opt;
    opt.stream = stream;
    opt.flags = flags;
    int rc = ResolveDirection((uint64_t)p.src, (uint64_t)p.dest, &dir, &opt);
    if (rc != BM_OK) {
        return rc;
    }
    if (SrcClassOf(dir) >= PC_GLOBAL_HOST) {
        MF_CHECK_RET(AddressInEntity((uint64_t)p.src, p.dataSize), BM_INVALID_PARAM,
                     "copy: " << p.dataSize << " bytes from " << VaManager::Instance().VaToInfo((uint64_t)p.src) << " leave the pool");
    }
    if (DstClassOf(dir) >= PC_GLOBAL_HOST) {
        MF_CHECK_RET(AddressInEntity((uint64_t)p.dest, p.dataSize), BM_INVALID_PARAM,
                     "copy: " << p.dataSize << " bytes to " << VaManager::Instance().VaToInfo((uint64_t)p.dest) << " leave the pool");
    }
    if (opt.srcRemote || opt.dstRemote) {
        return RemoteCopy((uint64_t)p.src, (uint64_t)p.dest, p.dataSize, opt);
    }
    return dataOp_->DataCopy(p, dir, opt);
}

int MemEntity::BatchCopyData(const BatchCopyParams &p, CopyDirection dir, void *stream, uint32_t flags)
{
    MF_CHECK_RET(p.sources != nullptr && p.destinations != nullptr && p.dataSizes != nullptr && p.batchSize > 0, BM_INVALID_PARAM,
                 "batch copy: empty or null parameters");
    MF_CHECK_RET(dataOp_ != nullptr, BM_NOT_SUPPORTED, "batch copy: this entity has no host data operator");
    std::shared_lock<std::shared_mutex> lk(mapMu_);
    // Every element is placed on its own: which rank owns each side, what the non-pool side really is (device memory,
    // pinned host memory a kernel can read, or pageable host memory only the copy engine or the CPU may touch), and whether
    // its pool side stays inside the pool. Elements are then grouped by (source rank, destination rank, direction,
    // visibility) and every group goes to the data operator as one sub-batch, so the tag rule of each rank pair applies and
    // an address a kernel cannot dereference never reaches a kernel.
    // Reference: hybm_entity_default.cpp:767-800 (grouping), :995-1017 (locating), hybm_compose_data_op.cpp:114-175 (use).
    struct Group {
        CopyDirection dir;
        ExtOptions opt;
        std::vector<uint32_t> idx;
    };
    std::vector<Group> groups;
    auto sameGroup = [](const Group &g, CopyDirection d, const ExtOptions &o) {
        return g.dir == d && g.opt.srcRank == o.srcRank && g.opt.dstRank == o.dstRank && g.opt.srcDeviceVisible == o.srcDeviceVisible &&
               g.opt.dstDeviceVisible == o.dstDeviceVisible && g.opt.srcRemote == o.srcRemote && g.opt.dstRemote == o.dstRemote;
    };
    size_t last = 0;
    for (uint32_t i = 0; i < p.batchSize; i++) {
        MF_CHECK_RET(p.sources[i] != nullptr && p.destinations[i] != nullptr, BM_INVALID_PARAM, "batch copy: null pointer at #" << i);
        ExtOptions opt;
        opt.stream = stream;
        opt.flags = flags;
        CopyDirection d = dir;
        int rc = ResolveDirection((uint64_t)p.sources[i], (uint64_t)p.destinations[i], &d, &opt);
        if (rc != BM_OK) {
            MF_ERROR("batch copy: element #" << i << " cannot be placed");
            return rc;
        }
        if (SrcClassOf(d) >= PC_GLOBAL_HOST) {
            MF_CHECK_RET(AddressInEntity((uint64_t)p.sources[i], p.dataSizes[i]), BM_INVALID_PARAM, "batch copy: source #" << i << " leaves the pool");
        }
        if (DstClassOf(d) >= PC_GLOBAL_HOST) {
            MF_CHECK_RET(AddressInEntity((uint64_t)p.destinations[i], p.dataSizes[i]), BM_INVALID_PARAM,
                         "batch copy: destination #" << i << " leaves the pool");
        }
        if (groups.empty() || !sameGroup(groups[last], d, opt)) {
            last = groups.size();
            for (size_t g = 0; g < groups.size(); g++) {
                if (sameGroup(groups[g], d, opt)) {
                    last = g;
                    break;
                }
            }
            if (last == groups.size()) {
                groups.push_back(Group{d, opt, {}});
            }
        }
        groups[last].idx.push_back(i);
    }
    NoteBatchGroups((uint32_t)groups.size());
    if (groups.size() == 1 && !groups[0].opt.srcRemote && !groups[0].opt.dstRemote) {
        return dataOp_->BatchDataCopy(p, groups[0].dir, groups[0].opt);  // the common case: the caller's arrays as they are
    }
    for (const Group &g : groups) {
        if (g.opt.srcRemote || g.opt.dstRemote) {
            // Host-side locals of one remote rank go out as one asynchronous batch and are waited for together; anything that
            // needs staging goes element by element.
            auto host = tp_ ? tp_->Host() : nullptr;
            MF_CHECK_RET(host != nullptr, BM_NOT_SUPPORTED, "batch copy: pool memory on another host needs cross-host mode");
            const bool oneSided = !(g.opt.srcRemote && g.opt.dstRemote);
            const uint32_t rank = g.opt.dstRemote ? g.opt.dstRank : g.opt.srcRank;
            bool queued = false;
            uint64_t queuedElems = 0;
            for (uint32_t i : g.idx) {
                const uint64_t src = (uint64_t)p.sources[i], dst = (uint64_t)p.destinations[i];
                const uint64_t local = g.opt.dstRemote ? src : dst;
                int rc;
                if (oneSided && !IsDeviceAddress(local)) {
                    rc = g.opt.dstRemote ? host->WriteRemoteAsync(rank, src, dst, p.dataSizes[i]) : host->ReadRemoteAsync(rank, dst, src, p.dataSizes[i]);
                    queued = true;
                    queuedElems++;
                } else {
                    rc = RemoteCopy(src, dst, p.dataSizes[i], g.opt);
                }
                if (rc != BM_OK) {
                    if (queued) {
                        host->Synchronize(rank);
                    }
                    return rc;
                }
            }
            if (queued) {
                NoteRemoteCopy(queuedElems);
                int rc = host->Synchronize(rank);
                if (rc != BM_OK) {
                    return rc;
                }
            }
            continue;
        }
        std::vector<void *> srcs(g.idx.size()), dsts(g.idx.size());
        std::vector<uint64_t> sizes(g.idx.size());
        for (size_t k = 0; k < g.idx.size(); k++) {
            srcs[k] = p.sources[g.idx[k]];
            dsts[k] = p.destinations[g.idx[k]];
            sizes[k] = p.dataSizes[g.idx[k]];
        }
        BatchCopyParams sub{srcs.data(), dsts.data(), sizes.data(), (uint32_t)g.idx.size()};
        int rc = dataOp_->BatchDataCopy(sub, g.dir, g.opt);
        if (rc != BM_OK) {
            return rc;
        }
    }
    return BM_OK;
}

int MemEntity::Wait()
{
    MF_CHECK_RET(dataOp_ != nullptr, BM_NOT_SUPPORTED, "wait: this entity has no host data operator");
    if (opt_.devId < 0 || !cu::Available()) {
        return BM_OK;
    }
    return dataOp_->Wait();
}

// ---------------------------------------------------------------------------------------------- factory

EntityFactory &EntityFactory::Instance()
{
    static EntityFactory *f = new EntityFactory();
    return *f;
}

std::shared_ptr<MemEntity> EntityFactory::Create(uint32_t id, const Options &opt, int *rc)
{
    std::lock_guard<std::mutex> g(mu_);
    if (id >= ENTITY_MAX || entities_.count(id)) {
        MF_ERROR("entity factory: id " << id << " is invalid or already in use");
        if (rc != nullptr) {
            *rc = BM_INVALID_PARAM;
        }
        return nullptr;
    }
    auto e = std::make_shared<MemEntity>(id, opt);
    int r = e->Initialize();
    if (rc != nullptr) {
        *rc = r;
    }
    if (r != BM_OK) {
        return nullptr;
    }
    entities_[id] = e;
    return e;
}

std::shared_ptr<MemEntity> EntityFactory::Find(uint32_t id)
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = entities_.find(id);
    return it == entities_.end() ? nullptr : it->second;
}

std::shared_ptr<MemEntity> EntityFactory::FindByPtr(const void *p)
{
    std::lock_guard<std::mutex> g(mu_);
    for (auto &kv : entities_) {
        if (kv.second.get() == p) {
            return kv.second;
        }
    }
    return nullptr;
}

void EntityFactory::Destroy(uint32_t id)
{
    std::shared_ptr<MemEntity> e;
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = entities_.find(id);
        if (it == entities_.end()) {
            return;
        }
        e = it->second;
        entities_.erase(it);
    }
}

void EntityFactory::DestroyAll()
{
    std::map<uint32_t, std::shared_ptr<MemEntity>> all;
    {
        std::lock_guard<std::mutex> g(mu_);
        all.swap(entities_);
    }
}

}  // namespace hybm
}  // namespace mf
