// Share Memory (symmetric heap) API (include/mf/mf_shm.h).
//
// Reference flow reproduced: smem_shm_init → store (rank 0 serves) + hybm init with the device-meta flag
// (src/smem/csrc/smem_shm/smem_shm.cpp:294-327, smem_shm_entry_manager.cpp:24-56); smem_shm_create → static group +
// barrier, then the rollback-able steps create entity → reserve → alloc slice → exchange slice → exchange entity → map
// (smem_shm_entry.cpp:23-39 step table, :97-119 run/rollback, :142-286 steps); control collectives, reach info, atomic
// values and exit broadcast are thin calls into the group engine (smem_shm.cpp:88-384).
// New here: (1) the ranks agree on the heap address by all-gathering proposals (CUDA treats a requested VA as a hint);
// (2) a second tiny symmetric segment holds signal words for device-side barriers; (3) the heap is optionally aliased
// by an NVLS multicast mapping for multimem reductions.
#include <cstdlib>
#include <cstring>
#include <functional>
#include <map>
#include <mutex>

#include "../hybm/mf_cuda.h"
#include "../hybm/mf_fd_channel.h"
#include "../store/mf_store_client.h"
#include "../util/mf_log.h"
#include "mf/mf_shm.h"
#include "mf_api_internal.h"

using namespace mf;
using mf::api::MapGroupCode;
using mf::api::MapHybmCode;

namespace {

constexpr uint32_t kMaxShmId = 63;
constexpr uint32_t kSignalEntityBase = 256;
constexpr uint64_t kMaxSymmetric = 64ull << 30;

struct ShmGlobal {
    std::mutex mu;
    bool inited{false};
    mf_shm_config_t cfg{};
    std::string url;
    uint32_t worldSize{0};
    uint32_t rankId{0};
    int32_t deviceId{-1};
    store::StorePtr base;
    std::map<uint32_t, class ShmEntry *> entries;
};
ShmGlobal &G()
{
    static ShmGlobal *g = new ShmGlobal();
    return *g;
}

// All ranks of a static group end up with the same window addresses or with an error.
int NegotiateReserve(group::GroupEngine *grp, hybm::MemEntity *e, uint32_t rankSize)
{
    struct Proposal {
        uint64_t hbm, dram;
        uint32_t ok, pad;
    };
    uint64_t hintH = 0, hintD = 0;
    const uint64_t totalH = e->Opt().maxHBMSize * rankSize, totalD = e->Opt().maxDRAMSize * rankSize;
    for (int attempt = 0; attempt < 12; attempt++) {
        int rc = e->ReserveMemorySpace(hintH, hintD);
        Proposal mine{e->MemoryPtr(hybm::MEM_TYPE_DEVICE), e->MemoryPtr(hybm::MEM_TYPE_HOST), rc == hybm::BM_OK ? 1u : 0u, 0};
        std::vector<Proposal> all(rankSize);
        int grc = grp->GroupAllGather(&mine, sizeof(mine), all.data(), (uint32_t)(all.size() * sizeof(Proposal)));
        if (grc != group::GR_OK) {
            if (rc == hybm::BM_OK) {
                e->UnreserveMemorySpace();
            }
            return MapGroupCode(grc);
        }
        bool allOk = true, same = true;
        uint64_t maxH = hintH, maxD = hintD;
        for (auto &p : all) {
            allOk = allOk && p.ok;
            same = same && p.hbm == all[0].hbm && p.dram == all[0].dram;
            if (p.ok) {
                maxH = std::max(maxH, p.hbm);
                maxD = std::max(maxD, p.dram);
            }
        }
        if (allOk && same) {
            return MF_OK;
        }
        if (rc == hybm::BM_OK) {
            e->UnreserveMemorySpace();
        }
        // Everybody retries at the highest address anybody obtained; if somebody could not reserve at all, move past it.
        const uint64_t bump = allOk ? 0 : (1ull << 40);
        hintH = totalH ? (maxH ? maxH : hybm::GVA_WINDOW_BEGIN) + (allOk ? 0 : totalH + bump) : 0;
        hintD = totalD ? (maxD ? maxD : hybm::GVA_HOST_BEGIN) + (allOk ? 0 : totalD + bump) : 0;
        MF_INFO("shm: address negotiation round " << attempt << " did not converge, retrying at hbm 0x" << std::hex << hintH << " dram 0x" << hintD
                                                  << std::dec);
    }
    MF_ERROR("shm: the ranks could not agree on a common address window");
    return MF_ERROR;
}

class ShmEntry {
public:
    ShmEntry(uint32_t id, uint32_t rankSize, uint32_t rankId, uint64_t symSize, uint32_t opType, uint32_t flags)
        : id_(id), rankSize_(rankSize), rankId_(rankId), symSize_(symSize), opType_(opType), flags_(flags)
    {
    }
    ~ShmEntry() { Teardown(); }

    int Initialize(void **gva)
    {
        ShmGlobal &g = G();
        store_ = store::StoreFactory::PrefixOf(g.base, "SHM_(" + std::to_string(id_) + ")_");
        group::GroupOption go;
        go.rankSize = rankSize_;
        go.rank = rankId_;
        go.timeoutMs = g.cfg.controlOperationTimeout * 1000u;
        go.dynamic = false;
        group_ = group::GroupEngine::Create(store_, go);
        MF_CHECK_RET(group_ != nullptr, MF_NEW_OBJECT_FAILED, "shm: cannot create the group engine");
        int rc = MapGroupCode(group_->GroupBarrier());
        MF_CHECK_RET(rc == MF_OK, rc, "shm: initial barrier failed (" << rc << ")");

        // Rollback-able steps: each entry is (name, do, undo).
        struct Step {
            const char *name;
            std::function<int()> run;
            std::function<void()> undo;
        };
        std::vector<Step> steps = {
            {"create_entity", [&]() { return CreateEntities(); }, [&]() { DestroyEntities(); }},
            {"reserve", [&]() { return Reserve(); }, [&]() { Unreserve(); }},
            {"alloc_slice", [&]() { return Alloc(); }, []() {}},
            {"exchange_slice", [&]() { return Exchange(false); }, []() {}},
            {"exchange_entity", [&]() { return Exchange(true); }, []() {}},
            {"map", [&]() { return Map(); }, [&]() { Unmap(); }},
            {"publish_meta", [&]() { return PublishMeta(); }, []() {}},
        };
        for (size_t i = 0; i < steps.size(); i++) {
            rc = steps[i].run();
            if (rc != MF_OK) {
                MF_ERROR("shm create: step " << steps[i].name << " failed (" << rc << "), rolling back");
                for (size_t j = i + 1; j-- > 0;) {
                    steps[j].undo();
                }
                return rc;
            }
        }
        rc = MapGroupCode(group_->GroupBarrier());
        if (rc != MF_OK) {
            Teardown();
            return rc;
        }
        *gva = (void *)data_->MemoryPtr(hybm::MEM_TYPE_DEVICE);
        return MF_OK;
    }

    void Teardown()
    {
        if (data_ || signal_) {
            Unmap();
            DestroyEntities();
        }
        if (group_) {
            group_->Stop();
            group_.reset();
        }
    }

    hybm::MemEntity *Data() { return data_.get(); }
    hybm::MemEntity *Signal() { return signal_.get(); }
    group::GroupEngine *Group() { return group_.get(); }
    uint32_t RankSize() const { return rankSize_; }
    uint32_t RankId() const { return rankId_; }
    uint64_t Multicast() const { return mcVa_; }
    uint64_t NextEpoch(uint32_t ch) { return ch < MF_SHM_CHANNELS ? ++epochs_[ch] : 0; }
    int SetDebugFlags(uint64_t flags) { return data_ ? MapHybmCode(data_->SetDebugFlags(flags)) : MF_NOT_INITIALIZED; }
    std::function<void(int)> exitFn;

private:
    hybm::Options BaseOptions(uint64_t window) const
    {
        ShmGlobal &g = G();
        hybm::Options o;
        o.bmType = hybm::INIT_DEVICE_KERNEL;
        o.scene = hybm::SCENE_SHM;
        o.memType = hybm::MEM_TYPE_DEVICE;
        o.dataOpType = hybm::OP_KERNEL_LDST | hybm::OP_COPY_ENGINE;
        o.rankCount = rankSize_;
        o.rankId = rankId_;
        o.devId = g.deviceId;
        o.maxHBMSize = window;
        o.flags = flags_;
        return o;
    }

    int CreateEntities()
    {
        int rc = hybm::BM_OK;
        data_ = hybm::EntityFactory::Instance().Create(id_ * 2, BaseOptions(symSize_), &rc);
        if (!data_) {
            return MapHybmCode(rc);
        }
        signal_ = hybm::EntityFactory::Instance().Create(kSignalEntityBase + id_, BaseOptions(MF_SHM_SIGNAL_BYTES), &rc);
        if (!signal_) {
            return MapHybmCode(rc);
        }
        return MF_OK;
    }
    void DestroyEntities()
    {
        if (mcVa_ != 0) {
            ReleaseMulticast();
        }
        if (data_) {
            hybm::EntityFactory::Instance().Destroy(data_->Id());
            data_.reset();
        }
        if (signal_) {
            hybm::EntityFactory::Instance().Destroy(signal_->Id());
            signal_.reset();
        }
    }
    int Reserve()
    {
        int rc = NegotiateReserve(group_.get(), data_.get(), rankSize_);
        if (rc != MF_OK) {
            return rc;
        }
        return NegotiateReserve(group_.get(), signal_.get(), rankSize_);
    }
    void Unreserve()
    {
        if (data_) {
            data_->UnreserveMemorySpace();
        }
        if (signal_) {
            signal_->UnreserveMemorySpace();
        }
    }
    int Alloc()
    {
        int rc = data_->AllocLocalMemory(symSize_, hybm::MEM_TYPE_DEVICE, 0, &dataSlice_);
        if (rc != hybm::BM_OK) {
            return MapHybmCode(rc);
        }
        rc = signal_->AllocLocalMemory(MF_SHM_SIGNAL_BYTES, hybm::MEM_TYPE_DEVICE, 0, &signalSlice_);
        if (rc != hybm::BM_OK) {
            return MapHybmCode(rc);
        }
        // Signal words start at zero; epochs only ever grow.
        uint64_t mine = signal_->MemoryPtr(hybm::MEM_TYPE_DEVICE) + (uint64_t)rankId_ * MF_SHM_SIGNAL_BYTES;
        MF_CUDA_CHECK_RET(cudaMemset((void *)mine, 0, MF_SHM_SIGNAL_BYTES), MF_ERROR);
        MF_CUDA_CHECK_RET(cudaDeviceSynchronize(), MF_ERROR);
        return MF_OK;
    }
    int ExchangeOne(hybm::MemEntity *e, uint64_t slice, bool entityInfo)
    {
        hybm::ExchangeInfo mine{};
        int rc = e->Export(entityInfo ? 0 : slice, entityInfo ? hybm::FLAG_EXPORT_ENTITY : 0, &mine);
        if (rc != hybm::BM_OK) {
            return MapHybmCode(rc);
        }
        std::vector<hybm::ExchangeInfo> all(rankSize_);
        rc = group_->GroupAllGather(&mine, sizeof(mine), all.data(), (uint32_t)(all.size() * sizeof(hybm::ExchangeInfo)));
        if (rc != group::GR_OK) {
            return MapGroupCode(rc);
        }
        rc = e->Import(all.data(), rankSize_, nullptr, 0);
        return MapHybmCode(rc);
    }
    int Exchange(bool entityInfo)
    {
        int rc = ExchangeOne(data_.get(), dataSlice_, entityInfo);
        if (rc != MF_OK) {
            return rc;
        }
        rc = ExchangeOne(signal_.get(), signalSlice_, entityInfo);
        if (rc != MF_OK) {
            return rc;
        }
        return MapGroupCode(group_->GroupBarrier());
    }
    int Map()
    {
        int rc = data_->Mmap();
        if (rc != hybm::BM_OK) {
            return MapHybmCode(rc);
        }
        rc = signal_->Mmap();
        return MapHybmCode(rc);
    }
    void Unmap()
    {
        if (data_) {
            data_->Unmap();
        }
        if (signal_) {
            signal_->Unmap();
        }
    }
    int PublishMeta()
    {
        SetupMulticast();  // optional: failure only means multimem kernels are not offered
        uint64_t sig = signal_->MemoryPtr(hybm::MEM_TYPE_DEVICE);
        int rc = MapHybmCode(data_->SetMetaExtras(sig, mcVa_));
        const char *chk = std::getenv("MF_CHECK_BOUNDS");
        if (rc == MF_OK && chk != nullptr && chk[0] == '1') {
            rc = MapHybmCode(data_->SetDebugFlags(1));
        }
        return rc;
    }


    // NVLS: one multicast object spanning the heap; every rank binds its own slice at offset 0, so a multimem access at
    // mc + off touches heap offset `off` of every rank.
    void SetupMulticast();
    void ReleaseMulticast();

    uint32_t id_, rankSize_, rankId_;
    uint64_t symSize_;
    uint32_t opType_, flags_;
    store::StorePtr store_;
    std::shared_ptr<group::GroupEngine> group_;
    std::shared_ptr<hybm::MemEntity> data_, signal_;
    uint64_t dataSlice_{0}, signalSlice_{0};
    uint64_t mcVa_{0}, mcHandle_{0}, mcSize_{0};
    uint64_t epochs_[MF_SHM_CHANNELS]{};
};

void ShmEntry::SetupMulticast()
{
    const char *env = std::getenv("MF_NVLS");
    if (env != nullptr && env[0] == '0') {
        return;
    }
    if (rankSize_ < 2 || !(opType_ & MF_SHM_DATA_OP_RDMA)) {
        return;  // requested explicitly through the RDMA op-type bit
    }
    const cu::DriverApi *d = cu::Driver();
    ShmGlobal &g = G();
    cu::DeviceCaps caps;
    uint32_t can = d != nullptr && d->MulticastCreate != nullptr && cu::ProbeDevice(g.deviceId, &caps) == 0 && caps.multicast ? 1u : 0u;
    std::vector<uint32_t> cans(rankSize_);
    if (group_->GroupAllGather(&can, sizeof(can), cans.data(), (uint32_t)(cans.size() * 4)) != group::GR_OK) {
        return;
    }
    for (uint32_t c : cans) {
        if (!c) {
            MF_INFO("shm: NVLS multicast not available on every rank, multimem kernels disabled");
            return;
        }
    }
    CUmulticastObjectProp prop{};
    prop.numDevices = rankSize_;
    prop.size = symSize_;
    prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t gran = 0;
    if (d->MulticastGetGranularity(&gran, &prop, CU_MULTICAST_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || gran == 0) {
        return;
    }
    prop.size = (symSize_ + gran - 1) / gran * gran;
    struct Ticket {
        uint64_t token;
        char name[48];
        uint32_t ok, pad;
    };
    Ticket mine{};
    CUmemGenericAllocationHandle mc = 0;
    if (rankId_ == 0) {
        CUresult r = d->MulticastCreate(&mc, &prop);
        if (r == CUDA_SUCCESS) {
            int fd = -1;
            if (d->MemExportToShareableHandle(&fd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) == CUDA_SUCCESS) {
                mine.token = hybm::FdChannel::Instance().Publish(fd);
                ::close(fd);
                std::strncpy(mine.name, hybm::FdChannel::Instance().Name().c_str(), sizeof(mine.name) - 1);
                mine.ok = mine.token != 0;
            }
        } else {
            MF_INFO("shm: cuMulticastCreate failed: " << cu::ErrStr(r));
        }
    }
    std::vector<Ticket> all(rankSize_);
    if (group_->GroupAllGather(&mine, sizeof(mine), all.data(), (uint32_t)(all.size() * sizeof(Ticket))) != group::GR_OK || !all[0].ok) {
        if (mc != 0) {
            d->MemRelease(mc);
        }
        return;
    }
    uint32_t ok = 1;
    if (rankId_ != 0) {
        int fd = hybm::FdChannel::Fetch(all[0].name, all[0].token);
        ok = fd >= 0 && d->MemImportFromShareableHandle(&mc, (void *)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) == CUDA_SUCCESS;
        if (fd >= 0) {
            ::close(fd);
        }
    }
    CUdevice dev = 0;
    ok = ok && d->DeviceGet(&dev, g.deviceId) == CUDA_SUCCESS && d->MulticastAddDevice(mc, dev) == CUDA_SUCCESS;
    // Binding is only legal once every device was added: agree before and after.
    std::vector<uint32_t> oks(rankSize_);
    bool allOk = group_->GroupAllGather(&ok, 4, oks.data(), (uint32_t)(oks.size() * 4)) == group::GR_OK;
    for (uint32_t o : oks) {
        allOk = allOk && o;
    }
    if (allOk) {
        CUmemGenericAllocationHandle local = 0;
        uint64_t mineVa = data_->MemoryPtr(hybm::MEM_TYPE_DEVICE) + (uint64_t)rankId_ * symSize_;
        ok = d->MemRetainAllocationHandle(&local, (void *)mineVa) == CUDA_SUCCESS;
        if (ok) {
            ok = d->MulticastBindMem(mc, 0, local, 0, symSize_, 0) == CUDA_SUCCESS;
            d->MemRelease(local);
        }
        CUdeviceptr va = 0;
        if (ok) {
            ok = d->MemAddressReserve(&va, prop.size, gran, 0, 0) == CUDA_SUCCESS;
        }
        if (ok) {
            ok = d->MemMap(va, prop.size, 0, mc, 0) == CUDA_SUCCESS;
            if (ok) {
                CUmemAccessDesc acc{};
                acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
                acc.location.id = g.deviceId;
                acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
                ok = d->MemSetAccess(va, prop.size, &acc, 1) == CUDA_SUCCESS;
            }
            if (!ok) {
                d->MemAddressFree(va, prop.size);
            }
        }
        allOk = group_->GroupAllGather(&ok, 4, oks.data(), (uint32_t)(oks.size() * 4)) == group::GR_OK;
        for (uint32_t o : oks) {
            allOk = allOk && o;
        }
        if (allOk) {
            mcVa_ = (uint64_t)va;
            mcHandle_ = (uint64_t)mc;
            mcSize_ = prop.size;
            MF_INFO("shm: NVLS multicast alias of the heap at 0x" << std::hex << mcVa_ << std::dec);
        } else if (ok) {
            d->MemUnmap(va, prop.size);
            d->MemAddressFree(va, prop.size);
        }
    }
    if (rankId_ == 0 && mine.token != 0) {
        hybm::FdChannel::Instance().Unpublish(mine.token);
    }
    if (!allOk && mc != 0) {
        d->MemRelease(mc);
    }
}

void ShmEntry::ReleaseMulticast()
{
    const cu::DriverApi *d = cu::Driver();
    if (d == nullptr || mcVa_ == 0) {
        return;
    }
    cudaDeviceSynchronize();
    d->MemUnmap((CUdeviceptr)mcVa_, mcSize_);
    d->MemAddressFree((CUdeviceptr)mcVa_, mcSize_);
    CUdevice dev = 0;
    if (d->DeviceGet(&dev, G().deviceId) == CUDA_SUCCESS && d->MulticastUnbind != nullptr) {
        d->MulticastUnbind((CUmemGenericAllocationHandle)mcHandle_, dev, 0, symSize_);
    }
    d->MemRelease((CUmemGenericAllocationHandle)mcHandle_);
    mcVa_ = mcHandle_ = mcSize_ = 0;
}

ShmEntry *EntryOf(mf_shm_t h)
{
    ShmGlobal &g = G();
    std::lock_guard<std::mutex> lk(g.mu);
    for (auto &kv : g.entries) {
        if (kv.second == h) {
            return kv.second;
        }
    }
    MF_ERROR("shm: invalid handle");
    return nullptr;
}

}  // namespace

extern "C" int32_t mf_shm_config_init(mf_shm_config_t *c)
{
    MF_CHECK_RET(c != nullptr, MF_INVALID_PARAM, "shm config_init: null config");
    c->shmInitTimeout = 120;
    c->shmCreateTimeout = 120;
    c->controlOperationTimeout = 120;
    c->startConfigStoreServer = true;
    c->flags = 0;
    return MF_OK;
}

extern "C" int32_t mf_shm_init(const char *url, uint32_t worldSize, uint32_t rankId, uint16_t deviceId, mf_shm_config_t *config)
{
    MF_CHECK_RET(url != nullptr && config != nullptr, MF_INVALID_PARAM, "shm init: null argument");
    MF_CHECK_RET(worldSize > 0 && worldSize <= MF_WORLD_SIZE_MAX && rankId < worldSize, MF_INVALID_PARAM,
                 "shm init: rank " << rankId << " / world " << worldSize << " out of range");
    MF_CHECK_RET(config->shmInitTimeout > 0 && config->shmCreateTimeout > 0 && config->controlOperationTimeout > 0, MF_INVALID_PARAM,
                 "shm init: timeouts must be at least 1 s");
    MF_CHECK_RET(deviceId < 0x7FFF, MF_INVALID_PARAM, "shm init: the symmetric heap needs a GPU");
    ShmGlobal &g = G();
    std::lock_guard<std::mutex> lk(g.mu);
    if (g.inited) {
        MF_WARN("shm init: already initialised");
        return MF_OK;
    }
    int rc = MF_OK;
    bool serve = config->startConfigStoreServer && rankId == 0;
    g.base = mf::api::OpenStore(url, serve, serve, worldSize, (int32_t)rankId, config->shmInitTimeout, &rc);
    MF_CHECK_RET(g.base != nullptr, rc == MF_OK ? MF_ERROR : rc, "shm init: cannot reach the config store at " << url);
    int hrc = hybm::HybmInit((int)deviceId, hybm::INIT_FLAG_DEVICE_META);
    if (hrc != hybm::BM_OK) {
        g.base.reset();
        return MapHybmCode(hrc);
    }
    g.cfg = *config;
    g.url = url;
    g.worldSize = worldSize;
    g.rankId = rankId;
    g.deviceId = deviceId;
    g.inited = true;
    return MF_OK;
}

extern "C" void mf_shm_uninit(uint32_t /*flags*/)
{
    ShmGlobal &g = G();
    std::map<uint32_t, ShmEntry *> entries;
    {
        std::lock_guard<std::mutex> lk(g.mu);
        entries.swap(g.entries);
    }
    for (auto &kv : entries) {
        delete kv.second;
    }
    std::lock_guard<std::mutex> lk(g.mu);
    if (!g.inited) {
        return;
    }
    hybm::HybmUninit();
    net::Endpoint ep;
    g.base.reset();
    if (net::ParseUrl(g.url, &ep)) {
        store::StoreFactory::DestroyStore(ep);
    }
    g.inited = false;
}

extern "C" uint32_t mf_shm_query_support_data_operation(void)
{
    uint32_t ops = 0;
    if (cu::Available()) {
        ops |= MF_SHM_DATA_OP_MTE | MF_SHM_DATA_OP_SDMA;
        cu::DeviceCaps caps;
        int dev = hybm::HybmDevice() >= 0 ? hybm::HybmDevice() : 0;
        if (cu::ProbeDevice(dev, &caps) == 0 && caps.multicast) {
            ops |= MF_SHM_DATA_OP_RDMA;
        }
    }
    return ops;
}

extern "C" mf_shm_t mf_shm_create(uint32_t id, uint32_t rankSize, uint32_t rankId, uint64_t symmetricSize, mf_shm_data_op_type dataOpType,
                                  uint32_t flags, void **gva)
{
    ShmGlobal &g = G();
    if (gva == nullptr || id > kMaxShmId || rankSize == 0 || rankSize > MF_WORLD_SIZE_MAX || rankId >= rankSize || symmetricSize == 0 ||
        symmetricSize % hybm::GRANULE != 0 || symmetricSize > kMaxSymmetric) {
        MF_ERROR("shm create: invalid argument (id<=63, rank<size<=1024, size a non-zero multiple of 2 MiB up to 64 GiB)");
        return nullptr;
    }
    {
        std::lock_guard<std::mutex> lk(g.mu);
        if (!g.inited) {
            MF_ERROR("shm create: call mf_shm_init first");
            return nullptr;
        }
        if (g.entries.count(id)) {
            MF_ERROR("shm create: id " << id << " already exists");
            return nullptr;
        }
    }
    auto *e = new ShmEntry(id, rankSize, rankId, symmetricSize, (uint32_t)dataOpType, flags);
    int rc = e->Initialize(gva);
    if (rc != MF_OK) {
        MF_ERROR("shm create: failed (" << rc << ")");
        delete e;
        return nullptr;
    }
    std::lock_guard<std::mutex> lk(g.mu);
    g.entries[id] = e;
    return e;
}

extern "C" int32_t mf_shm_destroy(mf_shm_t handle, uint32_t /*flags*/)
{
    ShmGlobal &g = G();
    ShmEntry *e = nullptr;
    {
        std::lock_guard<std::mutex> lk(g.mu);
        for (auto it = g.entries.begin(); it != g.entries.end(); ++it) {
            if (it->second == handle) {
                e = it->second;
                g.entries.erase(it);
                break;
            }
        }
    }
    MF_CHECK_RET(e != nullptr, MF_INVALID_PARAM, "shm destroy: invalid handle");
    delete e;
    return MF_OK;
}

extern "C" int32_t mf_shm_set_extra_context(mf_shm_t handle, const void *context, uint32_t size)
{
    ShmEntry *e = EntryOf(handle);
    MF_CHECK_RET(e != nullptr, MF_INVALID_PARAM, "shm set_extra_context: invalid handle");
    MF_CHECK_RET(context != nullptr && size > 0 && size <= MF_SHM_EXTRA_CONTEXT_MAX, MF_INVALID_PARAM, "shm set_extra_context: size must be 1..65536");
    return MapHybmCode(e->Data()->SetExtraContext(context, size));
}

extern "C" uint32_t mf_shm_get_global_rank(mf_shm_t handle)
{
    ShmEntry *e = EntryOf(handle);
    return e == nullptr ? UINT32_MAX : e->RankId();
}
extern "C" uint32_t mf_shm_get_global_rank_size(mf_shm_t handle)
{
    ShmEntry *e = EntryOf(handle);
    return e == nullptr ? UINT32_MAX : e->RankSize();
}

extern "C" int32_t mf_shm_control_barrier(mf_shm_t handle)
{
    ShmEntry *e = EntryOf(handle);
    return e == nullptr ? MF_INVALID_PARAM : MapGroupCode(e->Group()->GroupBarrier());
}

extern "C" int32_t mf_shm_control_allgather(mf_shm_t handle, const char *sendBuf, uint32_t sendSize, char *recvBuf, uint32_t recvSize)
{
    ShmEntry *e = EntryOf(handle);
    MF_CHECK_RET(e != nullptr, MF_INVALID_PARAM, "shm allgather: invalid handle");
    MF_CHECK_RET(sendBuf != nullptr && recvBuf != nullptr && sendSize >= 1 && sendSize <= 65536 && recvSize == sendSize * e->RankSize(),
                 MF_INVALID_PARAM, "shm allgather: send size must be 1..65536 and recv size = send size × ranks");
    return MapGroupCode(e->Group()->GroupAllGather(sendBuf, sendSize, recvBuf, recvSize));
}

extern "C" int32_t mf_shm_subgroup_barrier(mf_shm_t handle, const char *key, uint32_t rankSize, uint32_t rankId)
{
    ShmEntry *e = EntryOf(handle);
    MF_CHECK_RET(e != nullptr && key != nullptr, MF_INVALID_PARAM, "shm subgroup_barrier: invalid argument");
    return MapGroupCode(e->Group()->SubGroupBarrier(key, rankSize, rankId));
}

extern "C" int32_t mf_shm_subgroup_allgather(mf_shm_t handle, const char *key, uint32_t rankSize, uint32_t rankId, const char *sendBuf,
                                             uint32_t sendSize, char *recvBuf, uint32_t recvSize)
{
    ShmEntry *e = EntryOf(handle);
    MF_CHECK_RET(e != nullptr && key != nullptr && sendBuf != nullptr && recvBuf != nullptr, MF_INVALID_PARAM, "shm subgroup_allgather: invalid argument");
    MF_CHECK_RET(sendSize >= 1 && sendSize <= 65536 && recvSize == sendSize * rankSize, MF_INVALID_PARAM,
                 "shm subgroup_allgather: send size must be 1..65536 and recv size = send size × ranks");
    return MapGroupCode(e->Group()->SubGroupAllGather(key, rankSize, rankId, sendBuf, sendSize, recvBuf, recvSize));
}

extern "C" int32_t mf_shm_topology_can_reach(mf_shm_t handle, uint32_t remoteRank, uint32_t *reachInfo)
{
    ShmEntry *e = EntryOf(handle);
    MF_CHECK_RET(e != nullptr && reachInfo != nullptr && remoteRank < e->RankSize(), MF_INVALID_PARAM, "shm can_reach: invalid argument");
    uint32_t ops = MF_SHM_DATA_OP_MTE | MF_SHM_DATA_OP_SDMA;  // every peer of the heap is mapped over NVLink
    if (e->Multicast() != 0) {
        ops |= MF_SHM_DATA_OP_RDMA;
    }
    *reachInfo = ops;
    return MF_OK;
}

extern "C" int32_t mf_shm_atomic_alloc_value(mf_shm_t handle, uint32_t limit, uint32_t *value)
{
    ShmEntry *e = EntryOf(handle);
    MF_CHECK_RET(e != nullptr && value != nullptr, MF_INVALID_PARAM, "shm atomic_alloc_value: invalid argument");
    return MapGroupCode(e->Group()->AllocNumber(limit, value));
}

extern "C" int32_t mf_shm_atomic_release_value(mf_shm_t handle, uint32_t value)
{
    ShmEntry *e = EntryOf(handle);
    MF_CHECK_RET(e != nullptr, MF_INVALID_PARAM, "shm atomic_release_value: invalid handle");
    return MapGroupCode(e->Group()->ReleaseNumber(value));
}

extern "C" int32_t mf_shm_register_exit(mf_shm_t handle, void (*exitFn)(int))
{
    ShmEntry *e = EntryOf(handle);
    MF_CHECK_RET(e != nullptr && exitFn != nullptr, MF_INVALID_PARAM, "shm register_exit: invalid argument");
    return MapGroupCode(e->Group()->RegisterExit([exitFn](int s) { exitFn(s); }));
}

extern "C" int32_t mf_shm_global_exit(mf_shm_t handle, int status)
{
    ShmEntry *e = EntryOf(handle);
    return e == nullptr ? MF_INVALID_PARAM : MapGroupCode(e->Group()->GroupBroadcastExit(status));
}

extern "C" const void *mf_shm_get_device_meta(mf_shm_t handle)
{
    ShmEntry *e = EntryOf(handle);
    return e == nullptr ? nullptr : e->Data()->DeviceMetaPtr();
}

extern "C" void *mf_shm_get_signal_base(mf_shm_t handle)
{
    ShmEntry *e = EntryOf(handle);
    return e == nullptr ? nullptr : (void *)e->Signal()->MemoryPtr(hybm::MEM_TYPE_DEVICE);
}

extern "C" void *mf_shm_get_multicast_ptr(mf_shm_t handle)
{
    ShmEntry *e = EntryOf(handle);
    return e == nullptr ? nullptr : (void *)e->Multicast();
}

extern "C" int32_t mf_shm_set_debug_flags(mf_shm_t handle, uint64_t flags)
{
    ShmEntry *e = EntryOf(handle);
    return e == nullptr ? MF_INVALID_PARAM : e->SetDebugFlags(flags);
}

extern "C" uint64_t mf_shm_next_epoch(mf_shm_t handle, uint32_t channel)
{
    ShmEntry *e = EntryOf(handle);
    return e == nullptr ? 0 : e->NextEpoch(channel);
}
