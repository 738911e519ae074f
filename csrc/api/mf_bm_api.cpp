// Big Memory API (include/mf/mf_bm.h).
//
// Reference call flow reproduced here: smem_bm_init → store + auto-ranking (src/smem/csrc/smem_bm/smem_bm.cpp:62-93,
// smem_bm_entry_manager.cpp:60-151), smem_bm_create2 → dynamic group + entity + reserve + alloc + export
// (smem_bm_entry.cpp:23-105), smem_bm_join → GroupJoin whose callback all-gathers rank ids, entity infos and slice
// infos, imports and maps them (smem_bm_entry.cpp:135-237), copy-type → direction resolution (smem_bm_entry.cpp:256-310).
// New here: the ranks agree on the GVA windows through a store key ("first creator proposes, the others adopt"),
// because CUDA treats a requested virtual address as a hint rather than a vendor-reserved range.
#include <cstring>
#include <map>
#include <mutex>

#include "../net/mf_tls.h"
#include "../hybm/mf_cuda.h"
#include "../store/mf_store_client.h"
#include "../util/mf_log.h"
#include "../util/mf_tracer.h"
#include "mf/mf_bm.h"
#include "mf_api_internal.h"

using namespace mf;
using mf::api::MapGroupCode;
using mf::api::MapHybmCode;

namespace {

constexpr uint64_t kMaxHbmPerRank = 64ull << 30;
constexpr uint64_t kMaxDramPerRank = 2048ull << 30;
constexpr uint32_t kMaxBmId = 63;
constexpr uint16_t kNoDevice = 0xFFFF;

struct BmGlobal {
    std::mutex mu;
    bool inited{false};
    mf_bm_config_t cfg{};
    std::string url;
    uint32_t worldSize{0};
    uint32_t rankId{0};
    int32_t deviceId{-1};
    store::StorePtr base;
    store::StorePtr store;  // prefixed "MF_BM_"
    std::map<uint32_t, class BmEntry *> entries;
};
BmGlobal &G()
{
    static BmGlobal *g = new BmGlobal();
    return *g;
}

class BmEntry {
public:
    BmEntry(uint32_t id, const mf_bm_create_option_t &opt) : id_(id), opt_(opt) {}
    ~BmEntry() { Destroy(); }

    int Initialize()
    {
        BmGlobal &g = G();
        store_ = store::StoreFactory::PrefixOf(g.store, "(" + std::to_string(id_) + ")_");
        group::GroupOption go;
        go.rankSize = g.worldSize;
        go.rank = g.rankId;
        go.timeoutMs = g.cfg.controlOperationTimeout * 1000u;
        go.dynamic = true;
        go.joinCb = [this](uint32_t r) { return JoinHandle(r); };
        go.leaveCb = [this](uint32_t r) { return LeaveHandle(r); };
        group_ = group::GroupEngine::Create(store_, go);
        MF_CHECK_RET(group_ != nullptr, MF_NEW_OBJECT_FAILED, "bm: cannot create the group engine");
        group_->StartListenEvent();

        hybm::Options ho;
        ho.bmType = hybm::INIT_HOST;
        ho.scene = hybm::SCENE_DEFAULT;
        ho.role = hybm::ROLE_PEER;
        ho.rankCount = g.worldSize;
        ho.rankId = g.rankId;
        ho.devId = g.deviceId;
        ho.memType = 0;
        if (opt_.maxHbmSize > 0 && g.deviceId >= 0) {
            ho.memType |= hybm::MEM_TYPE_DEVICE;
        }
        if (opt_.maxDramSize > 0) {
            ho.memType |= hybm::MEM_TYPE_HOST;
        }
        ho.maxHBMSize = opt_.maxHbmSize;
        ho.maxDRAMSize = opt_.maxDramSize;
        ho.dataOpType = 0;
        if (opt_.dataOpType & (MF_BM_DATA_OP_SDMA | MF_BM_DATA_OP_DEVICE_RDMA)) {
            ho.dataOpType |= hybm::OP_KERNEL_LDST | hybm::OP_COPY_ENGINE;
        }
        if (opt_.dataOpType & MF_BM_DATA_OP_HOST_RDMA) {
            ho.dataOpType |= hybm::OP_HOST_RDMA;
        }
        if (opt_.dataOpType & MF_BM_DATA_OP_HOST_TCP) {
            ho.dataOpType |= hybm::OP_HOST_TCP;
        }
        if (opt_.dataOpType & MF_BM_DATA_OP_HOST_URMA) {
            ho.dataOpType |= hybm::OP_HOST_URMA;
        }
        ho.flags = opt_.flags;
        ho.dramShmFd = opt_.dramShmFd;
        std::memcpy(ho.tag, opt_.tag, sizeof(ho.tag));
        std::memcpy(ho.tagOpInfo, opt_.tagOpInfo, sizeof(ho.tagOpInfo));
        ho.tag[sizeof(ho.tag) - 1] = '\0';
        ho.tagOpInfo[sizeof(ho.tagOpInfo) - 1] = '\0';
        int rc = hybm::BM_OK;
        entity_ = hybm::EntityFactory::Instance().Create(id_ * 2 + 1, ho, &rc);
        if (!entity_) {
            return MapHybmCode(rc);
        }
        rc = ReserveAgreed();
        if (rc != MF_OK) {
            return rc;
        }
        if (entity_->Segment(hybm::MEM_TYPE_DEVICE)) {
            rc = entity_->AllocLocalMemory(opt_.localHBMSize, hybm::MEM_TYPE_DEVICE, opt_.flags, &hbmSlice_);
            if (rc != hybm::BM_OK) {
                return MapHybmCode(rc);
            }
            rc = entity_->Export(hbmSlice_, 0, &hbmInfo_);
            if (rc != hybm::BM_OK) {
                return MapHybmCode(rc);
            }
        }
        if (entity_->Segment(hybm::MEM_TYPE_HOST)) {
            rc = entity_->AllocLocalMemory(opt_.localDRAMSize, hybm::MEM_TYPE_HOST, opt_.flags, &dramSlice_);
            if (rc != hybm::BM_OK) {
                return MapHybmCode(rc);
            }
            rc = entity_->Export(dramSlice_, 0, &dramInfo_);
            if (rc != hybm::BM_OK) {
                return MapHybmCode(rc);
            }
        }
        rc = entity_->Export(0, hybm::FLAG_EXPORT_ENTITY, &entityInfo_);
        return MapHybmCode(rc);
    }

    void Destroy()
    {
        if (group_) {
            if (group_->Joined()) {
                group_->GroupLeave();
            }
            group_->Stop();
            group_.reset();
        }
        if (entity_) {
            hybm::EntityFactory::Instance().Destroy(entity_->Id());
            entity_.reset();
        }
    }

    int Join()
    {
        int ret = 0;
        MF_TRACE_SCOPE(MF_TP(TM_BM, 0), "BM_JOIN", &ret);
        ret = MapGroupCode(group_->GroupJoin());
        return ret;
    }
    int Leave()
    {
        std::vector<uint32_t> peers = group_->Members();
        int rc = MapGroupCode(group_->GroupLeave());
        for (uint32_t r : peers) {
            if (r != entity_->Opt().rankId) {
                entity_->RemoveImported(r);  // the leaver drops its view of everybody else; its own slices stay
            }
        }
        return rc;
    }

    hybm::MemEntity *Entity() { return entity_.get(); }
    group::GroupEngine *Group() { return group_.get(); }
    const mf_bm_create_option_t &Opt() const { return opt_; }

    int ResolveType(mf_bm_copy_type t, uint64_t src, uint64_t dst, hybm::CopyDirection *dir)
    {
        using namespace hybm;
        if (t == MF_BM_COPY_AUTO) {
            *dir = DIR_AUTO;
            return MF_OK;
        }
        bool v;
        PtrClass sc = entity_->Classify(src, &v), dc = entity_->Classify(dst, &v);
        auto isGlobal = [](PtrClass c) { return c == PC_GLOBAL_DEVICE || c == PC_GLOBAL_HOST; };
        PtrClass s = sc, d = dc;
        switch (t) {
            case MF_BM_COPY_L2G:
            case MF_BM_COPY_L2GH:
                s = isGlobal(sc) ? sc : PC_LOCAL_DEVICE;
                MF_CHECK_RET(isGlobal(dc), MF_INVALID_PARAM, "bm copy: destination is not in the pool");
                break;
            case MF_BM_COPY_H2G:
            case MF_BM_COPY_H2GH:
                s = isGlobal(sc) ? sc : PC_LOCAL_HOST;
                MF_CHECK_RET(isGlobal(dc), MF_INVALID_PARAM, "bm copy: destination is not in the pool");
                break;
            case MF_BM_COPY_G2L:
            case MF_BM_COPY_GH2L:
                d = isGlobal(dc) ? dc : PC_LOCAL_DEVICE;
                MF_CHECK_RET(isGlobal(sc), MF_INVALID_PARAM, "bm copy: source is not in the pool");
                break;
            case MF_BM_COPY_G2H:
            case MF_BM_COPY_GH2H:
                d = isGlobal(dc) ? dc : PC_LOCAL_HOST;
                MF_CHECK_RET(isGlobal(sc), MF_INVALID_PARAM, "bm copy: source is not in the pool");
                break;
            case MF_BM_COPY_G2G:
                MF_CHECK_RET(isGlobal(sc) && isGlobal(dc), MF_INVALID_PARAM, "bm copy: G2G needs both addresses in the pool");
                break;
            default:
                MF_ERROR("bm copy: invalid copy type " << (int)t);
                return MF_INVALID_PARAM;
        }
        *dir = DirectionOf(s, d);
        MF_CHECK_RET(*dir != DIR_BUTT, MF_INVALID_PARAM, "bm copy: no pool address involved");
        return MF_OK;
    }

    std::map<uint64_t, uint64_t> userMem;  // registered local ranges
    std::mutex userMu;

private:
    // First creator publishes the window addresses it obtained; everybody else reserves exactly those.
    int ReserveAgreed()
    {
        const char *key = "GVA_BASES";
        for (int attempt = 0; attempt < 4; attempt++) {
            std::string cur;
            int rc = store_->Get(key, &cur, 0);
            if (rc == store::ST_OK && cur.size() == 16) {
                uint64_t bases[2];
                std::memcpy(bases, cur.data(), 16);
                rc = entity_->ReserveMemorySpace(bases[0], bases[1]);
                bool same = rc == hybm::BM_OK && (bases[0] == 0 || entity_->MemoryPtr(hybm::MEM_TYPE_DEVICE) == 0 ||
                                                  entity_->MemoryPtr(hybm::MEM_TYPE_DEVICE) == bases[0]) &&
                            (bases[1] == 0 || entity_->MemoryPtr(hybm::MEM_TYPE_HOST) == 0 || entity_->MemoryPtr(hybm::MEM_TYPE_HOST) == bases[1]);
                if (!same) {
                    if (rc == hybm::BM_OK) {
                        entity_->UnreserveMemorySpace();
                    }
                    MF_ERROR("bm: cannot reserve the pool's agreed address windows (hbm 0x" << std::hex << bases[0] << ", dram 0x" << bases[1]
                                                                                         << std::dec << ") in this process");
                    return MF_ERROR;
                }
                return MF_OK;
            }
            // Nobody proposed yet: find windows that work here, then try to publish them.
            uint64_t hint = 0;
            rc = hybm::BM_ERROR;
            for (int t = 0; t < 16 && rc != hybm::BM_OK; t++) {
                rc = entity_->ReserveMemorySpace(hint, hint == 0 ? 0 : hint + (1ull << 40));
                if (rc != hybm::BM_OK) {
                    hint = (hint == 0 ? hybm::GVA_WINDOW_BEGIN : hint) + (2ull << 40);
                }
            }
            MF_CHECK_RET(rc == hybm::BM_OK, MapHybmCode(rc), "bm: cannot reserve any address window");
            uint64_t mine[2] = {entity_->MemoryPtr(hybm::MEM_TYPE_DEVICE), entity_->MemoryPtr(hybm::MEM_TYPE_HOST)};
            std::string prev;
            rc = store_->Cas(key, "", std::string((const char *)mine, 16), &prev);
            MF_CHECK_RET(rc == store::ST_OK, MF_ERROR, "bm: store error while agreeing on addresses");
            if (prev.empty()) {
                return MF_OK;
            }
            if (prev.size() == 16 && std::memcmp(prev.data(), mine, 16) == 0) {
                return MF_OK;
            }
            entity_->UnreserveMemorySpace();  // lost the race: adopt the winner's windows on the next trip
        }
        return MF_ERROR;
    }

    int JoinHandle(uint32_t rank)
    {
        (void)rank;
        BmGlobal &g = G();
        uint32_t n = group_->RankSize();
        std::vector<uint32_t> ranks(n);
        uint32_t me = g.rankId;
        int rc = group_->GroupAllGather(&me, sizeof(me), ranks.data(), n * sizeof(uint32_t));
        if (rc != group::GR_OK) {
            return rc;
        }
        auto exchange = [&](const hybm::ExchangeInfo &mine) -> int {
            std::vector<hybm::ExchangeInfo> all(n);
            int r = group_->GroupAllGather(&mine, sizeof(mine), all.data(), (uint32_t)(n * sizeof(hybm::ExchangeInfo)));
            if (r != group::GR_OK) {
                return r;
            }
            for (auto &x : all) {
                if (x.descLen == 0) {
                    continue;  // that rank has no segment of this kind
                }
                uint32_t magic;
                std::memcpy(&magic, x.desc, 4);
                if (magic == hybm::SLICE_EXPORT_MAGIC) {
                    hybm::SliceExport se;
                    std::memcpy(&se, x.desc, sizeof(se));
                    if (!entity_->Segment(se.memType)) {
                        continue;  // e.g. a CPU-only rank cannot map HBM slices
                    }
                }
                r = entity_->Import(&x, 1, nullptr, 0);
                if (r != hybm::BM_OK) {
                    return r;
                }
            }
            return 0;
        };
        rc = exchange(entityInfo_);
        if (rc != 0) {
            return rc;
        }
        rc = exchange(hbmInfo_);
        if (rc != 0) {
            return rc;
        }
        rc = exchange(dramInfo_);
        if (rc != 0) {
            return rc;
        }
        rc = entity_->Mmap();
        if (rc != hybm::BM_OK) {
            return rc;
        }
        return group_->GroupBarrier();
    }

    int LeaveHandle(uint32_t rank) { return entity_->RemoveImported(rank); }

    uint32_t id_;
    mf_bm_create_option_t opt_;
    store::StorePtr store_;
    std::shared_ptr<group::GroupEngine> group_;
    std::shared_ptr<hybm::MemEntity> entity_;
    uint64_t hbmSlice_{0}, dramSlice_{0};
    hybm::ExchangeInfo entityInfo_{}, hbmInfo_{}, dramInfo_{};
};

BmEntry *EntryOf(mf_bm_t h)
{
    BmGlobal &g = G();
    std::lock_guard<std::mutex> lk(g.mu);
    for (auto &kv : g.entries) {
        if (kv.second == h) {
            return kv.second;
        }
    }
    MF_ERROR("bm: invalid handle");
    return nullptr;
}

}  // namespace

extern "C" int32_t mf_bm_config_init(mf_bm_config_t *c)
{
    if (c == nullptr) {
        MF_ERROR("bm config_init: null config");
        return MF_INVALID_PARAM;
    }
    std::memset(c, 0, sizeof(*c));
    c->initTimeout = 120;
    c->createTimeout = 120;
    c->controlOperationTimeout = 120;
    c->startConfigStoreServer = true;
    c->startConfigStoreOnly = false;
    c->dynamicWorldSize = false;
    c->unifiedAddressSpace = true;
    c->autoRanking = false;
    c->rankId = 0xFFFF;
    c->flags = 0;
    return MF_OK;
}

extern "C" int32_t mf_bm_init(const char *storeURL, uint32_t worldSize, uint16_t deviceId, const mf_bm_config_t *config)
{
    MF_CHECK_RET(storeURL != nullptr && config != nullptr, MF_INVALID_PARAM, "bm init: null argument");
    MF_CHECK_RET(worldSize > 0 && worldSize <= MF_WORLD_SIZE_MAX, MF_INVALID_PARAM, "bm init: world size " << worldSize << " out of range");
    MF_CHECK_RET(config->initTimeout > 0 && config->createTimeout > 0 && config->controlOperationTimeout > 0, MF_INVALID_PARAM,
                 "bm init: timeouts must be at least 1 s");
    MF_CHECK_RET(config->unifiedAddressSpace, MF_INVALID_PARAM, "bm init: unifiedAddressSpace must be true");
    MF_CHECK_RET(config->autoRanking || config->rankId < worldSize, MF_INVALID_PARAM, "bm init: rank id " << config->rankId << " out of range");
    BmGlobal &g = G();
    std::lock_guard<std::mutex> lk(g.mu);
    if (g.inited) {
        MF_WARN("bm init: already initialised");
        return MF_OK;
    }
    int rc = MF_OK;
    if (config->storeTlsConfig.tlsEnable) {
        // The struct form of the store's TLS options; it applies to the stores created below.
        auto text = [](const char *p) { return std::string(p, strnlen(p, MF_TLS_PATH_SIZE)); };
        const mf_tls_config &t = config->storeTlsConfig;
        net::TlsConfigPaths paths;
        paths.enable = true;
        paths.caPath = text(t.caPath);
        paths.crlPath = text(t.crlPath);
        paths.certPath = text(t.certPath);
        paths.keyPath = text(t.keyPath);
        paths.keyPassPath = text(t.keyPassPath);
        paths.packagePath = text(t.packagePath);
        paths.decrypterLibPath = text(t.decrypterLibPath);
        net::TlsOptions opt;
        std::string why;
        MF_CHECK_RET(net::TlsOptionsFromPaths(paths, &opt, &why), MF_INVALID_PARAM, "bm init: " << why);
        net::SetStoreTlsOptions(opt);
    }
    if (config->startConfigStoreOnly) {
        g.base = mf::api::OpenStore(storeURL, true, true, worldSize, -1, config->initTimeout, &rc);
        return g.base ? MF_OK : rc;
    }
    if (config->autoRanking) {
        bool tryServe = config->startConfigStoreServer && mf::api::UrlIsLocal(storeURL);
        g.base = mf::api::OpenStore(storeURL, tryServe, false, worldSize, -1, config->initTimeout, &rc);
    } else {
        bool serve = config->startConfigStoreServer && config->rankId == 0;
        g.base = mf::api::OpenStore(storeURL, serve, serve, worldSize, config->rankId, config->initTimeout, &rc);
    }
    MF_CHECK_RET(g.base != nullptr, rc == MF_OK ? MF_ERROR : rc, "bm init: cannot reach the config store at " << storeURL);
    g.store = store::StoreFactory::PrefixOf(g.base, "MF_BM_");
    if (config->autoRanking) {
        std::string v;
        int src = g.store->Get(std::string(store::AUTO_RANKING_PREFIX) + "bm", &v, (int64_t)config->initTimeout * 1000);
        MF_CHECK_RET(src == store::ST_OK, MF_ERROR, "bm init: auto-ranking failed (" << src << ")");
        g.rankId = (uint32_t)std::strtoul(v.c_str(), nullptr, 10);
        MF_CHECK_RET(g.rankId < worldSize, MF_ERROR, "bm init: store handed out rank " << g.rankId << " beyond the world size");
    } else {
        g.rankId = config->rankId;
    }
    g.deviceId = deviceId >= 0x7FFF ? -1 : (int32_t)deviceId;
    int hrc = hybm::HybmInit(g.deviceId, 0);
    if (hrc != hybm::BM_OK) {
        net::Endpoint ep;
        if (net::ParseUrl(storeURL, &ep)) {
            store::StoreFactory::DestroyStore(ep);
        }
        g.base.reset();
        g.store.reset();
        return MapHybmCode(hrc);
    }
    g.cfg = *config;
    g.url = storeURL;
    g.worldSize = worldSize;
    g.inited = true;
    MF_INFO("bm init: rank " << g.rankId << "/" << worldSize << " device " << g.deviceId << " store " << storeURL);
    return MF_OK;
}

extern "C" void mf_bm_uninit(uint32_t /*flags*/)
{
    BmGlobal &g = G();
    std::map<uint32_t, BmEntry *> entries;
    {
        std::lock_guard<std::mutex> lk(g.mu);
        entries.swap(g.entries);
    }
    for (auto &kv : entries) {
        delete kv.second;
    }
    std::lock_guard<std::mutex> lk(g.mu);
    if (g.inited) {
        hybm::HybmUninit();
    }
    net::Endpoint ep;
    if (!g.url.empty() && net::ParseUrl(g.url, &ep)) {
        g.store.reset();
        g.base.reset();
        store::StoreFactory::DestroyStore(ep);
    }
    g.inited = false;
    g.url.clear();
}

extern "C" uint32_t mf_bm_get_rank_id(void)
{
    BmGlobal &g = G();
    std::lock_guard<std::mutex> lk(g.mu);
    return g.inited ? g.rankId : UINT32_MAX;
}

extern "C" mf_bm_t mf_bm_create2(uint32_t id, const mf_bm_create_option_t *option)
{
    BmGlobal &g = G();
    if (option == nullptr || id > kMaxBmId) {
        MF_ERROR("bm create: invalid id " << id << " or null option");
        return nullptr;
    }
    {
        std::lock_guard<std::mutex> lk(g.mu);
        if (!g.inited) {
            MF_ERROR("bm create: call mf_bm_init first");
            return nullptr;
        }
        if (g.entries.count(id)) {
            MF_ERROR("bm create: id " << id << " already exists");
            return nullptr;
        }
    }
    const mf_bm_create_option_t &o = *option;
    if (o.maxHbmSize > kMaxHbmPerRank || o.maxDramSize > kMaxDramPerRank || o.localHBMSize > o.maxHbmSize || o.localDRAMSize > o.maxDramSize ||
        (o.maxHbmSize | o.maxDramSize | o.localHBMSize | o.localDRAMSize) % hybm::GRANULE != 0 || (o.maxHbmSize == 0 && o.maxDramSize == 0)) {
        MF_ERROR("bm create: sizes must be multiples of 2 MiB, local <= max, HBM <= 64 GiB and DRAM <= 2 TiB per rank, and not all zero");
        return nullptr;
    }
    if (o.maxHbmSize > 0 && g.deviceId < 0 && o.localHBMSize > 0) {
        MF_ERROR("bm create: a CPU-only rank cannot contribute HBM");
        return nullptr;
    }
    auto *e = new BmEntry(id, o);
    int rc = e->Initialize();
    if (rc != MF_OK) {
        MF_ERROR("bm create: initialisation failed (" << rc << ")");
        delete e;
        return nullptr;
    }
    std::lock_guard<std::mutex> lk(g.mu);
    g.entries[id] = e;
    return e;
}

extern "C" mf_bm_t mf_bm_create(uint32_t id, uint32_t /*memberSize*/, mf_bm_data_op_type dataOpType, uint64_t localDRAMSize,
                                uint64_t localHBMSize, uint32_t flags)
{
    mf_bm_create_option_t o;
    std::memset(&o, 0, sizeof(o));
    o.maxDramSize = o.localDRAMSize = localDRAMSize;
    o.maxHbmSize = o.localHBMSize = localHBMSize;
    o.dataOpType = dataOpType;
    o.flags = flags;
    o.dramShmFd = -1;
    return mf_bm_create2(id, &o);
}

extern "C" void mf_bm_destroy(mf_bm_t handle)
{
    BmGlobal &g = G();
    BmEntry *e = nullptr;
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
    delete e;
}

extern "C" int32_t mf_bm_join(mf_bm_t handle, uint32_t /*flags*/)
{
    BmEntry *e = EntryOf(handle);
    return e == nullptr ? MF_INVALID_PARAM : e->Join();
}

extern "C" int32_t mf_bm_leave(mf_bm_t handle, uint32_t /*flags*/)
{
    BmEntry *e = EntryOf(handle);
    if (e == nullptr) {
        return MF_INVALID_PARAM;
    }
    return e->Leave();
}

extern "C" uint64_t mf_bm_get_local_mem_size_by_mem_type(mf_bm_t handle, mf_bm_mem_type memType)
{
    BmEntry *e = EntryOf(handle);
    if (e == nullptr) {
        return 0;
    }
    if (memType == MF_MEM_TYPE_DEVICE) {
        return e->Entity()->Segment(hybm::MEM_TYPE_DEVICE) ? e->Opt().localHBMSize : 0;
    }
    if (memType == MF_MEM_TYPE_HOST) {
        return e->Entity()->Segment(hybm::MEM_TYPE_HOST) ? e->Opt().localDRAMSize : 0;
    }
    return 0;
}

extern "C" void *mf_bm_ptr_by_mem_type(mf_bm_t handle, mf_bm_mem_type memType, uint16_t peerRankId)
{
    BmEntry *e = EntryOf(handle);
    if (e == nullptr) {
        return nullptr;
    }
    uint32_t mt = memType == MF_MEM_TYPE_DEVICE ? (uint32_t)hybm::MEM_TYPE_DEVICE : (memType == MF_MEM_TYPE_HOST ? (uint32_t)hybm::MEM_TYPE_HOST : 0u);
    if (mt == 0 || peerRankId >= e->Entity()->Opt().rankCount) {
        MF_ERROR("bm ptr: invalid memory type " << (int)memType << " or rank " << peerRankId);
        return nullptr;
    }
    uint64_t base = e->Entity()->MemoryPtr(mt);
    if (base == 0) {
        MF_ERROR("bm ptr: the pool has no memory of type " << (int)memType);
        return nullptr;
    }
    return (void *)(base + (uint64_t)peerRankId * e->Entity()->WindowSize(mt));
}

static int32_t CopyImpl(mf_bm_t handle, mf_copy_params *params, mf_bm_copy_type t, void *stream, uint32_t flags)
{
    BmEntry *e = EntryOf(handle);
    MF_CHECK_RET(e != nullptr && params != nullptr, MF_INVALID_PARAM, "bm copy: null argument");
    MF_CHECK_RET(params->src != nullptr && params->dest != nullptr, MF_INVALID_PARAM, "bm copy: null pointer");
    hybm::CopyDirection dir;
    int rc = e->ResolveType(t, (uint64_t)params->src, (uint64_t)params->dest, &dir);
    if (rc != MF_OK) {
        return rc;
    }
    hybm::CopyParams p{params->src, params->dest, params->dataSize};
    return MapHybmCode(e->Entity()->CopyData(p, dir, stream, flags));
}

static int32_t BatchImpl(mf_bm_t handle, mf_batch_copy_params *params, mf_bm_copy_type t, void *stream, uint32_t flags)
{
    BmEntry *e = EntryOf(handle);
    MF_CHECK_RET(e != nullptr && params != nullptr, MF_INVALID_PARAM, "bm copy_batch: null argument");
    MF_CHECK_RET(params->sources != nullptr && params->destinations != nullptr && params->dataSizes != nullptr && params->batchSize > 0,
                 MF_INVALID_PARAM, "bm copy_batch: empty batch or null arrays");
    MF_CHECK_RET(params->sources[0] != nullptr && params->destinations[0] != nullptr, MF_INVALID_PARAM, "bm copy_batch: null pointer");
    hybm::CopyDirection dir;
    int rc = e->ResolveType(t, (uint64_t)params->sources[0], (uint64_t)params->destinations[0], &dir);
    if (rc != MF_OK) {
        return rc;
    }
    hybm::BatchCopyParams p{params->sources, params->destinations, params->dataSizes, params->batchSize};
    return MapHybmCode(e->Entity()->BatchCopyData(p, dir, stream, flags));
}

extern "C" int32_t mf_bm_copy(mf_bm_t handle, mf_copy_params *params, mf_bm_copy_type t, uint32_t flags)
{
    return CopyImpl(handle, params, t, nullptr, flags);
}
extern "C" int32_t mf_bm_copy_batch(mf_bm_t handle, mf_batch_copy_params *params, mf_bm_copy_type t, uint32_t flags)
{
    return BatchImpl(handle, params, t, nullptr, flags);
}
extern "C" int32_t mf_bm_copy_on_stream(mf_bm_t handle, mf_copy_params *params, mf_bm_copy_type t, void *stream, uint32_t flags)
{
    // A null handle here means CUDA's default stream, not "pick one for me": hand the engines the explicit legacy-stream handle.
    return CopyImpl(handle, params, t, stream != nullptr ? stream : (void *)cudaStreamLegacy, flags | MF_ASYNC_COPY_FLAG);
}
extern "C" int32_t mf_bm_copy_batch_on_stream(mf_bm_t handle, mf_batch_copy_params *params, mf_bm_copy_type t, void *stream, uint32_t flags)
{
    return BatchImpl(handle, params, t, stream != nullptr ? stream : (void *)cudaStreamLegacy, flags | MF_ASYNC_COPY_FLAG);
}

extern "C" int32_t mf_bm_wait(mf_bm_t handle)
{
    BmEntry *e = EntryOf(handle);
    return e == nullptr ? MF_INVALID_PARAM : MapHybmCode(e->Entity()->Wait());
}

extern "C" int32_t mf_bm_register_user_mem(mf_bm_t handle, uint64_t addr, uint64_t size)
{
    BmEntry *e = EntryOf(handle);
    MF_CHECK_RET(e != nullptr && addr != 0 && size != 0, MF_INVALID_PARAM, "bm register: invalid argument");
    std::lock_guard<std::mutex> lk(e->userMu);
    MF_CHECK_RET(!e->userMem.count(addr), MF_DUPLICATED_OBJECT, "bm register: address already registered");
    if (e->Entity()->Opt().devId >= 0 && cu::Available()) {
        cudaPointerAttributes attr{};
        bool known = cudaPointerGetAttributes(&attr, (void *)addr) == cudaSuccess && attr.type != cudaMemoryTypeUnregistered;
        (void)cudaGetLastError();
        if (!known) {
            // Ordinary host memory: pin it so that copy engines and kernels can use it in place.
            cudaError_t ce = cudaHostRegister((void *)addr, size, cudaHostRegisterPortable | cudaHostRegisterMapped);
            if (ce != cudaSuccess) {
                (void)cudaGetLastError();
                MF_ERROR("bm register: cudaHostRegister failed: " << cu::ErrStr(ce));
                return MF_ERROR;
            }
            e->userMem[addr] = size;
            return MF_OK;
        }
    }
    e->userMem[addr] = 0;  // device or already-pinned memory: nothing to do, remembered for unregister
    return MF_OK;
}

extern "C" int32_t mf_bm_unregister_user_mem(mf_bm_t handle, uint64_t addr)
{
    BmEntry *e = EntryOf(handle);
    MF_CHECK_RET(e != nullptr, MF_INVALID_PARAM, "bm unregister: invalid handle");
    std::lock_guard<std::mutex> lk(e->userMu);
    auto it = e->userMem.find(addr);
    MF_CHECK_RET(it != e->userMem.end(), MF_OBJECT_NOT_EXISTS, "bm unregister: address was not registered");
    if (it->second != 0) {
        cudaHostUnregister((void *)addr);
        (void)cudaGetLastError();
    }
    e->userMem.erase(it);
    return MF_OK;
}

extern "C" uint32_t mf_bm_get_rank_id_by_gva(mf_bm_t handle, void *gva)
{
    BmEntry *e = EntryOf(handle);
    if (e == nullptr || gva == nullptr) {
        return UINT32_MAX;
    }
    uint32_t r = e->Entity()->RankOfAddress((uint64_t)gva);
    return r == hybm::RANK_MAX ? UINT32_MAX : r;
}

extern "C" uint32_t mf_bm_get_joined_size(mf_bm_t handle)
{
    BmEntry *e = EntryOf(handle);
    return e == nullptr ? 0 : e->Group()->RankSize();
}
