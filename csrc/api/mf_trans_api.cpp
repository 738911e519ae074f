// Transfer engine API (include/mf/mf_trans.h).
//
// Reference flow: smem_trans_create → store client under "/trans/", rank id from the store, entity with the user-memory
// segment, device record published (src/smem/csrc/smem_trans/smem_trans_entry.cpp:35-126); register_mem → register +
// export + publish a slice record (:245-306, :592-660); batch transfers translate (peer id, peer address) to a locally
// mapped address by lower_bound over the peer's registrations and run one batch copy (:314-385); a broken store link is
// retried once a second and the engine republishes its records afterwards (:409-451, :690-702).
// Store records (reference schema: smem_trans_store_helper.h:28-43, one status byte + payload per record):
//   /trans/dev/<id>      'N' + {rank, role, pid, device}                 — SET by the owner
//   /trans/slices/<id>   ('N'|'D'|'A') + SliceExport, appended           — 'D' written in place on deregistration
// Departures from the reference: peers' slice records are fetched on demand (first use of a peer, or an address that is
// not known yet) instead of by a polling thread, and nothing sleeps.
#include <sys/mman.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <atomic>
#include <cstring>
#include <map>
#include <mutex>
#include <shared_mutex>
#include <thread>

#include "../hybm/mf_cuda.h"
#include "../store/mf_store_client.h"
#include "../util/mf_log.h"
#include "../util/mf_retry.h"
#include "../util/mf_tracer.h"
#include "mf/mf_trans.h"
#include "mf_api_internal.h"

using namespace mf;
using mf::api::MapHybmCode;

namespace {

constexpr char kNormal = 'N', kDeregistered = 'D', kAbnormal = 'A';
constexpr size_t kSliceRecord = 1 + sizeof(hybm::SliceExport);
constexpr uint32_t kTransEntityBase = 129;  // the reference fixes (16 << 3) + 1; several engines per process count up from it

#pragma pack(push, 1)
struct DevRecord {
    char status;
    uint32_t rank;
    uint32_t role;
    uint32_t pid;
    int32_t devId;
};
#pragma pack(pop)

std::mutex g_mu;
bool g_inited = false;
mf_trans_config_t g_cfg{};
std::atomic<uint32_t> g_nextEntity{0};
std::map<void *, class TransEntry *> g_entries;

class TransEntry {
public:
    TransEntry(std::string url, std::string id, const mf_trans_config_t &cfg) : url_(std::move(url)), id_(std::move(id)), cfg_(cfg) {}
    ~TransEntry() { Shutdown(); }

    int Initialize()
    {
        int rc = MF_OK;
        base_ = mf::api::OpenStore(url_, cfg_.startConfigServer, false, 0, -1, cfg_.initTimeout, &rc);
        MF_CHECK_RET(base_ != nullptr, rc == MF_OK ? MF_ERROR : rc, "trans: cannot reach the config store at " << url_);
        store_ = store::StoreFactory::PrefixOf(base_, "/trans/");
        // A rank id per engine: lowest free id, given back by the server when this link dies.
        std::string v;
        int src = base_->Get(std::string(store::AUTO_RANKING_PREFIX) + "trans", &v, (int64_t)cfg_.initTimeout * 1000);
        MF_CHECK_RET(src == store::ST_OK, MF_ERROR, "trans: cannot obtain a rank id (" << src << ")");
        rank_ = (uint32_t)std::strtoul(v.c_str(), nullptr, 10);
        MF_CHECK_RET(rank_ < hybm::RANK_MAX, MF_ERROR, "trans: more than " << hybm::RANK_MAX << " engines");
        hybm::Options o;
        o.bmType = hybm::INIT_HOST;
        o.scene = hybm::SCENE_TRANS;
        o.role = cfg_.role == MF_TRANS_SENDER ? hybm::ROLE_SENDER : (cfg_.role == MF_TRANS_RECEIVER ? hybm::ROLE_RECEIVER : hybm::ROLE_PEER);
        o.rankCount = hybm::RANK_MAX;
        o.rankId = rank_;
        o.devId = (int32_t)cfg_.deviceId;
        o.memType = hybm::MEM_TYPE_DEVICE;
        o.dataOpType = hybm::OP_KERNEL_LDST | hybm::OP_COPY_ENGINE;
        int hrc = hybm::BM_OK;
        entity_ = hybm::EntityFactory::Instance().Create(kTransEntityBase + g_nextEntity.fetch_add(1) % 64, o, &hrc);
        if (!entity_) {
            return MapHybmCode(hrc);
        }
        rc = PublishDevice();
        if (rc != MF_OK) {
            return rc;
        }
        base_->SetBrokenHandler([this]() { OnBroken(); });
        // A peer whose link to the store breaks (it died, or it left without a word): what is cached about it is stale from that
        // moment on, the next transfer re-reads its records instead of writing into memory of a process that is gone.
        base_->WatchRankDown([this](uint32_t rank) { MarkStale(rank); }, &rankDownWid_);
        return MF_OK;
    }

    void MarkStale(uint32_t rank)
    {
        std::unique_lock<std::shared_mutex> lk(remoteMu_);
        for (auto &kv : remotes_) {
            if (kv.second.rank == rank) {
                kv.second.stale = true;
            }
        }
    }

    void Shutdown()
    {
        stop_.store(true);
        if (reconnect_.joinable()) {
            reconnect_.join();
        }
        if (base_ && rankDownWid_ != 0) {
            base_->Unwatch(rankDownWid_);
            rankDownWid_ = 0;
        }
        if (store_ && base_ && base_->Connected()) {
            // Tell the peers we are gone before the link drops.
            std::string dev = DevBlob(kAbnormal);
            store_->Set("dev/" + id_, dev);
            std::lock_guard<std::mutex> g(localMu_);
            for (auto &kv : local_) {
                store_->Write("slices/" + id_, std::string(1, kDeregistered), kv.second.recordOffset);
            }
        }
        {
            std::unique_lock<std::shared_mutex> lk(remoteMu_);
            remotes_.clear();
        }
        for (auto &kv : hostBlocks_) {
            if (cu::Available()) {
                cudaHostUnregister((void *)kv.first);
                (void)cudaGetLastError();
            }
            ::munmap((void *)kv.first, kv.second.size);
            ::close(kv.second.fd);
        }
        hostBlocks_.clear();
        if (entity_) {
            hybm::EntityFactory::Instance().Destroy(entity_->Id());
            entity_.reset();
        }
    }

    uint32_t Rank() const { return rank_; }

    void *Malloc(size_t capacity)
    {
        if (capacity == 0) {
            MF_ERROR("trans malloc: zero capacity");
            return nullptr;
        }
        size_t size = (capacity + hybm::GRANULE - 1) / hybm::GRANULE * hybm::GRANULE;
        int fd = (int)syscall(SYS_memfd_create, "mf_trans_host", 1u /* MFD_CLOEXEC */);
        if (fd < 0 || ftruncate(fd, (off_t)size) != 0) {
            MF_ERROR("trans malloc: cannot create a " << size << " byte shared file: " << strerror(errno));
            if (fd >= 0) {
                ::close(fd);
            }
            return nullptr;
        }
        // Blocks come out of one fixed window of the address space, bump-allocated (reference: the 128 GiB VA reservation of
        // smem_trans_entry.cpp:179-243), so that a restarted process gets the same addresses again and its peers' bookkeeping of
        // "where the decode side keeps its buffers" stays valid. If the slot is taken the kernel picks the address.
        static std::atomic<uint64_t> bump{0};
        constexpr uint64_t kWindowBase = 0x500000000000ull, kWindowSize = 128ull << 30;
        void *p = MAP_FAILED;
        const uint64_t off = bump.fetch_add(size);
        if (off + size <= kWindowSize) {
            p = ::mmap((void *)(kWindowBase + off), size, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE | MAP_FIXED_NOREPLACE, fd, 0);
            if (p != MAP_FAILED && (uint64_t)p != kWindowBase + off) {  // kernels before 4.17 treat the flag as a hint
                ::munmap(p, size);
                p = MAP_FAILED;
            }
        }
        if (p == MAP_FAILED) {
            p = ::mmap(nullptr, size, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd, 0);
        }
        if (p == MAP_FAILED) {
            MF_ERROR("trans malloc: mmap failed: " << strerror(errno));
            ::close(fd);
            return nullptr;
        }
        if (cu::Available()) {
            cudaSetDevice((int)cfg_.deviceId);
            if (cudaHostRegister(p, size, cudaHostRegisterPortable | cudaHostRegisterMapped) != cudaSuccess) {
                (void)cudaGetLastError();
                MF_WARN("trans malloc: could not pin the block; copies will be staged");
            }
        }
        auto seg = UserSegment();
        if (!seg || seg->AdoptHostBlock((uint64_t)p, size, fd) != hybm::BM_OK) {
            MF_ERROR("trans malloc: cannot make the block shareable");
            ::munmap(p, size);
            ::close(fd);
            return nullptr;
        }
        std::lock_guard<std::mutex> g(localMu_);
        hostBlocks_[(uint64_t)p] = HostBlock{size, fd};
        return p;
    }

    int Free(void *addr)
    {
        std::lock_guard<std::mutex> g(localMu_);
        auto it = hostBlocks_.find((uint64_t)addr);
        MF_CHECK_RET(it != hostBlocks_.end(), MF_INVALID_PARAM, "trans free: address was not returned by mf_trans_malloc");
        for (auto &kv : local_) {
            MF_CHECK_RET(kv.first < it->first || kv.first >= it->first + it->second.size, MF_ERROR,
                         "trans free: deregister the ranges inside the block first");
        }
        if (auto seg = UserSegment()) {
            seg->DropHostBlock(it->first);
        }
        if (cu::Available()) {
            cudaHostUnregister(addr);
            (void)cudaGetLastError();
        }
        ::munmap(addr, it->second.size);
        ::close(it->second.fd);
        hostBlocks_.erase(it);
        return MF_OK;
    }

    int Register(void *addr, size_t size)
    {
        MF_CHECK_RET(addr != nullptr && size != 0, MF_INVALID_PARAM, "trans register: empty range");
        std::lock_guard<std::mutex> g(localMu_);
        MF_CHECK_RET(!local_.count((uint64_t)addr), MF_DUPLICATED_OBJECT, "trans register: address already registered");
        uint64_t slice = 0;
        int rc = entity_->RegisterLocalMemory((uint64_t)addr, size, 0, &slice);
        if (rc != hybm::BM_OK) {
            return MapHybmCode(rc);
        }
        hybm::ExchangeInfo info{};
        rc = entity_->Export(slice, 0, &info);
        if (rc != hybm::BM_OK) {
            entity_->FreeLocalMemory(slice);
            return MapHybmCode(rc);
        }
        hybm::SliceExport se;
        std::memcpy(&se, info.desc, sizeof(se));
        if (se.handleKind == hybm::HK_NONE) {
            entity_->FreeLocalMemory(slice);
            MF_ERROR("trans register: this memory cannot be shared with other processes (use device memory or mf_trans_malloc)");
            return MF_INVALID_PARAM;
        }
        std::string rec(1, kNormal);
        rec.append((const char *)info.desc, sizeof(hybm::SliceExport));
        uint64_t total = 0;
        int src = store_->Append("slices/" + id_, rec, &total);
        if (src != store::ST_OK) {
            entity_->FreeLocalMemory(slice);
            MF_ERROR("trans register: cannot publish the registration (" << src << ")");
            return MF_ERROR;
        }
        local_[(uint64_t)addr] = LocalReg{size, slice, (uint32_t)(total - kSliceRecord), rec};
        return MF_OK;
    }

    int Deregister(void *addr)
    {
        std::lock_guard<std::mutex> g(localMu_);
        auto it = local_.find((uint64_t)addr);
        MF_CHECK_RET(it != local_.end(), MF_OBJECT_NOT_EXISTS, "trans deregister: address was not registered");
        store_->Write("slices/" + id_, std::string(1, kDeregistered), it->second.recordOffset);
        entity_->FreeLocalMemory(it->second.slice);
        local_.erase(it);
        return MF_OK;
    }

    // A transfer that fails because the peer is gone, restarting or not mappable right now is tried again after 1 s and after
    // 2 more seconds; before each new attempt everything known about the peer is dropped, so that the attempt re-reads the
    // peer's records from the store and maps its memory afresh (a restarted peer has new descriptors and maybe new
    // addresses). Errors in the arguments themselves are returned at once.
    int Transfer(bool write, const void *const *locals, const char *remoteId, const void *const *remotes, const size_t *sizes, uint32_t n,
                 void *stream, bool async, uint32_t flags)
    {
        int ret = MF_OK;
        RetryWithBackoff(
            [&]() {
                ret = TransferOnce(write, locals, remoteId, remotes, sizes, n, stream, async, flags);
                return ret == MF_OK || ret == MF_INVALID_PARAM || ret == MF_NOT_INITIALIZED || stop_.load();
            },
            [&](uint32_t failed) {
                MF_WARN("trans transfer to " << remoteId << " failed (" << ret << "), attempt " << failed + 1 << " after re-reading the peer's records");
                std::unique_lock<std::shared_mutex> lk(remoteMu_);
                auto it = remotes_.find(remoteId);
                if (it != remotes_.end()) {
                    DropRemote(it->second);
                    it->second.rank = hybm::RANK_MAX;
                }
            });
        return ret;
    }

    int TransferOnce(bool write, const void *const *locals, const char *remoteId, const void *const *remotes, const size_t *sizes, uint32_t n,
                     void *stream, bool async, uint32_t flags)
    {
        int ret = MF_OK;
        MF_TRACE_SCOPE(MF_TP(TM_TRANS, write ? 0 : 1), write ? "TRANS_BATCH_WRITE" : "TRANS_BATCH_READ", &ret);
        if (locals == nullptr || remotes == nullptr || sizes == nullptr || remoteId == nullptr || n == 0) {
            MF_ERROR("trans transfer: null or empty arguments");
            return ret = MF_INVALID_PARAM;
        }
        std::vector<void *> src(n), dst(n);
        std::vector<uint64_t> len(n);
        uint32_t remoteType = hybm::MEM_TYPE_DEVICE;
        uint32_t peerRank = hybm::RANK_MAX;
        {
            std::shared_lock<std::shared_mutex> lk(remoteMu_);
            auto it = remotes_.find(remoteId);
            if (it != remotes_.end()) {
                peerRank = it->second.rank;
            }
        }
        if (peerRank == hybm::RANK_MAX) {
            int rrc = Refresh(remoteId);
            if (rrc != MF_OK) {
                return ret = rrc;
            }
            std::shared_lock<std::shared_mutex> lk(remoteMu_);
            peerRank = remotes_[remoteId].rank;
        }
        if (peerRank != hybm::RANK_MAX && entity_->IsRemoteRank(peerRank)) {
            // The peer lives on another host: nothing of it is mapped here. Every piece is a one-sided put or get through the
            // host transport, addressed in the peer's own address space (device-side locals are staged by the entity).
            for (uint32_t i = 0; i < n; i++) {
                if (locals[i] == nullptr || remotes[i] == nullptr) {
                    MF_ERROR("trans transfer: null address at #" << i);
                    return ret = MF_INVALID_PARAM;
                }
                uint64_t mapped = 0;
                ret = Resolve(remoteId, (uint64_t)remotes[i], sizes[i], &mapped, &remoteType);
                if (ret != MF_OK) {
                    return ret;
                }
                ret = MapHybmCode(entity_->RemoteUserCopy(peerRank, (uint64_t)locals[i], mapped, sizes[i], write, stream));
                if (ret != MF_OK) {
                    return ret;
                }
            }
            return ret;
        }
        for (uint32_t i = 0; i < n; i++) {
            if (locals[i] == nullptr || remotes[i] == nullptr) {
                MF_ERROR("trans transfer: null address at #" << i);
                return ret = MF_INVALID_PARAM;
            }
            uint64_t mapped = 0;
            ret = Resolve(remoteId, (uint64_t)remotes[i], sizes[i], &mapped, &remoteType);
            if (ret != MF_OK) {
                return ret;
            }
            src[i] = write ? const_cast<void *>(locals[i]) : (void *)mapped;
            dst[i] = write ? (void *)mapped : const_cast<void *>(locals[i]);
            len[i] = sizes[i];
        }
        hybm::BatchCopyParams p{src.data(), dst.data(), len.data(), n};
        hybm::ExtOptions ext;
        ext.srcRank = ext.dstRank = rank_;
        ext.stream = stream;
        ext.flags = flags | (async ? hybm::FLAG_ASYNC_COPY : 0);
        bool localVisible = true;
        hybm::PtrClass lc = entity_->Classify((uint64_t)locals[0], &localVisible);
        if (lc == hybm::PC_GLOBAL_DEVICE) {
            lc = hybm::PC_LOCAL_DEVICE;  // a registered local buffer is still the local side of this transfer
        } else if (lc == hybm::PC_GLOBAL_HOST) {
            lc = hybm::PC_LOCAL_HOST;
        }
        const hybm::PtrClass rcls = remoteType == hybm::MEM_TYPE_DEVICE ? hybm::PC_GLOBAL_DEVICE : hybm::PC_GLOBAL_HOST;
        (write ? ext.srcDeviceVisible : ext.dstDeviceVisible) = localVisible;
        (write ? ext.dstDeviceVisible : ext.srcDeviceVisible) = cu::Available();
        const hybm::CopyDirection dir = write ? hybm::DirectionOf(lc, rcls) : hybm::DirectionOf(rcls, lc);
        std::shared_lock<std::shared_mutex> lk(remoteMu_);  // mappings stay put while the copy is being issued
        ret = MapHybmCode(entity_->DataOp()->BatchDataCopy(p, dir, ext));
        return ret;
    }

private:
    struct LocalReg {
        size_t size;
        uint64_t slice;
        uint32_t recordOffset;
        std::string record;
    };
    struct HostBlock {
        size_t size;
        int fd;
    };
    struct RemoteRange {
        uint64_t size;
        uint64_t local;
        uint32_t memType;
    };
    struct Remote {
        size_t parsedBytes{0};
        std::map<uint64_t, RemoteRange> ranges;  // peer address → mapping
        std::map<uint32_t, uint64_t> recordAddr;  // record offset → peer address (to honour later status changes)
        uint32_t rank{hybm::RANK_MAX};
        bool stale{false};  // the peer's link to the store broke after these mappings were made
    };

    std::shared_ptr<hybm::MemSegment> UserSegment() { return entity_ ? entity_->Segment(hybm::MEM_TYPE_DEVICE) : nullptr; }

    std::string DevBlob(char status) const
    {
        DevRecord d{status, rank_, (uint32_t)cfg_.role, (uint32_t)getpid(), (int32_t)cfg_.deviceId};
        return std::string((const char *)&d, sizeof(d));
    }

    int PublishDevice()
    {
        int rc = store_->Set("dev/" + id_, DevBlob(kNormal));
        MF_CHECK_RET(rc == store::ST_OK, MF_ERROR, "trans: cannot publish the device record (" << rc << ")");
        return MF_OK;
    }

    static bool Lookup(const Remote &r, uint64_t addr, uint64_t size, uint64_t *mapped, uint32_t *memType)
    {
        auto it = r.ranges.upper_bound(addr);
        if (it == r.ranges.begin()) {
            return false;
        }
        --it;
        if (addr < it->first || addr + size > it->first + it->second.size) {
            return false;
        }
        *mapped = it->second.local + (addr - it->first);
        *memType = it->second.memType;
        return true;
    }

    int Resolve(const std::string &remoteId, uint64_t addr, uint64_t size, uint64_t *mapped, uint32_t *memType)
    {
        {
            std::shared_lock<std::shared_mutex> lk(remoteMu_);
            auto it = remotes_.find(remoteId);
            if (it != remotes_.end() && !it->second.stale && Lookup(it->second, addr, size, mapped, memType)) {
                return MF_OK;
            }
        }
        int rc = Refresh(remoteId);
        if (rc != MF_OK) {
            return rc;
        }
        std::shared_lock<std::shared_mutex> lk(remoteMu_);
        auto it = remotes_.find(remoteId);
        if (it != remotes_.end() && Lookup(it->second, addr, size, mapped, memType)) {
            return MF_OK;
        }
        MF_ERROR("trans transfer: [0x" << std::hex << addr << ", +0x" << size << std::dec << ") is not inside memory registered by " << remoteId);
        return MF_INVALID_PARAM;
    }

    // Reads the peer's slice records and reconciles the local view with them.
    int Refresh(const std::string &remoteId)
    {
        std::string dev;
        int rc = store_->Get("dev/" + remoteId, &dev, (int64_t)cfg_.initTimeout * 1000);
        MF_CHECK_RET(rc == store::ST_OK && dev.size() == sizeof(DevRecord), MF_OBJECT_NOT_EXISTS, "trans: peer " << remoteId << " is not known to the store");
        DevRecord d;
        std::memcpy(&d, dev.data(), sizeof(d));
        std::unique_lock<std::shared_mutex> lk(remoteMu_);
        Remote &r = remotes_[remoteId];
        if (r.stale) {
            DropRemote(r);  // the process these mappings belonged to is gone; whoever holds the id now is mapped from scratch
            r.rank = hybm::RANK_MAX;
            r.stale = false;
        }
        if (d.status != kNormal) {
            DropRemote(r);
            MF_ERROR("trans: peer " << remoteId << " has left or died");
            return MF_OBJECT_NOT_EXISTS;
        }
        if (r.rank != hybm::RANK_MAX && r.rank != d.rank) {
            DropRemote(r);  // the id was taken over by a new process
        }
        r.rank = d.rank;
        // Transfers run between a sender and a receiver (or with an engine that is both): a sender never maps another sender's
        // memory, a receiver never another receiver's.
        const hybm::Role peerRole = d.role == MF_TRANS_SENDER ? hybm::ROLE_SENDER : (d.role == MF_TRANS_RECEIVER ? hybm::ROLE_RECEIVER : hybm::ROLE_PEER);
        entity_->SetPeerRole(d.rank, peerRole);
        if (!entity_->RolePermits(d.rank)) {
            MF_ERROR("trans: " << remoteId << " has the same role (" << (d.role == MF_TRANS_SENDER ? "sender" : "receiver")
                               << ") as this engine; transfers need a sender on one side and a receiver on the other");
            return MF_INVALID_PARAM;
        }
        std::string all;
        rc = store_->Get("slices/" + remoteId, &all, 0);
        if (rc == store::ST_NOT_EXIST) {
            return MF_OK;  // nothing registered yet
        }
        MF_CHECK_RET(rc == store::ST_OK, MF_ERROR, "trans: cannot read the registrations of " << remoteId << " (" << rc << ")");
        for (size_t off = 0; off + kSliceRecord <= all.size(); off += kSliceRecord) {
            const char status = all[off];
            auto known = r.recordAddr.find((uint32_t)off);
            if (status != kNormal) {
                if (known != r.recordAddr.end()) {
                    r.ranges.erase(known->second);
                    r.recordAddr.erase(known);
                }
                continue;
            }
            if (known != r.recordAddr.end()) {
                continue;
            }
            hybm::ExchangeInfo info{};
            std::memcpy(info.desc, all.data() + off + 1, sizeof(hybm::SliceExport));
            info.descLen = sizeof(hybm::SliceExport);
            hybm::SliceExport se;
            std::memcpy(&se, info.desc, sizeof(se));
            void *local = nullptr;
            int hrc = entity_->Import(&info, 1, &local, 0);
            if (hrc != hybm::BM_OK || local == nullptr) {
                MF_WARN("trans: cannot map a registration of " << remoteId << " (" << hrc << "), skipping it");
                continue;
            }
            r.ranges[se.gva] = RemoteRange{se.size, (uint64_t)local, se.memType};
            r.recordAddr[(uint32_t)off] = se.gva;
        }
        r.parsedBytes = all.size();
        if (entity_->IsRemoteRank(d.rank)) {
            // Peer on another host: "mapping" it means handing its address and keys to the host transport and linking up.
            int mrc = entity_->Mmap();
            MF_CHECK_RET(mrc == hybm::BM_OK, MF_ERROR, "trans: cannot link to " << remoteId << " on another host (" << mrc << ")");
        }
        return MF_OK;
    }

    void DropRemote(Remote &r)
    {
        if (r.rank != hybm::RANK_MAX && entity_) {
            entity_->RemoveImported(r.rank);
        }
        r.ranges.clear();
        r.recordAddr.clear();
        r.parsedBytes = 0;
    }

    void OnBroken()
    {
        if (stop_.load() || reconnecting_.exchange(true)) {
            return;
        }
        if (reconnect_.joinable()) {
            reconnect_.detach();
        }
        reconnect_ = std::thread([this]() {
            while (!stop_.load()) {
                if (base_->ReconnectAfterBroken(1) == store::ST_OK) {
                    Republish();
                    break;
                }
                for (int i = 0; i < 10 && !stop_.load(); i++) {
                    usleep(100 * 1000);
                }
            }
            reconnecting_.store(false);
        });
    }

    // After the store came back (possibly empty): put the device record and every live registration there again.
    void Republish()
    {
        std::string v;
        base_->Get(std::string(store::AUTO_RANKING_PREFIX) + "trans", &v, 5000);
        PublishDevice();
        std::lock_guard<std::mutex> g(localMu_);
        std::string cur;
        if (store_->Get("slices/" + id_, &cur, 0) == store::ST_OK && !cur.empty()) {
            return;  // the server kept our records
        }
        for (auto &kv : local_) {
            uint64_t total = 0;
            if (store_->Append("slices/" + id_, kv.second.record, &total) == store::ST_OK) {
                kv.second.recordOffset = (uint32_t)(total - kSliceRecord);
            }
        }
        MF_INFO("trans: records of " << id_ << " republished after a store reconnect");
    }

    uint32_t rankDownWid_{0};
    std::string url_, id_;
    mf_trans_config_t cfg_;
    store::StorePtr base_, store_;
    std::shared_ptr<hybm::MemEntity> entity_;
    uint32_t rank_{0};
    std::mutex localMu_;
    std::map<uint64_t, LocalReg> local_;
    std::map<uint64_t, HostBlock> hostBlocks_;
    std::shared_mutex remoteMu_;
    std::map<std::string, Remote> remotes_;
    std::atomic<bool> stop_{false};
    std::atomic<bool> reconnecting_{false};
    std::thread reconnect_;
};

TransEntry *EntryOf(mf_trans_t h)
{
    std::lock_guard<std::mutex> g(g_mu);
    auto it = g_entries.find(h);
    if (it == g_entries.end()) {
        MF_ERROR("trans: invalid handle");
        return nullptr;
    }
    return it->second;
}

}  // namespace

// ---------------------------------------------------------------------------------------------- server-side fault handler
// Learns which link owns which engine id and which slice records (reference: SmemStoreFaultHandler,
// src/smem/csrc/smem_trans/smem_trans_fault_handler.cpp:23-302). When a link breaks, the owner's device record and slice
// records are marked ABNORMAL in place so that peers drop their mappings on the next refresh; the rank id itself is
// recycled by the server's auto-ranking table.
namespace mf {
namespace api {

void AttachTransFaultHandler(store::StoreServer *server)
{
    struct State {
        std::mutex mu;
        std::map<net::LinkId, std::vector<std::string>> owned;  // link → engine ids whose dev record it SET
    };
    auto st = std::make_shared<State>();
    server->SetOpHook([st](uint16_t op, net::LinkId link, const std::string &key, const std::string &value, std::string *) -> int {
        static const std::string prefix = "/trans/dev/";
        if (op == store::OP_SET && key.compare(0, prefix.size(), prefix) == 0 && !value.empty() && value[0] == kNormal) {
            std::lock_guard<std::mutex> g(st->mu);
            auto &v = st->owned[link];
            std::string id = key.substr(prefix.size());
            if (std::find(v.begin(), v.end(), id) == v.end()) {
                v.push_back(id);
            }
        }
        return store::ST_ERROR;  // never answers a request itself
    });
    server->SetBrokenHook([st](net::LinkId link, store::StoreBackend *backend) {
        std::vector<std::string> ids;
        {
            std::lock_guard<std::mutex> g(st->mu);
            auto it = st->owned.find(link);
            if (it == st->owned.end()) {
                return;
            }
            ids.swap(it->second);
            st->owned.erase(it);
        }
        for (auto &id : ids) {
            if (std::string *dev = backend->Mutable("/trans/dev/" + id)) {
                if (!dev->empty()) {
                    (*dev)[0] = kAbnormal;
                }
            }
            if (std::string *sl = backend->Mutable("/trans/slices/" + id)) {
                for (size_t off = 0; off + kSliceRecord <= sl->size(); off += kSliceRecord) {
                    if ((*sl)[off] == kNormal) {
                        (*sl)[off] = kAbnormal;
                    }
                }
            }
            MF_INFO("trans fault handler: engine " << id << " marked abnormal after its link broke");
        }
    });
}

}  // namespace api
}  // namespace mf

// ---------------------------------------------------------------------------------------------- C API

extern "C" int32_t mf_trans_config_init(mf_trans_config_t *c)
{
    MF_CHECK_RET(c != nullptr, MF_INVALID_PARAM, "trans config_init: null config");
    c->role = MF_TRANS_BOTH;
    c->initTimeout = 120;
    c->deviceId = 0;
    c->flags = 0;
    c->dataOpType = MF_BM_DATA_OP_SDMA;
    c->startConfigServer = false;
    return MF_OK;
}

extern "C" int32_t mf_trans_init(const mf_trans_config_t *config)
{
    MF_CHECK_RET(config != nullptr, MF_INVALID_PARAM, "trans init: null config");
    MF_CHECK_RET(config->role > MF_TRANS_NONE && config->role < MF_TRANS_BUTT && config->initTimeout > 0, MF_INVALID_PARAM,
                 "trans init: invalid role or timeout");
    std::lock_guard<std::mutex> g(g_mu);
    if (g_inited) {
        return MF_OK;
    }
    int rc = hybm::HybmInit(cu::Available() ? (int)config->deviceId : -1, 0);
    if (rc != hybm::BM_OK) {
        return MapHybmCode(rc);
    }
    g_cfg = *config;
    g_inited = true;
    return MF_OK;
}

extern "C" void mf_trans_uninit(uint32_t /*flags*/)
{
    std::map<void *, TransEntry *> entries;
    {
        std::lock_guard<std::mutex> g(g_mu);
        entries.swap(g_entries);
    }
    for (auto &kv : entries) {
        delete kv.second;
    }
    std::lock_guard<std::mutex> g(g_mu);
    if (g_inited) {
        hybm::HybmUninit();
        g_inited = false;
    }
}

extern "C" mf_trans_t mf_trans_create(const char *storeUrl, const char *uniqueId, const mf_trans_config_t *config)
{
    if (storeUrl == nullptr || uniqueId == nullptr || config == nullptr || uniqueId[0] == '\0' || std::strlen(uniqueId) > 200) {
        MF_ERROR("trans create: null or malformed argument");
        return nullptr;
    }
    {
        std::lock_guard<std::mutex> g(g_mu);
        if (!g_inited) {
            MF_ERROR("trans create: call mf_trans_init first");
            return nullptr;
        }
    }
    auto *e = new TransEntry(storeUrl, uniqueId, *config);
    int rc = e->Initialize();
    if (rc != MF_OK) {
        MF_ERROR("trans create: failed (" << rc << ")");
        delete e;
        return nullptr;
    }
    std::lock_guard<std::mutex> g(g_mu);
    g_entries[e] = e;
    return e;
}

extern "C" int32_t mf_trans_destroy(mf_trans_t handle, uint32_t /*flags*/)
{
    TransEntry *e = nullptr;
    {
        std::lock_guard<std::mutex> g(g_mu);
        auto it = g_entries.find(handle);
        if (it != g_entries.end()) {
            e = it->second;
            g_entries.erase(it);
        }
    }
    MF_CHECK_RET(e != nullptr, MF_INVALID_PARAM, "trans destroy: invalid handle");
    delete e;
    return MF_OK;
}

extern "C" void *mf_trans_malloc(mf_trans_t handle, size_t capacity)
{
    TransEntry *e = EntryOf(handle);
    return e == nullptr ? nullptr : e->Malloc(capacity);
}

extern "C" int32_t mf_trans_free(mf_trans_t handle, void *address)
{
    TransEntry *e = EntryOf(handle);
    return e == nullptr ? MF_INVALID_PARAM : e->Free(address);
}

extern "C" int32_t mf_trans_register_mem(mf_trans_t handle, void *address, size_t capacity, uint32_t /*flags*/)
{
    TransEntry *e = EntryOf(handle);
    return e == nullptr ? MF_INVALID_PARAM : e->Register(address, capacity);
}

extern "C" int32_t mf_trans_batch_register_mem(mf_trans_t handle, void *addresses[], size_t capacities[], uint32_t count, uint32_t flags)
{
    MF_CHECK_RET(addresses != nullptr && capacities != nullptr && count > 0, MF_INVALID_PARAM, "trans batch_register: null or empty arguments");
    for (uint32_t i = 0; i < count; i++) {
        int rc = mf_trans_register_mem(handle, addresses[i], capacities[i], flags);
        if (rc != MF_OK) {
            return rc;
        }
    }
    return MF_OK;
}

extern "C" int32_t mf_trans_deregister_mem(mf_trans_t handle, void *address)
{
    TransEntry *e = EntryOf(handle);
    return e == nullptr ? MF_INVALID_PARAM : e->Deregister(address);
}

extern "C" int32_t mf_trans_write(mf_trans_t h, const void *l, const char *id, void *r, size_t n, uint32_t flags)
{
    TransEntry *e = EntryOf(h);
    const void *rc = r;
    return e == nullptr ? MF_INVALID_PARAM : e->Transfer(true, &l, id, &rc, &n, 1, nullptr, false, flags);
}
extern "C" int32_t mf_trans_read(mf_trans_t h, void *l, const char *id, const void *r, size_t n, uint32_t flags)
{
    TransEntry *e = EntryOf(h);
    const void *lc = l;
    return e == nullptr ? MF_INVALID_PARAM : e->Transfer(false, &lc, id, &r, &n, 1, nullptr, false, flags);
}
extern "C" int32_t mf_trans_batch_write(mf_trans_t h, const void *l[], const char *id, void *r[], size_t n[], uint32_t count, uint32_t flags)
{
    TransEntry *e = EntryOf(h);
    return e == nullptr ? MF_INVALID_PARAM : e->Transfer(true, l, id, (const void *const *)r, n, count, nullptr, false, flags);
}
extern "C" int32_t mf_trans_batch_read(mf_trans_t h, void *l[], const char *id, const void *r[], size_t n[], uint32_t count, uint32_t flags)
{
    TransEntry *e = EntryOf(h);
    return e == nullptr ? MF_INVALID_PARAM : e->Transfer(false, (const void *const *)l, id, r, n, count, nullptr, false, flags);
}
static void *StreamOrLegacy(void *s) { return s != nullptr ? s : (void *)cudaStreamLegacy; }
extern "C" int32_t mf_trans_write_submit(mf_trans_t h, const void *l, const char *id, void *r, size_t n, void *stream, uint32_t flags)
{
    TransEntry *e = EntryOf(h);
    const void *rc = r;
    return e == nullptr ? MF_INVALID_PARAM : e->Transfer(true, &l, id, &rc, &n, 1, StreamOrLegacy(stream), true, flags);
}
extern "C" int32_t mf_trans_read_submit(mf_trans_t h, void *l, const char *id, const void *r, size_t n, void *stream, uint32_t flags)
{
    TransEntry *e = EntryOf(h);
    const void *lc = l;
    return e == nullptr ? MF_INVALID_PARAM : e->Transfer(false, &lc, id, &r, &n, 1, StreamOrLegacy(stream), true, flags);
}
extern "C" int32_t mf_trans_batch_write_submit(mf_trans_t h, const void *l[], const char *id, void *r[], size_t n[], uint32_t count, void *stream,
                                               uint32_t flags)
{
    TransEntry *e = EntryOf(h);
    return e == nullptr ? MF_INVALID_PARAM : e->Transfer(true, l, id, (const void *const *)r, n, count, StreamOrLegacy(stream), true, flags);
}
extern "C" int32_t mf_trans_batch_read_submit(mf_trans_t h, void *l[], const char *id, const void *r[], size_t n[], uint32_t count, void *stream,
                                              uint32_t flags)
{
    TransEntry *e = EntryOf(h);
    return e == nullptr ? MF_INVALID_PARAM : e->Transfer(false, (const void *const *)l, id, r, n, count, StreamOrLegacy(stream), true, flags);
}

extern "C" uint32_t mf_trans_get_rank(mf_trans_t h)
{
    TransEntry *e = EntryOf(h);
    return e == nullptr ? UINT32_MAX : e->Rank();
}
