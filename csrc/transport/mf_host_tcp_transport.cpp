#include "mf_host_tcp_transport.h"

#include <algorithm>
#include <cstring>
#include <random>

#include "../util/mf_log.h"
#include "../util/mf_retry.h"

namespace mf {
namespace transport {

using hybm::BM_ERROR;
using hybm::BM_INVALID_PARAM;
using hybm::BM_NOT_INITIALIZED;
using hybm::BM_OK;
using hybm::BM_TIMEOUT;

namespace {
constexpr uint16_t kMsgRead = 0x0201;
constexpr uint16_t kMsgWrite = 0x0202;
constexpr uint64_t kMaxSliceBytes = 32ull << 20;  // well under the frame limit of the RPC layer

#pragma pack(push, 1)
struct OneSidedHeader {
    uint64_t token;
    uint64_t addr;
    uint64_t size;
};
#pragma pack(pop)

uint64_t RandomToken()
{
    static std::mutex mu;
    static std::mt19937_64 gen{std::random_device{}()};
    std::lock_guard<std::mutex> g(mu);
    uint64_t t;
    do {
        t = gen();
    } while (t == 0);
    return t;
}
}  // namespace

HostTcpTransport::HostTcpTransport() = default;

HostTcpTransport::~HostTcpTransport() { CloseDevice(); }

int HostTcpTransport::OpenDevice(const Options &opt)
{
    if (open_.load()) {
        return BM_OK;
    }
    if (opt.rankCount == 0 || opt.rankId >= opt.rankCount || opt.workers == 0 || opt.workers > 64 || opt.sliceBytes == 0) {
        MF_ERROR("host transport: invalid options rank=" << opt.rankId << "/" << opt.rankCount << " workers=" << opt.workers);
        return BM_INVALID_PARAM;
    }
    opt_ = opt;
    opt_.sliceBytes = std::min<uint64_t>(opt.sliceBytes, kMaxSliceBytes);
    net::Endpoint ep;
    const std::string nic = opt.nic.empty() ? std::string("127.0.0.1:0") : opt.nic;
    // ParseUrl refuses port 0, which here means "any free port": split it off by hand in that case.
    std::string text = nic.rfind("tcp://", 0) == 0 ? nic.substr(6) : nic;
    size_t colon = text.rfind(':');
    if (colon != std::string::npos && text.substr(colon + 1) == "0") {
        if (!net::ParseUrl(text.substr(0, colon) + ":1", &ep)) {
            MF_ERROR("host transport: bad listen address " << nic);
            return BM_INVALID_PARAM;
        }
        ep.port = 0;
    } else if (!net::ParseUrl(text, &ep)) {
        MF_ERROR("host transport: bad listen address " << nic);
        return BM_INVALID_PARAM;
    }
    if (opt.tls.enable) {
        std::string err;
        auto serverCtx = net::TlsContext::Create(opt.tls, true, &err);
        tlsClient_ = net::TlsContext::Create(opt.tls, false, &err);
        if (serverCtx == nullptr || tlsClient_ == nullptr) {
            MF_ERROR("host transport: TLS set-up failed: " << err);
            return BM_ERROR;
        }
        server_.SetTls(serverCtx);
    }
    server_.SetHandlers([this](net::LinkId l, const net::Frame &f) { OnRequest(l, f); }, nullptr, nullptr);
    int rc = server_.Start(ep);
    if (rc != 0) {
        MF_ERROR("host transport: cannot listen on " << nic << " (" << rc << ")");
        return BM_ERROR;
    }
    const bool bracket = ep.v6;
    nic_ = (bracket ? "[" + ep.host + "]" : ep.host) + ":" + std::to_string(server_.Port());
    {
        std::lock_guard<std::mutex> g(qMu_);
        stopping_ = false;
    }
    for (uint32_t i = 0; i < opt_.workers; i++) {
        workers_.emplace_back([this]() { WorkerLoop(); });
    }
    open_.store(true);
    MF_INFO("host transport: rank " << opt_.rankId << " serves its host memory at " << nic_);
    return BM_OK;
}

int HostTcpTransport::CloseDevice()
{
    if (!open_.exchange(false)) {
        return BM_OK;
    }
    {
        std::lock_guard<std::mutex> g(qMu_);
        stopping_ = true;
    }
    qCv_.notify_all();
    for (auto &w : workers_) {
        w.join();
    }
    workers_.clear();
    // Whatever was still queued will never run: finish it as failed so that nobody waits for it.
    for (auto &s : queue_) {
        s.peer->counter.Complete(BM_ERROR);
    }
    queue_.clear();
    if (connector_.joinable()) {
        connector_.join();
    }
    {
        util::WriteGuard g(peerMu_);
        for (auto &kv : peers_) {
            std::lock_guard<std::mutex> lg(kv.second->linkMu);
            if (kv.second->link) {
                kv.second->link->SetBrokenHandler(nullptr);
                kv.second->link->Close();
                kv.second->link.reset();
            }
        }
        peers_.clear();
    }
    server_.Stop();
    {
        util::WriteGuard g(regionMu_);
        regions_.clear();
    }
    return BM_OK;
}

// ------------------------------------------------------------------------------------------------------ regions

int HostTcpTransport::RegisterMemoryRegion(const MemoryRegion &mr)
{
    if (mr.addr == 0 || mr.size == 0 || mr.addr + mr.size < mr.addr) {
        return BM_INVALID_PARAM;
    }
    util::WriteGuard g(regionMu_);
    // No overlap with an existing region.
    auto next = regions_.lower_bound(mr.addr);
    if (next != regions_.end() && next->first < mr.addr + mr.size) {
        MF_ERROR("host transport: region 0x" << std::hex << mr.addr << "+0x" << mr.size << " overlaps a registered one" << std::dec);
        return BM_INVALID_PARAM;
    }
    if (next != regions_.begin()) {
        auto prev = std::prev(next);
        if (prev->second.addr + prev->second.size > mr.addr) {
            MF_ERROR("host transport: region 0x" << std::hex << mr.addr << "+0x" << mr.size << " overlaps a registered one" << std::dec);
            return BM_INVALID_PARAM;
        }
    }
    MemoryKey k;
    k.token = RandomToken();
    k.addr = mr.addr;
    k.size = mr.size;
    k.access = mr.access;
    k.flags = mr.flags == 0 ? MR_FLAG_DRAM : mr.flags;
    regions_[mr.addr] = k;
    return BM_OK;
}

int HostTcpTransport::UnregisterMemoryRegion(uint64_t addr)
{
    util::WriteGuard g(regionMu_);  // waits for requests that are copying from / into the region right now
    return regions_.erase(addr) == 1 ? BM_OK : BM_INVALID_PARAM;
}

bool HostTcpTransport::QueryHasRegistered(uint64_t addr, uint64_t size)
{
    util::ReadGuard g(regionMu_);
    auto it = regions_.upper_bound(addr);
    if (it == regions_.begin()) {
        return false;
    }
    --it;
    return it->second.Covers(addr, size);
}

int HostTcpTransport::QueryMemoryKey(uint64_t addr, MemoryKey *key)
{
    if (key == nullptr) {
        return BM_INVALID_PARAM;
    }
    util::ReadGuard g(regionMu_);
    auto it = regions_.upper_bound(addr);
    if (it == regions_.begin()) {
        return BM_INVALID_PARAM;
    }
    --it;
    if (!it->second.Covers(addr, 1)) {
        return BM_INVALID_PARAM;
    }
    *key = it->second;
    return BM_OK;
}

// ------------------------------------------------------------------------------------------------------ serving side

void HostTcpTransport::OnRequest(net::LinkId link, const net::Frame &f)
{
    net::Frame r;
    r.type = f.type;
    r.seq = f.seq;
    r.result = (int16_t)BM_INVALID_PARAM;
    OneSidedHeader h{};
    if ((f.type != kMsgRead && f.type != kMsgWrite) || f.body.size() < sizeof(h)) {
        stats_.refused.fetch_add(1);
        server_.Send(link, r);
        return;
    }
    std::memcpy(&h, f.body.data(), sizeof(h));
    const bool write = f.type == kMsgWrite;
    if (h.size == 0 || h.size > kMaxSliceBytes || (write && f.body.size() != sizeof(h) + h.size) || (!write && f.body.size() != sizeof(h))) {
        stats_.refused.fetch_add(1);
        server_.Send(link, r);
        return;
    }
    {
        util::ReadGuard g(regionMu_);  // the region cannot be unregistered while its bytes are being copied
        auto it = regions_.upper_bound(h.addr);
        const MemoryKey *k = nullptr;
        if (it != regions_.begin()) {
            --it;
            k = &it->second;
        }
        const uint32_t need = write ? MR_ACCESS_REMOTE_WRITE : MR_ACCESS_REMOTE_READ;
        if (k == nullptr || !k->Covers(h.addr, h.size) || k->token != h.token || (k->access & need) == 0) {
            stats_.refused.fetch_add(1);
            MF_WARN_LIMIT("host transport: refused a " << (write ? "write" : "read") << " of 0x" << std::hex << h.size << " at 0x" << h.addr
                                                          << std::dec << " (outside a region, wrong token or access not granted)");
        } else if ((k->flags & MR_FLAG_HBM) != 0) {
            // Device memory: staged through the frame's own buffer by the owner's copier.
            if (!deviceCopier_) {
                stats_.refused.fetch_add(1);
            } else if (write) {
                r.result = deviceCopier_((void *)h.addr, f.body.data() + sizeof(h), h.size) == 0 ? 0 : (int16_t)BM_ERROR;
            } else {
                r.body.resize(h.size);
                r.result = deviceCopier_(&r.body[0], (const void *)h.addr, h.size) == 0 ? 0 : (int16_t)BM_ERROR;
                if (r.result != 0) {
                    r.body.clear();
                }
            }
        } else if (write) {
            std::memcpy((void *)h.addr, f.body.data() + sizeof(h), h.size);
            r.result = 0;
        } else {
            // The reply's body is the region itself: it goes to the socket from where it lies, still under the read lock.
            r.result = 0;
            stats_.bytesServed.fetch_add(h.size);
            server_.SendWithPayload(link, r, (const void *)h.addr, h.size);
            return;
        }
    }
    if (r.result == 0) {
        stats_.bytesServed.fetch_add(h.size);
    }
    server_.Send(link, r);
}

// ------------------------------------------------------------------------------------------------------ peers and links

std::shared_ptr<HostTcpTransport::Peer> HostTcpTransport::FindPeer(uint32_t rankId)
{
    util::ReadGuard g(peerMu_);
    auto it = peers_.find(rankId);
    return it == peers_.end() ? nullptr : it->second;
}

int HostTcpTransport::ApplyRanks(const PrepareOptions &opt, bool replaceAll)
{
    util::WriteGuard g(peerMu_);
    if (replaceAll) {
        peers_.clear();
    }
    for (const auto &kv : opt.ranks) {
        if (kv.first >= opt_.rankCount) {
            MF_ERROR("host transport: rank " << kv.first << " beyond the rank count " << opt_.rankCount);
            return BM_INVALID_PARAM;
        }
        if (kv.first == opt_.rankId) {
            continue;
        }
        net::Endpoint ep;
        if (!net::ParseUrl(kv.second.nic, &ep)) {
            MF_ERROR("host transport: rank " << kv.first << " has a malformed address '" << kv.second.nic << "'");
            return BM_INVALID_PARAM;
        }
        auto it = peers_.find(kv.first);
        if (it == peers_.end()) {
            auto p = std::make_shared<Peer>();
            p->info = kv.second;
            p->ep = ep;
            peers_[kv.first] = p;
            continue;
        }
        // A known rank: a key for an address already known replaces the old one (a restarted rank serves the same pool
        // addresses under new tokens), other keys are added; a new address makes the open link stale.
        std::lock_guard<std::mutex> lg(it->second->linkMu);
        const bool moved = it->second->info.nic != kv.second.nic;
        std::vector<MemoryKey> keys = it->second->info.keys;
        for (const auto &k : kv.second.keys) {
            bool replaced = false;
            for (auto &old : keys) {
                if (old.addr == k.addr) {
                    old = k;
                    replaced = true;
                }
            }
            if (!replaced) {
                keys.push_back(k);
            }
        }
        it->second->info = kv.second;
        it->second->info.keys = std::move(keys);
        it->second->ep = ep;
        if (moved) {
            it->second->stale.store(true);
        }
    }
    return BM_OK;
}

int HostTcpTransport::Prepare(const PrepareOptions &opt)
{
    if (!open_.load()) {
        return BM_NOT_INITIALIZED;
    }
    return ApplyRanks(opt, true);
}

int HostTcpTransport::UpdateRankOptions(const PrepareOptions &opt)
{
    if (!open_.load()) {
        return BM_NOT_INITIALIZED;
    }
    int rc = ApplyRanks(opt, false);
    return rc != BM_OK ? rc : ConnectAll();
}

int HostTcpTransport::RemoveRanks(const std::vector<uint32_t> &ranks)
{
    util::WriteGuard g(peerMu_);
    for (uint32_t r : ranks) {
        auto it = peers_.find(r);
        if (it == peers_.end()) {
            continue;
        }
        std::lock_guard<std::mutex> lg(it->second->linkMu);
        if (it->second->link) {
            it->second->link->SetBrokenHandler(nullptr);
            it->second->link->Close();
            it->second->link.reset();
        }
        peers_.erase(it);
    }
    return BM_OK;
}

int HostTcpTransport::EnsureLink(const std::shared_ptr<Peer> &p, uint32_t rankId, bool force)
{
    std::lock_guard<std::mutex> g(p->linkMu);
    if (!RolePermitsLink(opt_.role, p->info.role)) {
        MF_ERROR("host transport: a rank of role " << opt_.role << " does not open links to rank " << rankId << " of role " << p->info.role);
        return BM_INVALID_PARAM;
    }
    if (p->link && p->link->Connected() && !p->stale.load() && !force) {
        return BM_OK;
    }
    if (p->link) {
        p->link->SetBrokenHandler(nullptr);
        p->link->Close();
        p->link.reset();
        stats_.reconnects.fetch_add(1);
    }
    auto link = std::make_shared<net::RpcClient>();
    if (tlsClient_) {
        link->SetTls(tlsClient_);
    }
    if (link->Connect(p->ep, ((uint64_t)opt_.rankCount << 32) | opt_.rankId, 1, 0) != 0) {
        MF_WARN_LIMIT("host transport: cannot reach rank " << rankId << " at " << p->info.nic);
        return BM_ERROR;
    }
    std::weak_ptr<Peer> weak = p;
    link->SetBrokenHandler([this, weak, rankId]() {
        if (auto sp = weak.lock()) {
            sp->stale.store(true);
        }
        if (onBroken_) {
            onBroken_(rankId);
        }
    });
    p->link = link;
    p->stale.store(false);
    return BM_OK;
}

bool HostTcpTransport::Linked(uint32_t rankId)
{
    auto p = FindPeer(rankId);
    if (!p) {
        return false;
    }
    std::lock_guard<std::mutex> g(p->linkMu);
    return p->link && p->link->Connected() && !p->stale.load();
}

int HostTcpTransport::ConnectAll()
{
    std::vector<std::pair<uint32_t, std::shared_ptr<Peer>>> todo;
    {
        util::ReadGuard g(peerMu_);
        for (auto &kv : peers_) {
            if (RolePermitsLink(opt_.role, kv.second->info.role)) {
                todo.emplace_back(kv.first, kv.second);
            }
        }
    }
    int result = BM_OK;
    for (auto &t : todo) {
        int rc = BM_ERROR;
        RetryWithBackoff([&]() { return (rc = EnsureLink(t.second, t.first, false)) == BM_OK; }, [](uint32_t) {});
        if (rc != BM_OK) {
            MF_ERROR("host transport: no link to rank " << t.first << " at " << t.second->info.nic);
            result = rc;
        }
    }
    return result;
}

int HostTcpTransport::Connect()
{
    if (!open_.load()) {
        return BM_NOT_INITIALIZED;
    }
    return ConnectAll();
}

int HostTcpTransport::AsyncConnect()
{
    if (!open_.load()) {
        return BM_NOT_INITIALIZED;
    }
    std::lock_guard<std::mutex> g(connMu_);
    if (connecting_) {
        return BM_OK;
    }
    if (connector_.joinable()) {
        connector_.join();
    }
    connecting_ = true;
    connector_ = std::thread([this]() {
        int rc = ConnectAll();
        std::lock_guard<std::mutex> lg(connMu_);
        connectResult_ = rc;
        connecting_ = false;
        connCv_.notify_all();
    });
    return BM_OK;
}

int HostTcpTransport::WaitForConnected(int64_t timeoutNs)
{
    std::unique_lock<std::mutex> lk(connMu_);
    auto done = [this]() { return !connecting_; };
    if (timeoutNs < 0) {
        connCv_.wait(lk, done);
    } else if (!connCv_.wait_for(lk, std::chrono::nanoseconds(timeoutNs), done)) {
        return BM_TIMEOUT;
    }
    return connectResult_;
}

// ------------------------------------------------------------------------------------------------------ requesting side

int HostTcpTransport::RunSliceOnce(const Slice &s)
{
    std::shared_ptr<net::RpcClient> link;
    {
        std::lock_guard<std::mutex> g(s.peer->linkMu);
        link = s.peer->link;
    }
    if (!link) {
        return BM_ERROR;
    }
    OneSidedHeader h{s.token, s.remote, s.size};
    net::Frame reply;
    // A write's payload leaves from the caller's memory, a read's data arrives in it: no staging copy on this side.
    int rc = s.write ? link->CallGather(kMsgWrite, &h, sizeof(h), (const void *)s.local, s.size, nullptr, 0, &reply, opt_.opTimeoutMs)
                     : link->CallGather(kMsgRead, &h, sizeof(h), nullptr, 0, (void *)s.local, s.size, &reply, opt_.opTimeoutMs);
    if (rc == net::RPC_TIMEOUT) {
        return BM_TIMEOUT;
    }
    if (rc != net::RPC_OK) {
        return BM_ERROR;
    }
    if (reply.result != 0) {
        return BM_INVALID_PARAM;  // the owner refused: retrying cannot help
    }
    if (!s.write) {
        if (!reply.body.empty()) {  // not delivered in place (TLS session data interleaved, or an odd size): copy it over
            if (reply.body.size() != s.size) {
                return BM_ERROR;
            }
            std::memcpy((void *)s.local, reply.body.data(), s.size);
        }
        stats_.bytesRead.fetch_add(s.size);
    } else {
        stats_.bytesWritten.fetch_add(s.size);
    }
    return BM_OK;
}

int HostTcpTransport::RunSlice(const Slice &s)
{
    int rc = BM_ERROR;
    bool force = false;
    RetryWithBackoff(
        [&]() {
            rc = EnsureLink(s.peer, s.rank, force);
            if (rc == BM_OK) {
                rc = RunSliceOnce(s);
            }
            return rc == BM_OK || rc == BM_INVALID_PARAM;  // a refusal ends the attempts
        },
        [&](uint32_t) { force = true; });  // forced reconnect before every further attempt
    stats_.slices.fetch_add(1);
    return rc;
}

void HostTcpTransport::WorkerLoop()
{
    while (true) {
        Slice s;
        {
            std::unique_lock<std::mutex> lk(qMu_);
            qCv_.wait(lk, [this]() { return stopping_ || !queue_.empty(); });
            if (stopping_) {
                return;
            }
            s = queue_.front();
            queue_.pop_front();
        }
        s.peer->counter.Complete(RunSlice(s));
    }
}

// The access token of the peer's region that covers [remoteAddr, +size) with the access the operation needs; checks the role rule.
int HostTcpTransport::TokenFor(const std::shared_ptr<Peer> &p, uint32_t rankId, bool write, uint64_t remoteAddr, uint64_t size, uint64_t *token)
{
    *token = 0;
    {
        std::lock_guard<std::mutex> g(p->linkMu);
        if (!RolePermitsLink(opt_.role, p->info.role)) {
            MF_ERROR("host transport: role " << opt_.role << " may not address rank " << rankId << " of role " << p->info.role);
            return BM_INVALID_PARAM;
        }
        const uint32_t need = write ? MR_ACCESS_REMOTE_WRITE : MR_ACCESS_REMOTE_READ;
        for (const auto &k : p->info.keys) {
            if (k.Covers(remoteAddr, size) && (k.access & need) != 0) {
                *token = k.token;
                break;
            }
        }
    }
    if (*token == 0) {
        MF_ERROR("host transport: rank " << rankId << " has no region that covers 0x" << std::hex << remoteAddr << "+0x" << size << std::dec
                                         << " with the access asked for");
        return BM_INVALID_PARAM;
    }
    return BM_OK;
}

// A blocking operation of at most one slice, with nothing queued before it for that peer, runs on the caller's thread: two
// thread hand-overs (to a worker and back) are most of the latency of a small transfer. Everything else is queued and waited for.
int HostTcpTransport::Blocking(uint32_t rankId, bool write, uint64_t localAddr, uint64_t remoteAddr, uint64_t size)
{
    if (open_.load() && rankId != opt_.rankId && localAddr != 0 && remoteAddr != 0 && size != 0 && size <= opt_.sliceBytes &&
        remoteAddr + size >= remoteAddr) {
        auto p = FindPeer(rankId);
        if (p && p->counter.Idle()) {
            uint64_t token = 0;
            int rc = TokenFor(p, rankId, write, remoteAddr, size, &token);
            if (rc != BM_OK) {
                return rc;
            }
            return RunSlice(Slice{p, rankId, write, localAddr, remoteAddr, size, token});
        }
    }
    int rc = Submit(rankId, write, localAddr, remoteAddr, size);
    return rc != BM_OK ? rc : Synchronize(rankId);
}

int HostTcpTransport::Submit(uint32_t rankId, bool write, uint64_t localAddr, uint64_t remoteAddr, uint64_t size)
{
    if (!open_.load()) {
        return BM_NOT_INITIALIZED;
    }
    if (localAddr == 0 || remoteAddr == 0 || size == 0 || remoteAddr + size < remoteAddr) {
        return BM_INVALID_PARAM;
    }
    if (rankId == opt_.rankId) {  // own memory: no wire
        MemoryKey own;
        if (!QueryHasRegistered(remoteAddr, size) || QueryMemoryKey(remoteAddr, &own) != BM_OK) {
            return BM_INVALID_PARAM;
        }
        if ((own.flags & MR_FLAG_HBM) != 0) {
            if (!deviceCopier_) {
                return BM_INVALID_PARAM;
            }
            return write ? deviceCopier_((void *)remoteAddr, (const void *)localAddr, size) : deviceCopier_((void *)localAddr, (const void *)remoteAddr, size);
        }
        if (write) {
            std::memcpy((void *)remoteAddr, (const void *)localAddr, size);
        } else {
            std::memcpy((void *)localAddr, (const void *)remoteAddr, size);
        }
        return BM_OK;
    }
    auto p = FindPeer(rankId);
    if (!p) {
        MF_ERROR("host transport: rank " << rankId << " is not known (Prepare / UpdateRankOptions first)");
        return BM_INVALID_PARAM;
    }
    uint64_t token = 0;
    int trc = TokenFor(p, rankId, write, remoteAddr, size, &token);
    if (trc != BM_OK) {
        return trc;
    }
    const uint64_t step = opt_.sliceBytes;
    const uint64_t pieces = (size + step - 1) / step;
    p->counter.Submit(pieces);
    {
        std::lock_guard<std::mutex> g(qMu_);
        for (uint64_t off = 0; off < size; off += step) {
            queue_.push_back(Slice{p, rankId, write, localAddr + off, remoteAddr + off, std::min(step, size - off), token});
        }
    }
    if (pieces > 1) {
        qCv_.notify_all();
    } else {
        qCv_.notify_one();
    }
    return BM_OK;
}

int HostTcpTransport::Synchronize(uint32_t rankId)
{
    if (rankId == opt_.rankId) {
        return BM_OK;
    }
    auto p = FindPeer(rankId);
    if (!p) {
        return BM_INVALID_PARAM;
    }
    // Long enough for every attempt of the retry policy to run its course.
    const RetryPolicy pol = GlobalRetryPolicy();
    int64_t limit = 1000;
    for (uint32_t a = 0; a < pol.attempts; a++) {
        limit += opt_.opTimeoutMs + (a > 0 ? pol.DelayMs(a) : 0);
    }
    return p->counter.Synchronize(limit, BM_TIMEOUT);
}

int HostTcpTransport::WriteRemoteAsync(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size)
{
    return Submit(rankId, true, localAddr, remoteAddr, size);
}

int HostTcpTransport::ReadRemoteAsync(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size)
{
    return Submit(rankId, false, localAddr, remoteAddr, size);
}

int HostTcpTransport::WriteRemote(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size)
{
    return Blocking(rankId, true, localAddr, remoteAddr, size);
}

int HostTcpTransport::ReadRemote(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size)
{
    return Blocking(rankId, false, localAddr, remoteAddr, size);
}

}  // namespace transport
}  // namespace mf
