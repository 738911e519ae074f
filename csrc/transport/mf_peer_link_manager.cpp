#include "mf_peer_link_manager.h"

#include "../util/mf_log.h"

namespace mf {
namespace transport {

using hybm::BM_ERROR;
using hybm::BM_INVALID_PARAM;
using hybm::BM_NOT_INITIALIZED;
using hybm::BM_NOT_SUPPORTED;
using hybm::BM_OK;

const char *LinkStateName(LinkState s)
{
    switch (s) {
        case LINK_NONE: return "none";
        case LINK_KNOWN: return "known";
        case LINK_IMPORTED: return "imported";
        case LINK_MAPPED: return "mapped";
        case LINK_REMOTE: return "remote";
        case LINK_REFUSED: return "refused";
        case LINK_STALE: return "stale";
        case LINK_REMOVED: return "removed";
    }
    return "?";
}

void PeerLinkManager::SetSelf(uint32_t rank, hybm::Role role, const std::string &hostId)
{
    std::lock_guard<std::mutex> g(mu_);
    self_ = rank;
    role_ = role;
    hostId_ = hostId;
}

void PeerLinkManager::SetState(PeerLink &l, LinkState s)
{
    if (l.state != s) {
        l.state = s;
        l.changes++;
    }
}

void PeerLinkManager::NoteIdentity(uint32_t rank, hybm::Role role, const std::string &hostId)
{
    std::lock_guard<std::mutex> g(mu_);
    PeerLink &l = links_[rank];
    const bool fresh = l.state == LINK_NONE || l.state == LINK_REMOVED || l.state == LINK_STALE;
    const std::string host = hostId.empty() && !fresh ? l.hostId : hostId;  // a caller that only knows the role keeps the host
    const bool changed = !fresh && (l.role != role || l.hostId != host);
    if (fresh || changed) {
        l.slices = l.remoteSlices = 0;
        l.bytes = 0;
    }
    l.rank = rank;
    l.role = role;
    l.hostId = host;
    l.sameHost = host.empty() || host == hostId_;
    if (!RolePermitsLink(role_, role)) {
        SetState(l, LINK_REFUSED);
    } else if (fresh || changed || l.state == LINK_REFUSED) {
        SetState(l, LINK_KNOWN);
    }
}

bool PeerLinkManager::Permits(uint32_t rank)
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = links_.find(rank);
    return it == links_.end() || RolePermitsLink(role_, it->second.role);
}

bool PeerLinkManager::SameHost(uint32_t rank)
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = links_.find(rank);
    return it == links_.end() || it->second.sameHost;
}

LinkState PeerLinkManager::NoteSlice(uint32_t rank, uint64_t bytes, bool remote)
{
    std::lock_guard<std::mutex> g(mu_);
    PeerLink &l = links_[rank];
    l.rank = rank;
    if (l.state == LINK_REFUSED) {
        return l.state;
    }
    l.slices++;
    l.bytes += bytes;
    if (remote) {
        l.remoteSlices++;
        l.sameHost = false;
        SetState(l, LINK_REMOTE);
    } else if (l.state != LINK_REMOTE) {
        SetState(l, LINK_IMPORTED);
    }
    return l.state;
}

void PeerLinkManager::NoteMapped()
{
    std::lock_guard<std::mutex> g(mu_);
    for (auto &kv : links_) {
        if (kv.second.state == LINK_IMPORTED) {
            SetState(kv.second, LINK_MAPPED);
        }
    }
}

void PeerLinkManager::NoteStale(uint32_t rank)
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = links_.find(rank);
    if (it != links_.end() && it->second.state != LINK_REMOVED) {
        SetState(it->second, LINK_STALE);
    }
}

void PeerLinkManager::NoteRemoved(uint32_t rank)
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = links_.find(rank);
    if (it != links_.end()) {
        it->second.slices = it->second.remoteSlices = 0;
        it->second.bytes = 0;
        SetState(it->second, LINK_REMOVED);
    }
}

LinkState PeerLinkManager::StateOf(uint32_t rank)
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = links_.find(rank);
    return it == links_.end() ? LINK_NONE : it->second.state;
}

std::vector<PeerLink> PeerLinkManager::Snapshot()
{
    std::lock_guard<std::mutex> g(mu_);
    std::vector<PeerLink> out;
    for (auto &kv : links_) {
        out.push_back(kv.second);
    }
    return out;
}

std::vector<uint32_t> PeerLinkManager::RanksIn(LinkState s)
{
    std::lock_guard<std::mutex> g(mu_);
    std::vector<uint32_t> out;
    for (auto &kv : links_) {
        if (kv.second.state == s) {
            out.push_back(kv.first);
        }
    }
    return out;
}

// ------------------------------------------------------------------------------------------------ DevicePeerTransport

int DevicePeerTransport::OpenDevice(const Options &opt)
{
    if (opt.rankCount == 0 || opt.rankId >= opt.rankCount) {
        return BM_INVALID_PARAM;
    }
    opt_ = opt;
    links_.SetSelf(opt.rankId, opt.role, "");
    open_ = true;
    return BM_OK;
}

int DevicePeerTransport::CloseDevice()
{
    if (!open_) {
        return BM_OK;
    }
    std::vector<uint32_t> all;
    {
        util::ReadGuard g(mu_);
        for (auto &kv : ranks_) {
            all.push_back(kv.first);
        }
    }
    RemoveRanks(all);
    util::WriteGuard g(mu_);
    regions_.clear();
    open_ = false;
    return BM_OK;
}

int DevicePeerTransport::RegisterMemoryRegion(const MemoryRegion &mr)
{
    if (mr.addr == 0 || mr.size == 0) {
        return BM_INVALID_PARAM;
    }
    util::WriteGuard g(mu_);
    MemoryKey k;
    k.token = mr.addr;  // device links need no secret: the mapping itself is the capability
    k.addr = mr.addr;
    k.size = mr.size;
    k.access = mr.access;
    k.flags = mr.flags == 0 ? MR_FLAG_HBM : mr.flags;
    regions_[mr.addr] = k;
    return BM_OK;
}

int DevicePeerTransport::UnregisterMemoryRegion(uint64_t addr)
{
    util::WriteGuard g(mu_);
    return regions_.erase(addr) == 1 ? BM_OK : BM_INVALID_PARAM;
}

bool DevicePeerTransport::QueryHasRegistered(uint64_t addr, uint64_t size)
{
    util::ReadGuard g(mu_);
    auto it = regions_.upper_bound(addr);
    if (it == regions_.begin()) {
        return false;
    }
    --it;
    return it->second.Covers(addr, size);
}

int DevicePeerTransport::QueryMemoryKey(uint64_t addr, MemoryKey *key)
{
    if (key == nullptr) {
        return BM_INVALID_PARAM;
    }
    util::ReadGuard g(mu_);
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

int DevicePeerTransport::Prepare(const PrepareOptions &opt)
{
    if (!open_) {
        return BM_NOT_INITIALIZED;
    }
    util::WriteGuard g(mu_);
    ranks_.clear();
    for (auto &kv : opt.ranks) {
        if (kv.first >= opt_.rankCount) {
            return BM_INVALID_PARAM;
        }
        if (kv.first == opt_.rankId) {
            continue;
        }
        ranks_[kv.first] = kv.second;
        links_.NoteIdentity(kv.first, kv.second.role, "");
    }
    return BM_OK;
}

int DevicePeerTransport::Connect()
{
    if (!open_) {
        return BM_NOT_INITIALIZED;
    }
    std::vector<uint32_t> todo;
    {
        util::ReadGuard g(mu_);
        for (auto &kv : ranks_) {
            if (links_.Permits(kv.first)) {
                todo.push_back(kv.first);
            }
        }
    }
    connectResult_ = BM_OK;
    for (uint32_t r : todo) {
        LinkState st = links_.StateOf(r);
        if (st == LINK_MAPPED) {
            continue;
        }
        int rc = hooks_.mapPeer ? hooks_.mapPeer(r) : BM_OK;
        if (rc != BM_OK) {
            MF_ERROR("device links: mapping rank " << r << " failed (" << rc << ")");
            connectResult_ = rc;
            continue;
        }
        links_.NoteSlice(r, 0, false);
    }
    links_.NoteMapped();
    return connectResult_;
}

int DevicePeerTransport::UpdateRankOptions(const PrepareOptions &opt)
{
    if (!open_) {
        return BM_NOT_INITIALIZED;
    }
    {
        util::WriteGuard g(mu_);
        for (auto &kv : opt.ranks) {
            if (kv.first >= opt_.rankCount) {
                return BM_INVALID_PARAM;
            }
            if (kv.first == opt_.rankId) {
                continue;
            }
            ranks_[kv.first] = kv.second;
            links_.NoteIdentity(kv.first, kv.second.role, "");
        }
    }
    // A peer that went stale is unmapped before it is mapped again: its old allocation is gone.
    for (uint32_t r : links_.RanksIn(LINK_STALE)) {
        if (hooks_.unmapPeer) {
            hooks_.unmapPeer(r);
        }
        links_.NoteRemoved(r);
        links_.NoteIdentity(r, ranks_.count(r) ? ranks_[r].role : hybm::ROLE_PEER, "");
    }
    return Connect();
}

int DevicePeerTransport::RemoveRanks(const std::vector<uint32_t> &ranks)
{
    for (uint32_t r : ranks) {
        {
            util::WriteGuard g(mu_);
            ranks_.erase(r);
        }
        LinkState st = links_.StateOf(r);
        if ((st == LINK_MAPPED || st == LINK_STALE || st == LINK_IMPORTED) && hooks_.unmapPeer) {
            hooks_.unmapPeer(r);
        }
        links_.NoteRemoved(r);
    }
    return BM_OK;
}

int DevicePeerTransport::Copy(uint32_t rankId, uint64_t dst, uint64_t src, uint64_t remoteAddr, uint64_t size, bool write, bool async)
{
    if (!open_) {
        return BM_NOT_INITIALIZED;
    }
    if (dst == 0 || src == 0 || size == 0) {
        return BM_INVALID_PARAM;
    }
    if (rankId != opt_.rankId) {
        LinkState st = links_.StateOf(rankId);
        if (st != LINK_MAPPED) {
            MF_ERROR("device links: rank " << rankId << " is " << LinkStateName(st) << ", not mapped");
            return st == LINK_REFUSED ? BM_INVALID_PARAM : BM_ERROR;
        }
        util::ReadGuard g(mu_);
        auto it = ranks_.find(rankId);
        bool covered = false;
        const uint32_t need = write ? MR_ACCESS_REMOTE_WRITE : MR_ACCESS_REMOTE_READ;
        if (it != ranks_.end()) {
            for (auto &k : it->second.keys) {
                covered = covered || (k.Covers(remoteAddr, size) && (k.access & need) != 0);
            }
        }
        if (!covered) {
            MF_ERROR("device links: rank " << rankId << " exported nothing that covers 0x" << std::hex << remoteAddr << "+0x" << size << std::dec);
            return BM_INVALID_PARAM;
        }
    }
    if (!hooks_.copy) {
        return BM_NOT_SUPPORTED;
    }
    return hooks_.copy(dst, src, size, async);
}

int DevicePeerTransport::ReadRemote(uint32_t r, uint64_t l, uint64_t ra, uint64_t n) { return Copy(r, l, ra, ra, n, false, false); }
int DevicePeerTransport::WriteRemote(uint32_t r, uint64_t l, uint64_t ra, uint64_t n) { return Copy(r, ra, l, ra, n, true, false); }
int DevicePeerTransport::ReadRemoteAsync(uint32_t r, uint64_t l, uint64_t ra, uint64_t n) { return Copy(r, l, ra, ra, n, false, true); }
int DevicePeerTransport::WriteRemoteAsync(uint32_t r, uint64_t l, uint64_t ra, uint64_t n) { return Copy(r, ra, l, ra, n, true, true); }

int DevicePeerTransport::Synchronize(uint32_t)
{
    return hooks_.sync ? hooks_.sync() : BM_OK;
}

}  // namespace transport
}  // namespace mf
