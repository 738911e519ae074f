// Per-peer link state of an entity, and the device-memory transport built on it.
//
// PeerLinkManager is the table an entity keeps about every other rank: its role, whether it shares this host (and so the
// NVSwitch domain and the host's shared memory), how many of its slices are known, mapped or only reachable through the host
// transport, and when that last changed. It answers the two questions the import path asks - "may this rank's memory be
// linked at all?" (the role rule) and "can it be mapped, or must it be reached over the wire?" - and is what diagnostics
// print. Role of the reference's per-rank connection records (src/hybm/csrc/transport/device/device_qp_manager.h and its
// fixed / joinable / bipartite subclasses), where a "connection" is a queue pair; here it is a mapping.
//
// DevicePeerTransport puts the TransportManager interface over device memory in the NVSwitch domain: a region is an exported
// allocation, connecting to a rank is mapping what it exported, a remote write is a copy on peer pointers. The mapping and
// the copy are supplied by the owner (the entity) as hooks, so the class itself holds no CUDA state.
#pragma once
#include <functional>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../util/mf_sync.h"
#include "mf_transport.h"

namespace mf {
namespace transport {

enum LinkState : uint32_t {
    LINK_NONE = 0,      // never heard of
    LINK_KNOWN = 1,     // identity (role, host) known, no memory yet
    LINK_IMPORTED = 2,  // slices recorded, not mapped
    LINK_MAPPED = 3,    // slices mapped into this process
    LINK_REMOTE = 4,    // lives on another host: reached through the host transport, never mapped
    LINK_REFUSED = 5,   // the role rule forbids a link
    LINK_STALE = 6,     // the peer went away; what was mapped must not be used and is dropped on the next update
    LINK_REMOVED = 7,
};
const char *LinkStateName(LinkState s);

struct PeerLink {
    uint32_t rank{0};
    hybm::Role role{hybm::ROLE_PEER};
    std::string hostId;
    bool sameHost{true};
    LinkState state{LINK_NONE};
    uint32_t slices{0};
    uint32_t remoteSlices{0};
    uint64_t bytes{0};
    uint64_t changes{0};  // how many times the state changed
};

class PeerLinkManager {
public:
    void SetSelf(uint32_t rank, hybm::Role role, const std::string &hostId);
    // Identity of a peer, from its entity export. A peer that comes back with another host id or role starts afresh.
    void NoteIdentity(uint32_t rank, hybm::Role role, const std::string &hostId);
    // Role rule. Unknown peers are permitted (their role is learned with their first export).
    bool Permits(uint32_t rank);
    bool SameHost(uint32_t rank);
    // A slice of `rank` was recorded; remote = it cannot be mapped here. Returns the state the link is in afterwards.
    LinkState NoteSlice(uint32_t rank, uint64_t bytes, bool remote);
    void NoteMapped();  // every imported same-host link becomes mapped
    void NoteStale(uint32_t rank);
    void NoteRemoved(uint32_t rank);
    LinkState StateOf(uint32_t rank);
    std::vector<PeerLink> Snapshot();
    std::vector<uint32_t> RanksIn(LinkState s);

private:
    void SetState(PeerLink &l, LinkState s);
    std::mutex mu_;
    uint32_t self_{0};
    hybm::Role role_{hybm::ROLE_PEER};
    std::string hostId_;
    std::map<uint32_t, PeerLink> links_;
};

struct DeviceHooks {
    // Maps everything the rank exported (idempotent). 0 on success.
    std::function<int(uint32_t rank)> mapPeer;
    std::function<int(uint32_t rank)> unmapPeer;
    // Copy between two addresses this process can dereference (local or mapped peer memory); async = do not wait.
    std::function<int(uint64_t dst, uint64_t src, uint64_t size, bool async)> copy;
    std::function<int()> sync;
};

class DevicePeerTransport : public TransportManager {
public:
    explicit DevicePeerTransport(DeviceHooks hooks = {}) : hooks_(std::move(hooks)) {}
    void SetHooks(DeviceHooks hooks) { hooks_ = std::move(hooks); }
    PeerLinkManager &Links() { return links_; }

    int OpenDevice(const Options &opt) override;
    int CloseDevice() override;
    int RegisterMemoryRegion(const MemoryRegion &mr) override;
    int UnregisterMemoryRegion(uint64_t addr) override;
    bool QueryHasRegistered(uint64_t addr, uint64_t size) override;
    int QueryMemoryKey(uint64_t addr, MemoryKey *key) override;
    int Prepare(const PrepareOptions &opt) override;
    int Connect() override;
    int AsyncConnect() override { return Connect(); }
    int WaitForConnected(int64_t) override { return connectResult_; }
    int UpdateRankOptions(const PrepareOptions &opt) override;
    int RemoveRanks(const std::vector<uint32_t> &ranks) override;
    std::string GetNic() const override { return ""; }
    int ReadRemote(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) override;
    int WriteRemote(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) override;
    int ReadRemoteAsync(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) override;
    int WriteRemoteAsync(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) override;
    int Synchronize(uint32_t rankId) override;

private:
    int Copy(uint32_t rankId, uint64_t dst, uint64_t src, uint64_t remoteAddr, uint64_t size, bool write, bool async);
    DeviceHooks hooks_;
    Options opt_;
    bool open_{false};
    int connectResult_{0};
    PeerLinkManager links_;
    util::RwLock mu_;
    std::map<uint64_t, MemoryKey> regions_;
    std::map<uint32_t, RankInfo> ranks_;
};

}  // namespace transport
}  // namespace mf
