// Transport layer: how bytes reach memory that is not mapped into this process.
//
// Same contract as the reference's TransportManager (src/hybm/csrc/transport/hybm_transport_manager.h:25-117: open a
// device/NIC, register memory regions and hand out keys, prepare with every rank's address + keys, connect, update the rank
// set later, one-sided read/write in blocking and asynchronous form with a per-rank synchronise, batched forms) with three
// implementations chosen for an NVLink machine:
//   * DevicePeerTransport (mf_peer_link_manager.h)  - GPU memory of peers in the NVSwitch domain: "connect" is mapping the
//     peer's exported allocation, "write" is a copy kernel on peer pointers. Keeps the per-peer link state and applies the
//     role rule (a sender maps receivers only; the reference's bipartite QP manager,
//     src/hybm/csrc/transport/device/bipartite_ranks_qp_manager.cpp).
//   * HostTcpTransport (mf_host_tcp_transport.h)     - host memory of ranks on ANOTHER host: one-sided put/get served by a
//     small TCP server next to the registered regions, sliced and pipelined, with the reference's retry policy
//     (src/hybm/csrc/transport/host/host_hcom_transport_manager.cpp:529-660, 865-883).
//   * ComposeTransport (mf_compose_transport.h)      - owns one of each and routes every call by the memory kind of the
//     region or of the remote address (src/hybm/csrc/transport/compose/compose_transport_manager.cpp).
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "../hybm/mf_hybm_types.h"
#include "../net/mf_tls.h"

namespace mf {
namespace transport {

enum TransportType : uint32_t { TT_DEVICE_PEER = 0, TT_HOST_TCP = 1, TT_COMPOSE = 2 };

constexpr uint32_t MR_FLAG_DRAM = 0x1;
constexpr uint32_t MR_FLAG_HBM = 0x2;
constexpr uint32_t MR_ACCESS_LOCAL_WRITE = 0x1;
constexpr uint32_t MR_ACCESS_REMOTE_WRITE = 0x2;
constexpr uint32_t MR_ACCESS_REMOTE_READ = 0x4;
constexpr uint32_t MR_ACCESS_ALL = 0x7;

struct Options {
    uint32_t rankId{0};
    uint32_t rankCount{1};
    hybm::Role role{hybm::ROLE_PEER};
    std::string nic;            // host transport: "ip:port" / "tcp://ip:port" to serve on (port 0 = any free port)
    uint32_t workers{4};        // host transport: threads that carry asynchronous slices
    uint64_t sliceBytes{4ull << 20};
    int64_t opTimeoutMs{30000};
    net::TlsOptions tls;        // host transport: TLS 1.3 on its links when enabled
};

struct MemoryRegion {
    uint64_t addr{0};
    uint64_t size{0};
    uint32_t access{MR_ACCESS_ALL};
    uint32_t flags{0};
};

// What a peer needs to address a registered region. POD so it travels inside exchange blobs and store records.
struct MemoryKey {
    uint64_t token{0};  // random per registration; a request must present it
    uint64_t addr{0};
    uint64_t size{0};
    uint32_t access{0};
    uint32_t flags{0};
    bool Covers(uint64_t a, uint64_t n) const { return size != 0 && a >= addr && n <= size && a - addr <= size - n; }
};
static_assert(sizeof(MemoryKey) == 32, "memory key is 32 bytes on the wire");

struct RankInfo {
    std::string nic;
    hybm::Role role{hybm::ROLE_PEER};
    bool sameHost{true};  // false: the rank is outside this host's NVSwitch domain, so even its device memory goes over the wire
    std::vector<MemoryKey> keys;
};

struct PrepareOptions {
    std::unordered_map<uint32_t, RankInfo> ranks;
};

// A list of (local, remote, size) pieces that go to one rank.
struct CopyBatch {
    std::vector<uint64_t> local;
    std::vector<uint64_t> remote;
    std::vector<uint64_t> sizes;
};

// The role rule shared by every transport: peers link with everybody; a sender and a receiver link with each other and with
// peers; two senders, or two receivers, never link (neither maps the other's memory nor addresses it).
inline bool RolePermitsLink(hybm::Role mine, hybm::Role theirs)
{
    return mine == hybm::ROLE_PEER || theirs == hybm::ROLE_PEER || mine != theirs;
}

class TransportManager {
public:
    static std::shared_ptr<TransportManager> Create(TransportType type);
    virtual ~TransportManager() = default;

    virtual int OpenDevice(const Options &opt) = 0;
    virtual int CloseDevice() = 0;

    virtual int RegisterMemoryRegion(const MemoryRegion &mr) = 0;
    virtual int UnregisterMemoryRegion(uint64_t addr) = 0;
    virtual bool QueryHasRegistered(uint64_t addr, uint64_t size) = 0;
    virtual int QueryMemoryKey(uint64_t addr, MemoryKey *key) = 0;

    // Records every rank's address, role and keys. Nothing is contacted yet.
    virtual int Prepare(const PrepareOptions &opt) = 0;
    // Opens the links the role rule allows. Blocking.
    virtual int Connect() = 0;
    virtual int AsyncConnect() = 0;
    virtual int WaitForConnected(int64_t timeoutNs) = 0;
    // After Connect: adds ranks, replaces the records of known ones (a restarted peer has new keys), keeps the others.
    virtual int UpdateRankOptions(const PrepareOptions &opt) = 0;
    virtual int RemoveRanks(const std::vector<uint32_t> &ranks) = 0;

    // Address peers use to reach this rank ("ip:port" for the host transport, "" for device links).
    virtual std::string GetNic() const = 0;

    // One-sided copies between local memory and a region the rank `rankId` registered. Blocking forms return when the bytes
    // are in place; asynchronous forms return once queued and complete by Synchronize(rankId), which reports the first
    // failure since the previous call.
    virtual int ReadRemote(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) = 0;
    virtual int WriteRemote(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) = 0;
    virtual int ReadRemoteAsync(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) = 0;
    virtual int WriteRemoteAsync(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) = 0;
    virtual int Synchronize(uint32_t rankId) = 0;
    virtual int ReadRemoteBatchAsync(uint32_t rankId, const CopyBatch &batch);
    virtual int WriteRemoteBatchAsync(uint32_t rankId, const CopyBatch &batch);
};

using TransportPtr = std::shared_ptr<TransportManager>;

}  // namespace transport
}  // namespace mf
