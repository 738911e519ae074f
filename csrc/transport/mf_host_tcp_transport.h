// One-sided put/get on host memory of ranks that live on another host, over TCP.
//
// Every rank serves its registered regions: a small request server answers READ (token, address, size → bytes) and WRITE
// (token, address, bytes → ack) after checking that the range lies inside a registered region, that the token matches and
// that the region allows the access. The requesting side cuts a transfer into slices, runs the slices on a worker pool over
// one pipelined link per peer, and counts completions per peer (CounterStream), so a large transfer keeps several requests
// in flight and the asynchronous forms cost nothing until Synchronize. A failed slice is retried under the process-wide
// retry policy (three attempts, pauses of 1 s and 2 s by default) with the link closed and opened again in between; a link
// that breaks marks the peer so that the next operation reconnects first. Role of the reference's host transport over its
// RDMA library (src/hybm/csrc/transport/host/host_hcom_transport_manager.cpp: registration :246-330, sliced asynchronous
// put/get :529-660, retry with forced reconnect :865-883 and :959-977, broken-channel handler :1010-1030), with sockets
// standing in for the RDMA verbs that do not exist on this platform's hosts.
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <map>
#include <mutex>
#include <thread>

#include "../net/mf_rpc.h"
#include "../util/mf_sync.h"
#include "mf_counter_stream.h"
#include "mf_transport.h"

namespace mf {
namespace transport {

struct HostTcpStats {
    std::atomic<uint64_t> bytesWritten{0};   // payload bytes this rank put into peers
    std::atomic<uint64_t> bytesRead{0};      // payload bytes this rank got from peers
    std::atomic<uint64_t> bytesServed{0};    // payload bytes peers read from / wrote into this rank
    std::atomic<uint64_t> slices{0};
    std::atomic<uint64_t> reconnects{0};
    std::atomic<uint64_t> refused{0};        // requests this rank's server refused (bad token, range or access)
};

class HostTcpTransport : public TransportManager {
public:
    HostTcpTransport();
    ~HostTcpTransport() override;

    int OpenDevice(const Options &opt) override;
    int CloseDevice() override;
    int RegisterMemoryRegion(const MemoryRegion &mr) override;
    int UnregisterMemoryRegion(uint64_t addr) override;
    bool QueryHasRegistered(uint64_t addr, uint64_t size) override;
    int QueryMemoryKey(uint64_t addr, MemoryKey *key) override;
    int Prepare(const PrepareOptions &opt) override;
    int Connect() override;
    int AsyncConnect() override;
    int WaitForConnected(int64_t timeoutNs) override;
    int UpdateRankOptions(const PrepareOptions &opt) override;
    int RemoveRanks(const std::vector<uint32_t> &ranks) override;
    std::string GetNic() const override { return nic_; }
    int ReadRemote(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) override;
    int WriteRemote(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) override;
    int ReadRemoteAsync(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) override;
    int WriteRemoteAsync(uint32_t rankId, uint64_t localAddr, uint64_t remoteAddr, uint64_t size) override;
    int Synchronize(uint32_t rankId) override;

    const HostTcpStats &Stats() const { return stats_; }
    // Called (on an internal thread) when the link to a rank breaks; the peer stays known and is reconnected on next use.
    void SetBrokenHandler(std::function<void(uint32_t rank)> cb) { onBroken_ = std::move(cb); }
    // True if a link to the rank is currently open.
    bool Linked(uint32_t rankId);
    // Regions flagged MR_FLAG_HBM are device memory: the serving thread cannot memcpy them, it calls this instead
    // (dst, src, bytes) -> 0 on success; one side is the region, the other an ordinary host buffer. Without a copier such
    // regions are refused.
    void SetDeviceCopier(std::function<int(void *dst, const void *src, size_t n)> fn) { deviceCopier_ = std::move(fn); }

private:
    struct Peer {
        RankInfo info;
        net::Endpoint ep;
        std::shared_ptr<net::RpcClient> link;
        std::mutex linkMu;  // serialises connect / reconnect of this peer
        std::atomic<bool> stale{false};
        CounterStream counter;
    };
    struct Slice {
        std::shared_ptr<Peer> peer;
        uint32_t rank;
        bool write;
        uint64_t local, remote, size, token;
    };

    void OnRequest(net::LinkId link, const net::Frame &f);
    std::shared_ptr<Peer> FindPeer(uint32_t rankId);
    int EnsureLink(const std::shared_ptr<Peer> &p, uint32_t rankId, bool force);
    int Submit(uint32_t rankId, bool write, uint64_t localAddr, uint64_t remoteAddr, uint64_t size);
    int Blocking(uint32_t rankId, bool write, uint64_t localAddr, uint64_t remoteAddr, uint64_t size);
    int TokenFor(const std::shared_ptr<Peer> &p, uint32_t rankId, bool write, uint64_t remoteAddr, uint64_t size, uint64_t *token);
    int RunSlice(const Slice &s);
    int RunSliceOnce(const Slice &s);
    void WorkerLoop();
    int ApplyRanks(const PrepareOptions &opt, bool replaceAll);
    int ConnectAll();

    Options opt_;
    std::string nic_;
    std::atomic<bool> open_{false};
    net::RpcServer server_;
    std::shared_ptr<net::TlsContext> tlsClient_;

    util::RwLock regionMu_;
    std::map<uint64_t, MemoryKey> regions_;  // by base address

    util::RwLock peerMu_;
    std::unordered_map<uint32_t, std::shared_ptr<Peer>> peers_;

    std::mutex qMu_;
    std::condition_variable qCv_;
    std::deque<Slice> queue_;
    std::vector<std::thread> workers_;
    bool stopping_{false};

    std::thread connector_;
    std::mutex connMu_;
    std::condition_variable connCv_;
    bool connecting_{false};
    int connectResult_{0};

    HostTcpStats stats_;
    std::function<void(uint32_t)> onBroken_;
    std::function<int(void *, const void *, size_t)> deviceCopier_;
};

}  // namespace transport
}  // namespace mf
