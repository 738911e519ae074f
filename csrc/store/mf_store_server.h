// Store server: serves the key-value protocol of mf_store.h over mf::net::RpcServer.
//
// Behaviour follows the reference server (src/smem/csrc/config_store/tcp_store/smem_tcp_config_store_server.cpp):
// blocked GETs parked per key and woken by SET/ADD/APPEND/CAS (:257-303,356-428), a timer that answers TIMEOUT
// (:798-830), auto-ranking through keys prefixed "AutoRanking#" (:305-354), heartbeat supervision — a link is
// declared dead after more than 3 missed intervals (:865-887) — rank-down notification to subscribers (:832-863),
// and "clear everything when the last client leaves" (:203-245). Unlike the reference, waiters parked by a dead
// link are removed eagerly. Per-op hooks and a link-broken hook let a fault handler observe traffic.
#pragma once
#include <atomic>
#include <condition_variable>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <thread>
#include <unordered_map>

#include "../net/mf_rpc.h"
#include "mf_store.h"
#include "mf_store_backend.h"

namespace mf {
namespace store {

struct ServerTiming {
    uint32_t heartbeatIntervalMs{2000};  // clients send at this period
    uint32_t heartbeatMissLimit{3};      // link is dead after more than this many silent intervals
    uint32_t serverLingerMs{1500};       // on shutdown the hosting process waits this long for the other clients to leave first
};
// Process-wide timing (tests shorten it; MF_STORE_HEARTBEAT_MS overrides the interval).
ServerTiming &GlobalTiming();

class StoreServer {
public:
    // Hook called after the server handled `op` for `link`. For GET misses the hook may fill *reply and return
    // ST_RESTORE (or ST_OK) to answer the request itself; any other return means "not handled".
    using OpHook = std::function<int(uint16_t op, net::LinkId link, const std::string &key, const std::string &value, std::string *reply)>;
    using BrokenHook = std::function<void(net::LinkId link, StoreBackend *backend)>;

    StoreServer();
    ~StoreServer();
    // worldSize 0 = unbounded auto-ranking range. Returns 0, or -EADDRINUSE etc.
    int Start(const net::Endpoint &ep, uint32_t worldSize = 0);
    void Stop();
    uint16_t Port() const { return rpc_.Port(); }
    bool Running() const { return rpc_.Running(); }
    void SetOpHook(OpHook h) { opHook_ = std::move(h); }
    void SetBrokenHook(BrokenHook h) { brokenHook_ = std::move(h); }
    StoreBackend *Backend() { return backend_.get(); }
    size_t AliveLinks();
    // Test hook: stop answering (simulates a hung server without closing sockets).
    void SetMute(bool m) { mute_.store(m); }

private:
    struct Waiter {
        net::LinkId link;
        uint32_t seq;
        uint64_t deadlineMs;  // 0 = none
        uint64_t id;
    };
    void OnMessage(net::LinkId link, const net::Frame &f);
    bool OnLinkUp(net::LinkId link, uint64_t peerId);
    void OnLinkDown(net::LinkId link);
    void Reply(net::LinkId link, const net::Frame &req, int result, const std::string &value);
    void ReplyText(net::LinkId link, uint32_t seq, uint16_t type, int result, const std::string &value);
    void WakeWaiters(const std::string &key, const std::string &value);
    void HandleGet(net::LinkId link, const net::Frame &f, const StoreMessage &m);
    void HandleRendezvous(net::LinkId link, const net::Frame &f, const StoreMessage &m);
    int AssignRank(net::LinkId link, const std::string &key, std::string *out);
    void HouseKeeping();
    void LinkGone(net::LinkId link, bool fromHeartbeat);

    net::RpcServer rpc_;
    std::unique_ptr<StoreBackend> backend_;
    std::mutex mu_;  // guards everything below
    std::unordered_map<std::string, std::vector<Waiter>> keyWaiters_;
    std::multimap<uint64_t, std::pair<std::string, uint64_t>> timed_;  // deadline → (key, waiter id)
    std::vector<std::pair<net::LinkId, uint32_t>> rankWatchers_;
    std::unordered_map<net::LinkId, uint64_t> lastSeenMs_;
    std::unordered_map<net::LinkId, uint64_t> helloId_;
    std::unordered_map<net::LinkId, std::map<std::string, uint32_t>> linkRanks_;  // link → (auto-ranking key → rank)
    std::map<std::string, std::set<uint32_t>> usedRanks_;                           // auto-ranking key → taken ranks
    std::unordered_map<net::LinkId, uint32_t> linkWorldRank_;                       // rank announced in the handshake
    uint64_t nextWaiterId_{1};
    uint32_t worldSize_{0};
    OpHook opHook_;
    BrokenHook brokenHook_;
    std::thread house_;
    std::condition_variable cv_;
    std::atomic<bool> stop_{false};
    std::atomic<bool> mute_{false};
};

}  // namespace store
}  // namespace mf
