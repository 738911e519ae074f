// Store client (optionally hosting the server in the same object) and the url → store factory.
//
// Follows the reference client (src/smem/csrc/config_store/tcp_store/smem_tcp_config_store.cpp): connect with up to
// 60 retries (:142-208), the handshake identity packs (worldSize << 32) | rankId (:21-23), a heartbeat thread, one
// transparent reconnect when a send fails (smem_tcp_config_store.h:111-120), failing every waiter and calling the
// broken handler when the link drops (:643-660), ReconnectAfterBroken + reconnect callback (:688-733). The factory
// mirrors src/smem/csrc/config_store/smem_store_factory.cpp:26-171 (cache by url, failure reason RESOURCE_IN_USE
// when somebody else already serves the port).
#pragma once
#include <atomic>
#include <condition_variable>
#include <mutex>
#include <thread>
#include <unordered_map>

#include "../net/mf_rpc.h"
#include "mf_store.h"
#include "mf_store_server.h"

namespace mf {
namespace store {

class TcpStore : public ConfigStore {
public:
    // rankId < 0: identity unknown at connect time (auto-ranking clients).
    TcpStore(net::Endpoint ep, bool isServer, uint32_t worldSize, int32_t rankId);
    ~TcpStore() override;
    // Starts the server (if isServer) and connects. Returns ST_OK, or a negative code; -EADDRINUSE from the server bind
    // is passed through so callers racing for the server role can tell.
    int Startup(int connectRetries = 60, int retryDelayMs = 1000);
    void Shutdown();
    StoreServer *Server() { return server_.get(); }

    int Set(const std::string &key, const std::string &value) override;
    int Get(const std::string &key, std::string *value, int64_t timeoutMs = -1) override;
    int Add(const std::string &key, int64_t delta, int64_t *newValue) override;
    int Remove(const std::string &key, bool quiet = false) override;
    int Append(const std::string &key, const std::string &value, uint64_t *newSize) override;
    int Cas(const std::string &key, const std::string &expect, const std::string &exchange, std::string *previous) override;
    int Write(const std::string &key, const std::string &value, uint32_t offset) override;
    int Watch(const std::string &key, WatchKeyCb cb, uint32_t *wid) override;
    int WatchRankDown(WatchRankCb cb, uint32_t *wid) override;
    int Unwatch(uint32_t wid) override;
    int Arrive(const std::string &counterKey, const std::string &wakeKey, uint32_t expected, int64_t timeoutMs,
               const std::vector<std::string> &gcKeys, int64_t *arrived) override;
    int Gather(const std::string &dataKey, const std::string &wakeKey, const std::string &record, uint64_t fullSize,
               int64_t timeoutMs, const std::vector<std::string> &gcKeys, std::string *all) override;
    bool Connected() const override { return rpc_.Connected(); }
    void SetBrokenHandler(std::function<void()> f) override { onBroken_ = std::move(f); }
    void SetReconnectHandler(std::function<void()> f) override { onReconnect_ = std::move(f); }
    int ReconnectAfterBroken(int retries) override;
    uint32_t AddReconnectListener(std::function<void()> f) override;
    void RemoveReconnectListener(uint32_t id) override;
    // Test hook: stop sending heartbeats (the server will declare this link dead).
    void SetDropHeartbeat(bool drop) { dropHeartbeat_.store(drop); }

private:
    int Request(uint16_t op, const StoreMessage &m, int64_t waitMs, net::Frame *reply);
    int Connect(int retries, int retryDelayMs);
    void HeartbeatLoop();

    net::Endpoint ep_;
    bool isServer_;
    uint32_t worldSize_;
    int32_t rankId_;
    std::unique_ptr<StoreServer> server_;
    net::RpcClient rpc_;
    std::thread heartbeat_;
    std::mutex hbMu_;
    std::condition_variable hbCv_;
    std::atomic<bool> stop_{false};
    std::atomic<bool> dropHeartbeat_{false};
    std::mutex reconnectMu_;
    std::function<void()> onBroken_;
    std::function<void()> onReconnect_;
    void NotifyReconnected();
    std::mutex listenerMu_;
    std::map<uint32_t, std::function<void()>> reconnectListeners_;
    uint32_t nextListener_{1};
    std::mutex watchMu_;
    std::unordered_map<uint32_t, uint32_t> watchSeq_;  // watch id → rpc seq
    uint32_t nextWid_{1};
};

// Swappable delegate (reference: config_store/ha/smem_ha_config_store.{h,cpp}): every call is forwarded under a
// read lock to the current delegate, which a leader-change procedure may replace under the write lock.
class HaStore : public ConfigStore {
public:
    explicit HaStore(StorePtr d) : delegate_(std::move(d)) {}
    void Swap(StorePtr d);
    StorePtr Current();
    int Set(const std::string &k, const std::string &v) override { return Current()->Set(k, v); }
    int Get(const std::string &k, std::string *v, int64_t t = -1) override { return Current()->Get(k, v, t); }
    int Add(const std::string &k, int64_t d, int64_t *n) override { return Current()->Add(k, d, n); }
    int Remove(const std::string &k, bool q = false) override { return Current()->Remove(k, q); }
    int Append(const std::string &k, const std::string &v, uint64_t *n) override { return Current()->Append(k, v, n); }
    int Cas(const std::string &k, const std::string &e, const std::string &x, std::string *p) override { return Current()->Cas(k, e, x, p); }
    int Write(const std::string &k, const std::string &v, uint32_t off) override { return Current()->Write(k, v, off); }
    int Watch(const std::string &k, WatchKeyCb cb, uint32_t *wid) override { return Current()->Watch(k, std::move(cb), wid); }
    int WatchRankDown(WatchRankCb cb, uint32_t *wid) override { return Current()->WatchRankDown(std::move(cb), wid); }
    int Unwatch(uint32_t wid) override { return Current()->Unwatch(wid); }
    int Arrive(const std::string &c, const std::string &w, uint32_t expected, int64_t t, const std::vector<std::string> &gc,
               int64_t *arrived) override
    {
        return Current()->Arrive(c, w, expected, t, gc, arrived);
    }
    int Gather(const std::string &d, const std::string &w, const std::string &rec, uint64_t fullSize, int64_t t,
               const std::vector<std::string> &gc, std::string *all) override
    {
        return Current()->Gather(d, w, rec, fullSize, t, gc, all);
    }
    bool Connected() const override { return const_cast<HaStore *>(this)->Current()->Connected(); }
    void SetBrokenHandler(std::function<void()> f) override { Current()->SetBrokenHandler(std::move(f)); }
    void SetReconnectHandler(std::function<void()> f) override { Current()->SetReconnectHandler(std::move(f)); }
    int ReconnectAfterBroken(int r) override { return Current()->ReconnectAfterBroken(r); }
    uint32_t AddReconnectListener(std::function<void()> f) override { return Current()->AddReconnectListener(std::move(f)); }
    void RemoveReconnectListener(uint32_t id) override { Current()->RemoveReconnectListener(id); }

private:
    std::mutex mu_;
    StorePtr delegate_;
};

// url-keyed cache of stores. Thread-safe.
class StoreFactory {
public:
    // Creates (or returns the cached) store for ip:port. isServer starts the server in this process first.
    static StorePtr CreateStore(const net::Endpoint &ep, bool isServer, uint32_t worldSize, int32_t rankId, int connectRetries = 60);
    static StorePtr PrefixOf(const StorePtr &base, const std::string &prefix);
    static void DestroyStore(const net::Endpoint &ep);
    static void DestroyAll();
    // Reason of the calling thread's last CreateStore failure (ST_OK if none); -EADDRINUSE maps to "resource in use".
    static int LastFailure();
    // Start a standalone server in this process (no client). Idempotent per port.
    static int CreateServer(const net::Endpoint &ep, uint32_t worldSize, StoreServer **out = nullptr);
    static void DestroyServer(uint16_t port);
};

}  // namespace store
}  // namespace mf
