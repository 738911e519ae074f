#include "mf_store_client.h"

#include <unistd.h>

#include "../net/mf_tls.h"

#include <cerrno>
#include <cstring>
#include <map>

#include "../util/mf_log.h"

namespace mf {
namespace store {

TcpStore::TcpStore(net::Endpoint ep, bool isServer, uint32_t worldSize, int32_t rankId)
    : ep_(std::move(ep)), isServer_(isServer), worldSize_(worldSize), rankId_(rankId)
{
}

TcpStore::~TcpStore() { Shutdown(); }

int TcpStore::Connect(int retries, int retryDelayMs)
{
    uint64_t id = ((uint64_t)worldSize_ << 32) | (rankId_ < 0 ? 0xffffffffull : (uint64_t)(uint32_t)rankId_);
    net::Endpoint target = ep_;
    if (isServer_ && (target.host == "0.0.0.0" || target.host == "::")) {
        target.host = target.v6 ? "::1" : "127.0.0.1";
    }
    net::TlsOptions tls = net::GetStoreTlsOptions();
    if (tls.enable) {
        std::string err;
        auto ctx = net::TlsContext::Create(tls, false, &err);
        if (!ctx) {
            MF_ERROR("store client: TLS is enabled but cannot be set up: " << err);
            return ST_IO_ERROR;
        }
        rpc_.SetTls(ctx);
    } else {
        rpc_.SetTls(nullptr);
    }
    const bool afterGoodbye = rpc_.PeerSaidGoodbye();
    int rc = rpc_.Connect(target, id, retries, retryDelayMs);
    if (rc != 0) {
        if (afterGoodbye || stop_.load()) {
            MF_INFO("store client: the server at " << target.host << ":" << target.port << " has shut down");
        } else {
            MF_ERROR("store client: cannot connect to " << target.host << ":" << target.port);
        }
        return ST_IO_ERROR;
    }
    return ST_OK;
}

int TcpStore::Startup(int connectRetries, int retryDelayMs)
{
    stop_.store(false);
    if (isServer_) {
        server_.reset(new StoreServer());
        int rc = server_->Start(ep_, 0);
        if (rc != 0) {
            server_.reset();
            if (rc != -EADDRINUSE) {
                MF_ERROR("store server: start failed on port " << ep_.port << ": " << strerror(-rc));
            }
            return rc;
        }
        if (ep_.port == 0) {
            ep_.port = server_->Port();
        }
    }
    rpc_.SetBrokenHandler([this]() {
        if (rpc_.PeerSaidGoodbye()) {
            MF_INFO("store client: the server closed the link in good order");
        } else {
            MF_WARN("store client: link to the server is broken");
        }
        if (onBroken_) {
            onBroken_();
        }
    });
    int rc = Connect(connectRetries, retryDelayMs);
    if (rc != ST_OK) {
        return rc;
    }
    heartbeat_ = std::thread([this]() { HeartbeatLoop(); });
    return ST_OK;
}

void TcpStore::Shutdown()
{
    if (stop_.exchange(true)) {
        return;
    }
    hbCv_.notify_all();
    if (heartbeat_.joinable()) {
        heartbeat_.join();
    }
    rpc_.Close();
    if (server_) {
        // The process that hosts the server leaves last: give the other ranks a moment to close their links themselves
        // (they are usually inside the same tear-down), then say goodbye to whoever is still there.
        const uint32_t lingerMs = GlobalTiming().serverLingerMs;
        for (uint32_t waited = 0; waited < lingerMs && server_->AliveLinks() > 0; waited += 10) {
            usleep(10 * 1000);
        }
        server_->Stop();
        server_.reset();
    }
}

void TcpStore::HeartbeatLoop()
{
    std::unique_lock<std::mutex> lk(hbMu_);
    while (!stop_.load()) {
        uint32_t period = GlobalTiming().heartbeatIntervalMs;
        hbCv_.wait_for(lk, std::chrono::milliseconds(period));
        if (stop_.load()) {
            break;
        }
        if (dropHeartbeat_.load() || !rpc_.Connected()) {
            continue;
        }
        lk.unlock();
        net::Frame reply;
        rpc_.Call(OP_HEARTBEAT, "", &reply, period);
        lk.lock();
    }
}

int TcpStore::ReconnectAfterBroken(int retries)
{
    std::lock_guard<std::mutex> g(reconnectMu_);
    if (rpc_.Connected()) {
        return ST_OK;
    }
    int rc = Connect(retries, 1000);
    if (rc == ST_OK) {
        NotifyReconnected();
    }
    return rc;
}

void TcpStore::NotifyReconnected()
{
    if (onReconnect_) {
        onReconnect_();
    }
    std::vector<std::function<void()>> fns;
    {
        std::lock_guard<std::mutex> g(listenerMu_);
        for (auto &kv : reconnectListeners_) {
            fns.push_back(kv.second);
        }
    }
    for (auto &f : fns) {
        f();
    }
}

uint32_t TcpStore::AddReconnectListener(std::function<void()> f)
{
    std::lock_guard<std::mutex> g(listenerMu_);
    uint32_t id = nextListener_++;
    reconnectListeners_[id] = std::move(f);
    return id;
}

void TcpStore::RemoveReconnectListener(uint32_t id)
{
    std::lock_guard<std::mutex> g(listenerMu_);
    reconnectListeners_.erase(id);
}

int TcpStore::Request(uint16_t op, const StoreMessage &m, int64_t waitMs, net::Frame *reply)
{
    std::string body = PackMessage(m);
    int rc = rpc_.Call(op, body, reply, waitMs);
    if (rc == net::RPC_IO_ERROR && !stop_.load() && !dropHeartbeat_.load()) {
        // One transparent reconnect, then one retry.
        bool again = false;
        {
            std::lock_guard<std::mutex> g(reconnectMu_);
            again = rpc_.Connected() || Connect(2, 200) == ST_OK;
        }
        if (again) {
            NotifyReconnected();
            rc = rpc_.Call(op, body, reply, waitMs);
        }
    }
    if (rc == net::RPC_IO_ERROR) {
        return ST_IO_ERROR;
    }
    if (rc == net::RPC_TIMEOUT) {
        return ST_TIMEOUT;
    }
    return reply->result;
}

static bool KeyOk(const std::string &key) { return !key.empty() && key.size() <= MAX_KEY_LEN_CLIENT; }
static constexpr int64_t kControlWaitMs = 60000;  // transport-level wait for ops the server answers at once

int TcpStore::Set(const std::string &key, const std::string &value)
{
    if (!KeyOk(key)) {
        return ST_INVALID_KEY;
    }
    if (value.size() > MAX_VALUE_LEN) {
        return ST_INVALID_MESSAGE;
    }
    StoreMessage m;
    m.keys = {key};
    m.values = {value};
    net::Frame r;
    return Request(OP_SET, m, kControlWaitMs, &r);
}

int TcpStore::Get(const std::string &key, std::string *value, int64_t timeoutMs)
{
    if (!KeyOk(key)) {
        return ST_INVALID_KEY;
    }
    StoreMessage m;
    m.userDef = timeoutMs;
    m.keys = {key};
    net::Frame r;
    // The server answers TIMEOUT itself; the transport wait is a little longer so that answer is what we see.
    int rc = Request(OP_GET, m, timeoutMs < 0 ? -1 : timeoutMs + 5000, &r);
    if (rc == ST_OK || rc == ST_RESTORE) {
        if (value != nullptr) {
            *value = std::move(r.body);
        }
    }
    return rc;
}

int TcpStore::Add(const std::string &key, int64_t delta, int64_t *newValue)
{
    if (!KeyOk(key)) {
        return ST_INVALID_KEY;
    }
    StoreMessage m;
    m.keys = {key};
    m.values = {std::to_string(delta)};
    net::Frame r;
    int rc = Request(OP_ADD, m, kControlWaitMs, &r);
    if (rc == ST_OK && newValue != nullptr) {
        *newValue = std::strtoll(r.body.c_str(), nullptr, 10);
    }
    return rc;
}

int TcpStore::Remove(const std::string &key, bool quiet)
{
    if (!KeyOk(key)) {
        return ST_INVALID_KEY;
    }
    StoreMessage m;
    m.keys = {key};
    net::Frame r;
    int rc = Request(OP_REMOVE, m, kControlWaitMs, &r);
    if (rc == ST_NOT_EXIST && !quiet) {
        MF_DEBUG("store: remove of absent key " << key);
    }
    return rc;
}

int TcpStore::Append(const std::string &key, const std::string &value, uint64_t *newSize)
{
    if (!KeyOk(key)) {
        return ST_INVALID_KEY;
    }
    StoreMessage m;
    m.keys = {key};
    m.values = {value};
    net::Frame r;
    int rc = Request(OP_APPEND, m, kControlWaitMs, &r);
    if (rc == ST_OK && newSize != nullptr) {
        *newSize = std::strtoull(r.body.c_str(), nullptr, 10);
    }
    return rc;
}

int TcpStore::Arrive(const std::string &counterKey, const std::string &wakeKey, uint32_t expected, int64_t timeoutMs,
                     const std::vector<std::string> &gcKeys, int64_t *arrived)
{
    if (!KeyOk(counterKey) || !KeyOk(wakeKey) || gcKeys.size() + 2 > MAX_KEYS_PER_MSG) {
        return ST_INVALID_KEY;
    }
    StoreMessage m;
    m.userDef = timeoutMs;
    m.keys = {counterKey, wakeKey};
    m.keys.insert(m.keys.end(), gcKeys.begin(), gcKeys.end());
    m.values = {std::to_string(expected)};
    net::Frame r;
    int rc = Request(OP_ARRIVE, m, timeoutMs < 0 ? -1 : timeoutMs + 5000, &r);
    if (arrived != nullptr) {
        *arrived = -1;  // only the server knows; the reply of a parked arrival carries the wake value
    }
    return rc;
}

int TcpStore::Gather(const std::string &dataKey, const std::string &wakeKey, const std::string &record, uint64_t fullSize,
                     int64_t timeoutMs, const std::vector<std::string> &gcKeys, std::string *all)
{
    if (!KeyOk(dataKey) || !KeyOk(wakeKey) || gcKeys.size() + 2 > MAX_KEYS_PER_MSG) {
        return ST_INVALID_KEY;
    }
    if (record.size() > MAX_VALUE_LEN || fullSize > MAX_VALUE_LEN) {
        return ST_INVALID_MESSAGE;
    }
    StoreMessage m;
    m.userDef = timeoutMs;
    m.keys = {dataKey, wakeKey};
    m.keys.insert(m.keys.end(), gcKeys.begin(), gcKeys.end());
    m.values = {record, std::to_string(fullSize)};
    net::Frame r;
    int rc = Request(OP_GATHER, m, timeoutMs < 0 ? -1 : timeoutMs + 5000, &r);
    if (rc == ST_OK && all != nullptr) {
        *all = std::move(r.body);
    }
    return rc;
}

int TcpStore::Cas(const std::string &key, const std::string &expect, const std::string &exchange, std::string *previous)
{
    if (!KeyOk(key)) {
        return ST_INVALID_KEY;
    }
    StoreMessage m;
    m.keys = {key};
    m.values = {expect, exchange};
    net::Frame r;
    int rc = Request(OP_CAS, m, kControlWaitMs, &r);
    if (rc == ST_OK && previous != nullptr) {
        *previous = std::move(r.body);
    }
    return rc;
}

int TcpStore::Write(const std::string &key, const std::string &value, uint32_t offset)
{
    if (!KeyOk(key)) {
        return ST_INVALID_KEY;
    }
    StoreMessage m;
    m.keys = {key};
    std::string v((const char *)&offset, 4);
    v.append(value);
    m.values = {std::move(v)};
    net::Frame r;
    return Request(OP_WRITE, m, kControlWaitMs, &r);
}

int TcpStore::Watch(const std::string &key, WatchKeyCb cb, uint32_t *wid)
{
    if (!KeyOk(key)) {
        return ST_INVALID_KEY;
    }
    StoreMessage m;
    m.userDef = -1;
    m.keys = {key};
    // watchMu_ is held across the send and the bookkeeping so that a reply racing in on the reader thread
    // finds its entry.
    std::lock_guard<std::mutex> g(watchMu_);
    uint32_t id = nextWid_++;
    uint32_t seq = rpc_.CallPersistent(OP_GET, PackMessage(m), [this, cb, key, id](const net::Frame &f) {
        bool live;
        {
            std::lock_guard<std::mutex> g2(watchMu_);
            live = watchSeq_.erase(id) > 0;
        }
        rpc_.Cancel(f.seq);  // one-shot
        if (live) {
            cb(f.result, key, f.body);
        }
    });
    if (seq == 0) {
        return ST_IO_ERROR;
    }
    watchSeq_[id] = seq;
    if (wid != nullptr) {
        *wid = id;
    }
    return ST_OK;
}

int TcpStore::WatchRankDown(WatchRankCb cb, uint32_t *wid)
{
    StoreMessage m;
    m.keys = {WATCH_RANK_DOWN_KEY};
    uint32_t seq = rpc_.CallPersistent(OP_WATCH_RANK_STATE, PackMessage(m), [cb](const net::Frame &f) {
        if (f.result == ST_OK && f.body.size() == sizeof(uint32_t)) {
            uint32_t rank;
            std::memcpy(&rank, f.body.data(), sizeof(rank));
            cb(rank);
        }
    });
    if (seq == 0) {
        return ST_IO_ERROR;
    }
    std::lock_guard<std::mutex> g(watchMu_);
    uint32_t id = nextWid_++;
    watchSeq_[id] = seq;
    if (wid != nullptr) {
        *wid = id;
    }
    return ST_OK;
}

int TcpStore::Unwatch(uint32_t wid)
{
    uint32_t seq = 0;
    {
        std::lock_guard<std::mutex> g(watchMu_);
        auto it = watchSeq_.find(wid);
        if (it == watchSeq_.end()) {
            return ST_NOT_EXIST;
        }
        seq = it->second;
        watchSeq_.erase(it);
    }
    rpc_.Cancel(seq);
    return ST_OK;
}

// ---------------------------------------------------------------------------------------------- HA delegate

void HaStore::Swap(StorePtr d)
{
    std::lock_guard<std::mutex> g(mu_);
    delegate_ = std::move(d);
}

StorePtr HaStore::Current()
{
    std::lock_guard<std::mutex> g(mu_);
    return delegate_;
}

// ---------------------------------------------------------------------------------------------- factory

static std::mutex g_factoryMu;
static std::map<std::string, std::shared_ptr<TcpStore>> g_stores;
static std::map<uint16_t, std::unique_ptr<StoreServer>> g_servers;
static thread_local int g_lastFailure = ST_OK;

static std::string KeyOf(const net::Endpoint &ep) { return ep.host + ":" + std::to_string(ep.port); }

StorePtr StoreFactory::CreateStore(const net::Endpoint &ep, bool isServer, uint32_t worldSize, int32_t rankId, int connectRetries)
{
    std::lock_guard<std::mutex> g(g_factoryMu);
    g_lastFailure = ST_OK;
    auto it = g_stores.find(KeyOf(ep));
    if (it != g_stores.end()) {
        return it->second;
    }
    auto st = std::make_shared<TcpStore>(ep, isServer, worldSize, rankId);
    int rc = st->Startup(connectRetries);
    if (rc != ST_OK) {
        g_lastFailure = rc;
        return nullptr;
    }
    g_stores[KeyOf(ep)] = st;
    return st;
}

StorePtr StoreFactory::PrefixOf(const StorePtr &base, const std::string &prefix)
{
    if (!base) {
        return nullptr;
    }
    return std::make_shared<PrefixStore>(base, prefix);
}

void StoreFactory::DestroyStore(const net::Endpoint &ep)
{
    std::shared_ptr<TcpStore> st;
    {
        std::lock_guard<std::mutex> g(g_factoryMu);
        auto it = g_stores.find(KeyOf(ep));
        if (it == g_stores.end()) {
            return;
        }
        st = it->second;
        g_stores.erase(it);
    }
    st->Shutdown();
}

void StoreFactory::DestroyAll()
{
    std::map<std::string, std::shared_ptr<TcpStore>> all;
    std::map<uint16_t, std::unique_ptr<StoreServer>> servers;
    {
        std::lock_guard<std::mutex> g(g_factoryMu);
        all.swap(g_stores);
        servers.swap(g_servers);
    }
    for (auto &kv : all) {
        kv.second->Shutdown();
    }
    for (auto &kv : servers) {
        kv.second->Stop();
    }
}

int StoreFactory::LastFailure() { return g_lastFailure; }

int StoreFactory::CreateServer(const net::Endpoint &ep, uint32_t worldSize, StoreServer **out)
{
    std::lock_guard<std::mutex> g(g_factoryMu);
    auto it = g_servers.find(ep.port);
    if (it != g_servers.end() && ep.port != 0) {
        if (out != nullptr) {
            *out = it->second.get();
        }
        return ST_OK;
    }
    std::unique_ptr<StoreServer> s(new StoreServer());
    int rc = s->Start(ep, worldSize);
    if (rc != 0) {
        return rc;
    }
    if (out != nullptr) {
        *out = s.get();
    }
    g_servers[s->Port()] = std::move(s);
    return ST_OK;
}

void StoreFactory::DestroyServer(uint16_t port)
{
    std::unique_ptr<StoreServer> s;
    {
        std::lock_guard<std::mutex> g(g_factoryMu);
        auto it = g_servers.find(port);
        if (it == g_servers.end()) {
            return;
        }
        s = std::move(it->second);
        g_servers.erase(it);
    }
    s->Stop();
}

}  // namespace store
}  // namespace mf
