// Config store: the TCP key-value control plane every rank of a job connects to.
//
// Semantics reproduced from the reference (interface src/smem/csrc/config_store/smem_config_store.h:44-281,
// message body tcp_store/smem_message_packer.h:29-77, per-op behaviour tcp_store/smem_tcp_config_store_server.cpp:257-737):
//   Set            overwrite, wakes every blocked Get on the key
//   Get            timeoutMs 0 = immediate NOT_EXIST, >0 = timed wait, <0 = wait forever
//   Add            int64 counter stored as decimal text, returns the new value
//   Remove         NOT_EXIST if absent
//   Append         returns the new total size
//   Cas            expected "" matches an absent key; returns the PREVIOUS value, the caller compares
//   Write          in-place write at an offset, zero-filling any gap
//   Watch          one-shot notification when a key appears
//   WatchRankDown  repeated notification carrying the rank id of every link that died
// plus heartbeats, auto-ranking (lowest free rank id per link) and pluggable server-side hooks.
#pragma once
#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

namespace mf {
namespace store {

enum StoreCode : int {
    ST_OK = 0,
    ST_ERROR = -1,
    ST_INVALID_MESSAGE = -400,
    ST_INVALID_KEY = -401,
    ST_NOT_EXIST = -404,
    ST_RESTORE = -405,  // answered from a fault handler's pool of recycled ids
    ST_TIMEOUT = -601,
    ST_IO_ERROR = -602,
};

enum StoreOp : uint16_t {
    OP_SET = 1,
    OP_GET = 2,
    OP_ADD = 3,
    OP_REMOVE = 4,
    OP_APPEND = 5,
    OP_CAS = 6,
    OP_WRITE = 7,
    OP_WATCH_RANK_STATE = 8,
    OP_HEARTBEAT = 9,
    OP_ARRIVE = 10,  // counter += 1 and wait for the wake key in one round trip (group barrier)
    OP_GATHER = 11,  // append a record and wait until the value has its full size (group all-gather)
};

constexpr size_t MAX_KEY_LEN_CLIENT = 1024;
constexpr size_t MAX_KEY_LEN_SERVER = 2048;
constexpr size_t MAX_VALUE_LEN = 64ull * 1024 * 1024;
constexpr size_t MAX_KEYS_PER_MSG = 10;
constexpr size_t MAX_VALUES_PER_MSG = 10;
constexpr const char *AUTO_RANKING_PREFIX = "AutoRanking#";
constexpr const char *WATCH_RANK_DOWN_KEY = "__WATCH_RANK_LINK_DOWN__";

struct StoreMessage {
    int64_t userDef{-1};  // GET: timeout in ms
    std::vector<std::string> keys;
    std::vector<std::string> values;
};
std::string PackMessage(const StoreMessage &m);
// Returns false when the buffer is truncated, over a limit, or has trailing bytes.
bool UnpackMessage(const std::string &buf, StoreMessage *out);

using WatchKeyCb = std::function<void(int result, const std::string &key, const std::string &value)>;
using WatchRankCb = std::function<void(uint32_t rankId)>;

// Abstract store used by every layer above; decorated by PrefixStore / HaStore.
class ConfigStore {
public:
    virtual ~ConfigStore() = default;
    virtual int Set(const std::string &key, const std::string &value) = 0;
    virtual int Get(const std::string &key, std::string *value, int64_t timeoutMs = -1) = 0;
    virtual int Add(const std::string &key, int64_t delta, int64_t *newValue) = 0;
    virtual int Remove(const std::string &key, bool quiet = false) = 0;
    virtual int Append(const std::string &key, const std::string &value, uint64_t *newSize) = 0;
    virtual int Cas(const std::string &key, const std::string &expect, const std::string &exchange, std::string *previous) = 0;
    virtual int Write(const std::string &key, const std::string &value, uint32_t offset) = 0;
    virtual int Watch(const std::string &key, WatchKeyCb cb, uint32_t *wid) = 0;
    virtual int WatchRankDown(WatchRankCb cb, uint32_t *wid) = 0;
    virtual int Unwatch(uint32_t wid) = 0;
    // Barrier arrival: adds 1 to `counterKey`; the arrival that makes it `expected` sets `wakeKey` and removes `gcKeys`
    // (keys of finished rounds); every caller returns once `wakeKey` exists or after `timeoutMs` (ST_TIMEOUT). The base
    // version composes it from Add / Set / Get / Remove; a TCP store sends ONE request that the server parks until the last
    // member has arrived, so a barrier costs one round trip per rank instead of three to seven.
    virtual int Arrive(const std::string &counterKey, const std::string &wakeKey, uint32_t expected, int64_t timeoutMs,
                       const std::vector<std::string> &gcKeys, int64_t *arrived)
    {
        int64_t val = 0;
        int rc = Add(counterKey, 1, &val);
        if (rc != ST_OK) {
            return rc;
        }
        if (arrived != nullptr) {
            *arrived = val;
        }
        if ((uint64_t)val == expected) {
            for (const auto &k : gcKeys) {
                Remove(k, true);
            }
            rc = Set(wakeKey, "ok");
            if (rc != ST_OK) {
                return rc;
            }
        }
        std::string v;
        return Get(wakeKey, &v, timeoutMs);
    }
    // All-gather contribution: appends `record` to `dataKey` and returns the whole value in *all once it is `fullSize`
    // bytes long (every member has appended), or ST_TIMEOUT. `wakeKey` is set by the completing append. Base version:
    // Append / Set / Get / Get; a TCP store does it in one request.
    virtual int Gather(const std::string &dataKey, const std::string &wakeKey, const std::string &record, uint64_t fullSize,
                       int64_t timeoutMs, const std::vector<std::string> &gcKeys, std::string *all)
    {
        uint64_t total = 0;
        int rc = Append(dataKey, record, &total);
        if (rc != ST_OK) {
            return rc;
        }
        if (total == fullSize) {
            for (const auto &k : gcKeys) {
                Remove(k, true);
            }
            rc = Set(wakeKey, "ok");
            if (rc != ST_OK) {
                return rc;
            }
        }
        std::string v;
        rc = Get(wakeKey, &v, timeoutMs);
        if (rc != ST_OK) {
            return rc;
        }
        return Get(dataKey, all, timeoutMs);
    }
    virtual std::string CommonPrefix() const { return ""; }
    virtual bool Connected() const { return true; }
    // Handlers for a lost / re-established link to the server (client stores only).
    virtual void SetBrokenHandler(std::function<void()>) {}
    virtual void SetReconnectHandler(std::function<void()>) {}
    virtual int ReconnectAfterBroken(int /*retries*/) { return ST_OK; }
    // Any number of additional subscribers to "the link to the server is up again" (the group engines on one store each
    // repair their own state). Returns an id for RemoveReconnectListener; 0 if the store has no notion of a link. The
    // callback runs on whichever thread noticed the reconnect and must not call back into the store.
    virtual uint32_t AddReconnectListener(std::function<void()>) { return 0; }
    virtual void RemoveReconnectListener(uint32_t) {}
};
using StorePtr = std::shared_ptr<ConfigStore>;

// Namespacing decorator (reference: tcp_store/smem_prefix_config_store.h). Nested prefixes concatenate.
class PrefixStore : public ConfigStore {
public:
    PrefixStore(StorePtr base, std::string prefix) : base_(std::move(base)), prefix_(std::move(prefix)) {}
    int Set(const std::string &k, const std::string &v) override { return base_->Set(prefix_ + k, v); }
    int Get(const std::string &k, std::string *v, int64_t t = -1) override { return base_->Get(prefix_ + k, v, t); }
    int Add(const std::string &k, int64_t d, int64_t *n) override { return base_->Add(prefix_ + k, d, n); }
    int Remove(const std::string &k, bool q = false) override { return base_->Remove(prefix_ + k, q); }
    int Append(const std::string &k, const std::string &v, uint64_t *n) override { return base_->Append(prefix_ + k, v, n); }
    int Cas(const std::string &k, const std::string &e, const std::string &x, std::string *p) override
    {
        return base_->Cas(prefix_ + k, e, x, p);
    }
    int Write(const std::string &k, const std::string &v, uint32_t off) override { return base_->Write(prefix_ + k, v, off); }
    int Watch(const std::string &k, WatchKeyCb cb, uint32_t *wid) override
    {
        size_t n = prefix_.size();
        return base_->Watch(prefix_ + k,
                            [cb, n](int r, const std::string &key, const std::string &v) { cb(r, key.size() >= n ? key.substr(n) : key, v); },
                            wid);
    }
    int WatchRankDown(WatchRankCb cb, uint32_t *wid) override { return base_->WatchRankDown(std::move(cb), wid); }
    int Unwatch(uint32_t wid) override { return base_->Unwatch(wid); }
    int Arrive(const std::string &c, const std::string &w, uint32_t expected, int64_t t, const std::vector<std::string> &gc,
               int64_t *arrived) override
    {
        std::vector<std::string> full;
        for (const auto &k : gc) {
            full.push_back(prefix_ + k);
        }
        return base_->Arrive(prefix_ + c, prefix_ + w, expected, t, full, arrived);
    }
    int Gather(const std::string &d, const std::string &w, const std::string &rec, uint64_t fullSize, int64_t t,
               const std::vector<std::string> &gc, std::string *all) override
    {
        std::vector<std::string> full;
        for (const auto &k : gc) {
            full.push_back(prefix_ + k);
        }
        return base_->Gather(prefix_ + d, prefix_ + w, rec, fullSize, t, full, all);
    }
    std::string CommonPrefix() const override { return base_->CommonPrefix() + prefix_; }
    bool Connected() const override { return base_->Connected(); }
    void SetBrokenHandler(std::function<void()> f) override { base_->SetBrokenHandler(std::move(f)); }
    void SetReconnectHandler(std::function<void()> f) override { base_->SetReconnectHandler(std::move(f)); }
    int ReconnectAfterBroken(int r) override { return base_->ReconnectAfterBroken(r); }
    uint32_t AddReconnectListener(std::function<void()> f) override { return base_->AddReconnectListener(std::move(f)); }
    void RemoveReconnectListener(uint32_t id) override { base_->RemoveReconnectListener(id); }
    StorePtr Base() const { return base_; }

private:
    StorePtr base_;
    std::string prefix_;
};

}  // namespace store
}  // namespace mf
