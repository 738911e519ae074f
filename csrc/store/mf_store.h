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
