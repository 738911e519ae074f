// Storage backend of the store server: where key/value pairs physically live.
//
// Same seam as the reference's ConfigStoreBackend (src/smem/csrc/config_store/backend/smem_config_store_backend.h:36-298):
// Get / Put(with optional TTL) / Delete / Exist / Clear plus an advisory lock API with an RAII guard. Only the
// in-process map backend ships (the reference ships only that one as well); a replicated backend can be slotted
// in behind the same interface.
#pragma once
#include <chrono>
#include <cstdint>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>

namespace mf {
namespace store {

class StoreBackend {
public:
    virtual ~StoreBackend() = default;
    virtual bool Get(const std::string &key, std::string *value) = 0;
    // ttlMs 0 = no expiry.
    virtual void Put(const std::string &key, const std::string &value, uint64_t ttlMs = 0) = 0;
    virtual bool Delete(const std::string &key) = 0;
    virtual bool Exist(const std::string &key) = 0;
    virtual void Clear() = 0;
    virtual size_t Size() = 0;
    // Mutable access for in-place operations (Append/Write); returns nullptr if absent. Valid until the next call.
    virtual std::string *Mutable(const std::string &key) = 0;
    // Advisory named locks: TryLock succeeds if nobody or the same owner holds it, or the holder's lease ran out.
    virtual bool TryLock(const std::string &name, const std::string &owner, uint64_t leaseMs) = 0;
    virtual bool Unlock(const std::string &name, const std::string &owner) = 0;
};

class LocalMemoryBackend : public StoreBackend {
public:
    bool Get(const std::string &key, std::string *value) override;
    void Put(const std::string &key, const std::string &value, uint64_t ttlMs = 0) override;
    bool Delete(const std::string &key) override;
    bool Exist(const std::string &key) override;
    void Clear() override;
    size_t Size() override;
    std::string *Mutable(const std::string &key) override;
    bool TryLock(const std::string &name, const std::string &owner, uint64_t leaseMs) override;
    bool Unlock(const std::string &name, const std::string &owner) override;

private:
    struct Entry {
        std::string value;
        uint64_t expireAtMs{0};
    };
    struct LockRec {
        std::string owner;
        uint64_t expireAtMs{0};
    };
    bool Expired(const Entry &e) const;
    std::mutex mu_;
    std::unordered_map<std::string, Entry> kv_;
    std::unordered_map<std::string, LockRec> locks_;
};

// RAII guard: holds the named lock for its lifetime when Locked() is true.
class BackendLockGuard {
public:
    BackendLockGuard(StoreBackend *b, std::string name, std::string owner, uint64_t leaseMs)
        : b_(b), name_(std::move(name)), owner_(std::move(owner))
    {
        locked_ = b_->TryLock(name_, owner_, leaseMs);
    }
    ~BackendLockGuard()
    {
        if (locked_) {
            b_->Unlock(name_, owner_);
        }
    }
    bool Locked() const { return locked_; }

private:
    StoreBackend *b_;
    std::string name_, owner_;
    bool locked_{false};
};

}  // namespace store
}  // namespace mf
