// Best-fit sub-allocator over a fixed address range: free blocks indexed by address (for coalescing) and by size (for
// best fit), spin-locked, with an RAII element. Reference: RbtreeRangePool / SpaceAllocator
// (src/hybm/csrc/common/hybm_rbtree_range_pool.{h,cpp}, common/hybm_space_allocator.h). Here it carves tensors out of the
// symmetric heap and out of pinned host blocks; it never touches the memory it manages.
#pragma once
#include <atomic>
#include <cstdint>
#include <map>
#include <set>

namespace mf {
namespace hybm {

class RangePool {
public:
    RangePool(uint64_t base, uint64_t size, uint64_t align = 256) : base_(base), size_(size), align_(align ? align : 1)
    {
        if (size_ > 0) {
            byAddr_[base_] = size_;
            bySize_.insert({size_, base_});
        }
    }

    // Returns 0 when no free block is large enough.
    uint64_t Allocate(uint64_t bytes)
    {
        if (bytes == 0) {
            return 0;
        }
        bytes = (bytes + align_ - 1) / align_ * align_;
        Lock g(lock_);
        auto it = bySize_.lower_bound({bytes, 0});
        if (it == bySize_.end()) {
            return 0;
        }
        const uint64_t addr = it->second, blk = it->first;
        bySize_.erase(it);
        byAddr_.erase(addr);
        if (blk > bytes) {
            byAddr_[addr + bytes] = blk - bytes;
            bySize_.insert({blk - bytes, addr + bytes});
        }
        used_[addr] = bytes;
        inUse_ += bytes;
        return addr;
    }

    // False if `addr` was not returned by Allocate (double free, foreign pointer).
    bool Release(uint64_t addr)
    {
        Lock g(lock_);
        auto u = used_.find(addr);
        if (u == used_.end()) {
            return false;
        }
        uint64_t start = addr, len = u->second;
        inUse_ -= len;
        used_.erase(u);
        auto next = byAddr_.lower_bound(start);
        if (next != byAddr_.end() && next->first == start + len) {  // merge with the following free block
            len += next->second;
            bySize_.erase({next->second, next->first});
            next = byAddr_.erase(next);
        }
        if (next != byAddr_.begin()) {  // merge with the preceding free block
            auto prev = std::prev(next);
            if (prev->first + prev->second == start) {
                start = prev->first;
                len += prev->second;
                bySize_.erase({prev->second, prev->first});
                byAddr_.erase(prev);
            }
        }
        byAddr_[start] = len;
        bySize_.insert({len, start});
        return true;
    }

    uint64_t InUse() const { return inUse_; }
    uint64_t Capacity() const { return size_; }
    uint64_t LargestFree()
    {
        Lock g(lock_);
        return bySize_.empty() ? 0 : bySize_.rbegin()->first;
    }
    size_t FreeBlocks()
    {
        Lock g(lock_);
        return byAddr_.size();
    }

private:
    struct Lock {
        explicit Lock(std::atomic_flag &f) : f_(f)
        {
            while (f_.test_and_set(std::memory_order_acquire)) {
            }
        }
        ~Lock() { f_.clear(std::memory_order_release); }
        std::atomic_flag &f_;
    };
    uint64_t base_, size_, align_;
    std::atomic_flag lock_ = ATOMIC_FLAG_INIT;
    std::map<uint64_t, uint64_t> byAddr_;             // free: address → size
    std::set<std::pair<uint64_t, uint64_t>> bySize_;  // free: (size, address)
    std::map<uint64_t, uint64_t> used_;               // allocated: address → size
    uint64_t inUse_{0};
};

// RAII element: releases its range when it goes out of scope.
class PoolElement {
public:
    PoolElement(RangePool *pool, uint64_t bytes) : pool_(pool), addr_(pool->Allocate(bytes)) {}
    ~PoolElement()
    {
        if (addr_ != 0) {
            pool_->Release(addr_);
        }
    }
    PoolElement(const PoolElement &) = delete;
    PoolElement &operator=(const PoolElement &) = delete;
    uint64_t Address() const { return addr_; }
    explicit operator bool() const { return addr_ != 0; }

private:
    RangePool *pool_;
    uint64_t addr_;
};

}  // namespace hybm
}  // namespace mf
