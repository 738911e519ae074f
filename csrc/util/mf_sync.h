// Lock primitives (roles of src/util/csrc/mf_rwlock.h:11-90 and mf_spinlock.h:22-50 of the reference): a readers/writer
// lock with scope guards for the read-mostly tables (imported peers, registered regions) and a test-and-test-and-set spin
// lock with back-off for the few-instruction critical sections on the transfer path.
#pragma once
#include <atomic>
#include <pthread.h>
#include <thread>

namespace mf {
namespace util {

class RwLock {
public:
    RwLock()
    {
        pthread_rwlockattr_t attr;
        pthread_rwlockattr_init(&attr);
        // Writers are rare and must not starve behind a stream of readers.
        pthread_rwlockattr_setkind_np(&attr, PTHREAD_RWLOCK_PREFER_WRITER_NONRECURSIVE_NP);
        pthread_rwlock_init(&lock_, &attr);
        pthread_rwlockattr_destroy(&attr);
    }
    ~RwLock() { pthread_rwlock_destroy(&lock_); }
    RwLock(const RwLock &) = delete;
    RwLock &operator=(const RwLock &) = delete;
    void LockRead() { pthread_rwlock_rdlock(&lock_); }
    void LockWrite() { pthread_rwlock_wrlock(&lock_); }
    bool TryLockRead() { return pthread_rwlock_tryrdlock(&lock_) == 0; }
    bool TryLockWrite() { return pthread_rwlock_trywrlock(&lock_) == 0; }
    void Unlock() { pthread_rwlock_unlock(&lock_); }

private:
    pthread_rwlock_t lock_;
};

class ReadGuard {
public:
    explicit ReadGuard(RwLock &l) : l_(l) { l_.LockRead(); }
    ~ReadGuard() { l_.Unlock(); }
    ReadGuard(const ReadGuard &) = delete;
    ReadGuard &operator=(const ReadGuard &) = delete;

private:
    RwLock &l_;
};

class WriteGuard {
public:
    explicit WriteGuard(RwLock &l) : l_(l) { l_.LockWrite(); }
    ~WriteGuard() { l_.Unlock(); }
    WriteGuard(const WriteGuard &) = delete;
    WriteGuard &operator=(const WriteGuard &) = delete;

private:
    RwLock &l_;
};

class SpinLock {
public:
    void Lock()
    {
        int spins = 0;
        while (true) {
            if (!flag_.load(std::memory_order_relaxed) && !flag_.exchange(true, std::memory_order_acquire)) {
                return;
            }
            if (++spins < 64) {
#if defined(__x86_64__) || defined(__i386__)
                __builtin_ia32_pause();
#endif
            } else {
                std::this_thread::yield();
                spins = 0;
            }
        }
    }
    bool TryLock() { return !flag_.load(std::memory_order_relaxed) && !flag_.exchange(true, std::memory_order_acquire); }
    void Unlock() { flag_.store(false, std::memory_order_release); }

private:
    std::atomic<bool> flag_{false};
};

class SpinGuard {
public:
    explicit SpinGuard(SpinLock &l) : l_(l) { l_.Lock(); }
    ~SpinGuard() { l_.Unlock(); }
    SpinGuard(const SpinGuard &) = delete;
    SpinGuard &operator=(const SpinGuard &) = delete;

private:
    SpinLock &l_;
};

}  // namespace util
}  // namespace mf
