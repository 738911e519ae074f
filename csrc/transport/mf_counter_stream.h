// Completion accounting for asynchronous one-sided operations: a monotonically growing count of submitted pieces, a count
// of finished ones and the first error, per destination rank. Role of the reference's counting stream
// (src/hybm/csrc/transport/host/host_hcom_counter_stream.h:12-64): Submit() before a piece is queued, Complete() from the
// thread that finished it, Synchronize() blocks until everything submitted so far is finished and hands back (and clears)
// the first failure.
#pragma once
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <mutex>

namespace mf {
namespace transport {

class CounterStream {
public:
    void Submit(uint64_t pieces = 1)
    {
        std::lock_guard<std::mutex> g(mu_);
        submitted_ += pieces;
    }
    void Complete(int result)
    {
        std::lock_guard<std::mutex> g(mu_);
        finished_++;
        if (result != 0 && firstError_ == 0) {
            firstError_ = result;
        }
        if (finished_ >= submitted_) {
            cv_.notify_all();
        }
    }
    // 0, the first error of the pieces waited for, or `timeoutCode` if they do not finish within timeoutMs (< 0: no limit).
    int Synchronize(int64_t timeoutMs, int timeoutCode)
    {
        std::unique_lock<std::mutex> lk(mu_);
        const uint64_t target = submitted_;
        auto done = [&]() { return finished_ >= target; };
        if (timeoutMs < 0) {
            cv_.wait(lk, done);
        } else if (!cv_.wait_for(lk, std::chrono::milliseconds(timeoutMs), done)) {
            return timeoutCode;
        }
        int rc = firstError_;
        firstError_ = 0;
        return rc;
    }
    // Nothing submitted that has not finished (a blocking operation may then run on the caller's thread without overtaking
    // anything queued before it).
    bool Idle()
    {
        std::lock_guard<std::mutex> g(mu_);
        return finished_ >= submitted_;
    }
    uint64_t Submitted()
    {
        std::lock_guard<std::mutex> g(mu_);
        return submitted_;
    }
    uint64_t Finished()
    {
        std::lock_guard<std::mutex> g(mu_);
        return finished_;
    }

private:
    std::mutex mu_;
    std::condition_variable cv_;
    uint64_t submitted_{0};
    uint64_t finished_{0};
    int firstError_{0};
};

}  // namespace transport
}  // namespace mf
