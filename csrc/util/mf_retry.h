// Bounded retry with growing pauses for operations that a reconnect or a restarted peer can cure.
//
// Policy of the reference's host transport (src/hybm/csrc/transport/host/host_hcom_transport_manager.cpp:865-883, 959-977):
// three attempts, a pause of 1 s before the second and 2 s before the third, and between attempts the link state is thrown
// away and set up afresh ("forced reconnect"). Here the same policy wraps the steps that depend on another process being
// there: fetching a peer's file descriptor and a transfer-engine transfer (whose refresh step re-reads the peer's records
// from the store and maps its memory again).
#pragma once
#include <unistd.h>

#include <atomic>
#include <cstdint>

namespace mf {

struct RetryPolicy {
    uint32_t attempts{3};
    uint32_t firstDelayMs{1000};  // pause before attempt 2; every later pause is `factor` times the previous one
    uint32_t factor{2};
    uint32_t DelayMs(uint32_t failedAttempts) const
    {
        uint64_t d = firstDelayMs;
        for (uint32_t i = 1; i < failedAttempts; i++) {
            d *= factor;
        }
        return d > 60000 ? 60000 : (uint32_t)d;
    }
};

// Process-wide policy (tests shorten the pauses). Defined in the core library so that every module of the process shares it.
RetryPolicy &GlobalRetryPolicy();

// Counters for observability and tests.
struct RetryStats {
    std::atomic<uint64_t> retries{0};
    std::atomic<uint64_t> gaveUp{0};
};
RetryStats &GlobalRetryStats();

// Runs attempt() until it returns true or the policy is exhausted; beforeRetry(n) runs after the pause that follows the n-th
// failure (n = 1, 2, ...) and is the place to drop and rebuild link state. Returns whether an attempt succeeded.
template <typename Attempt, typename BeforeRetry>
bool RetryWithBackoff(Attempt attempt, BeforeRetry beforeRetry)
{
    const RetryPolicy pol = GlobalRetryPolicy();
    for (uint32_t failed = 0;;) {
        if (attempt()) {
            return true;
        }
        failed++;
        if (failed >= pol.attempts) {
            GlobalRetryStats().gaveUp.fetch_add(1);
            return false;
        }
        GlobalRetryStats().retries.fetch_add(1);
        usleep((useconds_t)pol.DelayMs(failed) * 1000);
        beforeRetry(failed);
    }
}

}  // namespace mf
