// Logging, thread-local last-error text and small helpers shared by every host component.
//
// Behaviour mirrors the reference logger (src/util/csrc/mf_out_logger.h:54-218): four levels, a default sink
// that prints "<time> <level> [pid-tid] file:line msg" to stdout, an external sink hook, and a per-thread
// rate-limited variant. The last-error API follows src/smem/csrc/common/smem_last_error.h.
#pragma once
#include <atomic>
#include <chrono>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <sstream>
#include <string>
#include <sys/syscall.h>
#include <unistd.h>

namespace mf {

enum LogLevel : int { LOG_DEBUG = 0, LOG_INFO = 1, LOG_WARN = 2, LOG_ERROR = 3, LOG_FATAL = 4, LOG_OFF = 5 };

using ExternLogFn = void (*)(int level, const char *msg);

class Logger {
public:
    static Logger &Instance();
    void SetLevel(int lv) { level_.store(lv); }
    int Level() const { return level_.load(); }
    void SetExtern(ExternLogFn fn) { extern_.store(fn); }
    void Write(int level, const char *file, int line, const std::string &msg);
    // At most `burst` messages per `windowSec` seconds per calling thread (reference: 5 per 7 s).
    bool Throttle(int burst = 5, int windowSec = 7);

private:
    Logger();
    std::atomic<int> level_{LOG_WARN};
    std::atomic<ExternLogFn> extern_{nullptr};
    std::mutex mu_;
};

// Thread-local last error text: Set() overwrites, Get() peeks, GetAndClear() drains.
struct LastError {
    static void Set(const std::string &s);
    static const char *Get();
    static const char *GetAndClear();
};

inline uint64_t NowNs()
{
    return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
               std::chrono::steady_clock::now().time_since_epoch())
        .count();
}
inline uint64_t NowMs() { return NowNs() / 1000000ull; }

}  // namespace mf

#define MF_LOG_AT(lv, expr)                                                    \
    do {                                                                       \
        if ((lv) >= ::mf::Logger::Instance().Level()) {                        \
            std::ostringstream mf_oss_;                                        \
            mf_oss_ << expr;                                                   \
            ::mf::Logger::Instance().Write((lv), __FILE__, __LINE__, mf_oss_.str()); \
        }                                                                      \
    } while (0)

#define MF_DEBUG(expr) MF_LOG_AT(::mf::LOG_DEBUG, expr)
#define MF_INFO(expr) MF_LOG_AT(::mf::LOG_INFO, expr)
#define MF_WARN(expr) MF_LOG_AT(::mf::LOG_WARN, expr)
// Errors are also remembered as the calling thread's last error so that bindings can surface them.
#define MF_ERROR(expr)                                  \
    do {                                                \
        std::ostringstream mf_eoss_;                    \
        mf_eoss_ << expr;                               \
        ::mf::LastError::Set(mf_eoss_.str());           \
        MF_LOG_AT(::mf::LOG_ERROR, mf_eoss_.str());     \
    } while (0)
#define MF_ERROR_LIMIT(expr)                                 \
    do {                                                     \
        if (::mf::Logger::Instance().Throttle()) { MF_ERROR(expr); } \
    } while (0)

#define MF_WARN_LIMIT(expr)                                 \
    do {                                                    \
        if (::mf::Logger::Instance().Throttle()) { MF_WARN(expr); } \
    } while (0)

#define MF_CHECK_RET(cond, ret, expr) \
    do {                              \
        if (!(cond)) {                \
            MF_ERROR(expr);           \
            return (ret);             \
        }                             \
    } while (0)
