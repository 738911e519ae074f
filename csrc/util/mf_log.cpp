#include "mf_log.h"

#include <cstdlib>
#include <ctime>
#include <sys/time.h>

namespace mf {

static const char *kLevelNames[] = {"DEBUG", "INFO", "WARN", "ERROR", "FATAL"};

Logger::Logger()
{
    // MF_LOG_LEVEL (or the reference's ASCEND_MF_LOG_LEVEL) preselects the level: 0 debug … 3 error.
    const char *env = std::getenv("MF_LOG_LEVEL");
    if (env == nullptr) {
        env = std::getenv("ASCEND_MF_LOG_LEVEL");
    }
    if (env != nullptr && env[0] >= '0' && env[0] <= '5' && env[1] == '\0') {
        level_.store(env[0] - '0');
    }
}

Logger &Logger::Instance()
{
    static Logger *inst = new Logger();  // leaked on purpose: usable during static destruction / atfork
    return *inst;
}

void Logger::Write(int level, const char *file, int line, const std::string &msgIn)
{
    if (level < level_.load() || level >= LOG_OFF) {
        return;
    }
    std::string msg = msgIn;
    for (auto &c : msg) {
        if (c == '\n' || c == '\r') {
            c = ' ';
        }
    }
    const char *base = std::strrchr(file, '/');
    base = base ? base + 1 : file;
    ExternLogFn ext = extern_.load();
    if (ext != nullptr) {
        std::ostringstream oss;
        oss << base << ":" << line << " " << msg;
        ext(level, oss.str().c_str());
        return;
    }
    struct timeval tv;
    gettimeofday(&tv, nullptr);
    struct tm tmv;
    time_t sec = tv.tv_sec;
    localtime_r(&sec, &tmv);
    char ts[64];
    strftime(ts, sizeof(ts), "%Y-%m-%d %H:%M:%S", &tmv);
    std::lock_guard<std::mutex> g(mu_);
    fprintf(stdout, "%s.%06ld %s [%d-%ld] %s:%d %s\n", ts, (long)tv.tv_usec, kLevelNames[level], (int)getpid(),
            (long)syscall(SYS_gettid), base, line, msg.c_str());
    fflush(stdout);
}

bool Logger::Throttle(int burst, int windowSec)
{
    thread_local uint64_t windowStart = 0;
    thread_local int used = 0;
    uint64_t now = NowMs();
    if (now - windowStart > (uint64_t)windowSec * 1000ull) {
        windowStart = now;
        used = 0;
    }
    return used++ < burst;
}

static thread_local std::string g_lastErr;
static thread_local std::string g_lastErrOut;

void LastError::Set(const std::string &s) { g_lastErr = s; }
const char *LastError::Get() { return g_lastErr.c_str(); }
const char *LastError::GetAndClear()
{
    g_lastErrOut.swap(g_lastErr);
    g_lastErr.clear();
    return g_lastErrOut.c_str();
}

}  // namespace mf
