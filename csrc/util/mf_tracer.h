// Aggregate tracepoint recorder (count / good / bad / min / max / total ns per tracepoint id) with an optional
// periodic dump thread. Same role as the reference's ptracer (src/util/csrc/ptracer/include/ptracer.h:15-77,
// table layout ptracer_tracepoint.h:12-249, text dump doc/ptracer.md:20-38). Disabled tracepoints cost one branch.
#pragma once
#include <atomic>
#include <cstdint>
#include <string>

namespace mf {

constexpr int TRACE_MODULES = 16;
constexpr int TRACE_IDS_PER_MODULE = 128;

// Tracepoint ids: (module << 8) | index. Names are registered on first use.
enum TraceModule : int { TM_STORE = 0, TM_GROUP = 1, TM_HYBM = 2, TM_DATAOP = 3, TM_BM = 4, TM_SHM = 5, TM_TRANS = 6, TM_KERNEL = 7 };
#define MF_TP(module, idx) (((module) << 8) | (idx))

struct TracePoint {
    std::atomic<uint64_t> begin{0}, good{0}, bad{0}, totalNs{0};
    std::atomic<uint64_t> minNs{UINT64_MAX}, maxNs{0};
    const char *name{nullptr};
};

class Tracer {
public:
    static Tracer &Instance();
    // dumpDir empty: no dump thread (text is still available through Dump()).
    int Init(const std::string &dumpDir, int periodSec = 10);
    void Shutdown();
    bool Enabled() const { return enabled_.load(std::memory_order_relaxed); }
    void Enable(bool on) { enabled_.store(on); }
    void Begin(int tp, const char *name);
    void End(int tp, uint64_t startNs, int ret);
    std::string Dump(bool reset = false);
    // (count, goodCount, badCount, totalNs) for tests.
    bool Query(int tp, uint64_t out[4]);

private:
    Tracer() = default;
    TracePoint *At(int tp);
    std::atomic<bool> enabled_{false};
    struct Impl;
    Impl *impl_{nullptr};
};

struct TraceScope {
    int tp;
    uint64_t t0;
    int *ret;
    TraceScope(int tpId, const char *name, int *retPtr);
    ~TraceScope();
};

}  // namespace mf

// Usage: int ret = 0; MF_TRACE_SCOPE(MF_TP(TM_DATAOP, 3), "COPY_GD_TO_GD", &ret);
#define MF_TRACE_SCOPE(tp, name, retPtr) ::mf::TraceScope mf_trace_scope_##__LINE__((tp), (name), (retPtr))
