#include "mf_file_util.h"
#include "mf_tracer.h"

#include <condition_variable>
#include <cstdio>
#include <mutex>
#include <sstream>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>

#include "mf_log.h"

namespace mf {

struct Tracer::Impl {
    TracePoint table[TRACE_MODULES][TRACE_IDS_PER_MODULE];
    std::thread dumper;
    std::mutex mu;
    std::condition_variable cv;
    bool stop{false};
    std::string path;
    int periodSec{10};
};

static constexpr long kMaxDumpBytes = 10L * 1024 * 1024;  // file is overwritten from the start past this size

Tracer &Tracer::Instance()
{
    static Tracer *t = new Tracer();
    return *t;
}

TracePoint *Tracer::At(int tp)
{
    int m = (tp >> 8) & 0xff, i = tp & 0xff;
    if (impl_ == nullptr || m >= TRACE_MODULES || i >= TRACE_IDS_PER_MODULE) {
        return nullptr;
    }
    return &impl_->table[m][i];
}

int Tracer::Init(const std::string &dumpDir, int periodSec)
{
    if (impl_ != nullptr) {
        enabled_.store(true);
        return 0;
    }
    impl_ = new Impl();
    impl_->periodSec = periodSec;
    enabled_.store(true);
    if (!dumpDir.empty()) {
        std::string dir = dumpDir;
        if (!util::MakeDirs(dir, 0750) || !util::Canonicalize(&dir) || !util::Writable(dir)) {
            MF_WARN("tracer: dump directory " << dumpDir << " cannot be created or written; periodic dumps are off");
            return 0;
        }
        impl_->path = dir + "/mf_tracer_" + std::to_string((int)getpid()) + ".dat";
        impl_->dumper = std::thread([this]() {
            std::unique_lock<std::mutex> lk(impl_->mu);
            while (!impl_->stop) {
                impl_->cv.wait_for(lk, std::chrono::seconds(impl_->periodSec));
                if (impl_->stop) {
                    break;
                }
                lk.unlock();
                std::string text = Dump(false);
                FILE *f = fopen(impl_->path.c_str(), "a");
                if (f != nullptr) {
                    if (ftell(f) > kMaxDumpBytes) {
                        f = freopen(impl_->path.c_str(), "w", f);
                    }
                    if (f != nullptr) {
                        fwrite(text.data(), 1, text.size(), f);
                        fclose(f);
                    }
                }
                lk.lock();
            }
        });
    }
    return 0;
}

void Tracer::Shutdown()
{
    enabled_.store(false);
    if (impl_ == nullptr) {
        return;
    }
    {
        std::lock_guard<std::mutex> g(impl_->mu);
        impl_->stop = true;
    }
    impl_->cv.notify_all();
    if (impl_->dumper.joinable()) {
        impl_->dumper.join();
    }
    // The table is kept (tracepoints may still be referenced by late scopes); only the thread ends.
    impl_->stop = false;
}

void Tracer::Begin(int tp, const char *name)
{
    TracePoint *p = At(tp);
    if (p == nullptr) {
        return;
    }
    if (p->name == nullptr) {
        p->name = name;
    }
    p->begin.fetch_add(1, std::memory_order_relaxed);
}

void Tracer::End(int tp, uint64_t startNs, int ret)
{
    TracePoint *p = At(tp);
    if (p == nullptr) {
        return;
    }
    uint64_t d = NowNs() - startNs;
    (ret == 0 ? p->good : p->bad).fetch_add(1, std::memory_order_relaxed);
    p->totalNs.fetch_add(d, std::memory_order_relaxed);
    uint64_t cur = p->minNs.load(std::memory_order_relaxed);
    while (d < cur && !p->minNs.compare_exchange_weak(cur, d)) {
    }
    cur = p->maxNs.load(std::memory_order_relaxed);
    while (d > cur && !p->maxNs.compare_exchange_weak(cur, d)) {
    }
}

bool Tracer::Query(int tp, uint64_t out[4])
{
    TracePoint *p = At(tp);
    if (p == nullptr) {
        return false;
    }
    out[0] = p->begin.load();
    out[1] = p->good.load();
    out[2] = p->bad.load();
    out[3] = p->totalNs.load();
    return true;
}

std::string Tracer::Dump(bool reset)
{
    std::ostringstream oss;
    if (impl_ == nullptr) {
        return oss.str();
    }
    char line[256];
    snprintf(line, sizeof(line), "%-36s %10s %10s %8s %12s %12s %12s %14s\n", "TP_NAME", "BEGIN", "GOOD_END", "BAD_END",
             "MIN(us)", "MAX(us)", "AVG(us)", "TOTAL(us)");
    oss << line;
    for (int m = 0; m < TRACE_MODULES; m++) {
        for (int i = 0; i < TRACE_IDS_PER_MODULE; i++) {
            TracePoint &p = impl_->table[m][i];
            uint64_t b = p.begin.load();
            if (b == 0 || p.name == nullptr) {
                continue;
            }
            uint64_t ends = p.good.load() + p.bad.load();
            double tot = p.totalNs.load() / 1e3;
            double mn = p.minNs.load() == UINT64_MAX ? 0.0 : p.minNs.load() / 1e3;
            snprintf(line, sizeof(line), "%-36s %10lu %10lu %8lu %12.3f %12.3f %12.3f %14.3f\n", p.name, (unsigned long)b,
                     (unsigned long)p.good.load(), (unsigned long)p.bad.load(), mn, p.maxNs.load() / 1e3,
                     ends ? tot / ends : 0.0, tot);
            oss << line;
            if (reset) {
                p.begin = 0;
                p.good = 0;
                p.bad = 0;
                p.totalNs = 0;
                p.minNs = UINT64_MAX;
                p.maxNs = 0;
            }
        }
    }
    return oss.str();
}

TraceScope::TraceScope(int tpId, const char *name, int *retPtr) : tp(tpId), t0(0), ret(retPtr)
{
    if (Tracer::Instance().Enabled()) {
        t0 = NowNs();
        Tracer::Instance().Begin(tp, name);
    }
}

TraceScope::~TraceScope()
{
    if (t0 != 0) {
        Tracer::Instance().End(tp, t0, ret ? *ret : 0);
    }
}

}  // namespace mf
