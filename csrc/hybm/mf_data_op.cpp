#include "mf_data_op.h"
#include "mf_range_pool.h"

#include <deque>
#include <memory>

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstdlib>
#include <functional>
#include <mutex>
#include <cstring>
#include <thread>
#include <unistd.h>
#include <unordered_map>

#include "../kernels/mf_kernels.h"
#include "../util/mf_log.h"
#include "../util/mf_tracer.h"
#include "mf_cuda.h"
#include "mf_tag_info.h"

namespace mf {
namespace hybm {

uint32_t DefaultSyncTimeoutMs()
{
    static uint32_t v = []() {
        const char *e = std::getenv("MF_COPY_TIMEOUT_MS");
        long t = e != nullptr ? std::strtol(e, nullptr, 10) : 0;
        return (uint32_t)(t > 0 ? t : 30000);
    }();
    return v;
}

int BoundedStreamSync(int device, void *stream, uint32_t timeoutMs)
{
    cudaStream_t s = stream != nullptr ? (cudaStream_t)stream : cu::ThreadStream(device);
    // Fast path: most copies finish within the first few hundred polls.
    uint64_t deadline = NowNs() + (uint64_t)timeoutMs * 1000000ull;
    uint32_t spins = 0;
    while (true) {
        cudaError_t e = cudaStreamQuery(s);
        if (e == cudaSuccess) {
            return BM_OK;
        }
        if (e != cudaErrorNotReady) {
            MF_ERROR("data op: stream reported " << cu::ErrStr(e));
            (void)cudaGetLastError();
            return BM_ERROR;
        }
        if (++spins > 2000) {
            if (NowNs() > deadline) {
                MF_ERROR("data op: copy did not complete within " << timeoutMs << " ms");
                return BM_TIMEOUT;
            }
            if (spins > 200000) {
                usleep(50);
            }
        }
    }
}

// =============================================================================================== kernel engine

namespace {

// Staging space for copy tables that do not fit the kernel parameters: one pinned host block and one device block of the same
// size per thread, carved up by a range pool (the reference's RbtreeRangePool serves its staging buffers the same way,
// src/hybm/csrc/common/hybm_rbtree_range_pool.{h,cpp}). A table's range is handed back when the kernel that reads it has
// finished, which an event recorded AFTER the launch tells. Nothing is allocated on the request path once the arena exists;
// a table larger than the arena makes it grow, once.
struct StageArena {
    char *host{nullptr};
    char *dev{nullptr};
    size_t cap{0};
    std::unique_ptr<RangePool> pool;
    struct InFlight {
        uint64_t off;
        cudaEvent_t ev;
    };
    std::deque<InFlight> inflight;
    std::vector<cudaEvent_t> freeEvents;
};
constexpr size_t kArenaBase = 256;  // offsets handed out by the pool start here: 0 means "no room"
constexpr size_t kArenaDefault = 2u << 20;

struct ThreadCtx {
    volatile uint32_t *flag{nullptr};  // pinned host word, device-visible under the same address
    uint32_t *counter{nullptr};        // device word, self-resetting
    uint32_t seq{0};
    StageArena arena;
    std::vector<mf_copy_desc_t> scratch;
};

class KernelDataOp : public DataOperator {
public:
    explicit KernelDataOp(int device) : device_(device) {}
    uint32_t Type() const override { return OP_KERNEL_LDST; }
    const char *Name() const override { return "kernel_ldst"; }

    int Initialize() override
    {
        MF_CHECK_RET(cu::Available() && device_ >= 0, BM_NOT_SUPPORTED, "kernel engine: no GPU");
        MF_CUDA_CHECK_RET(cudaSetDevice(device_), BM_ERROR);
        const char *e = std::getenv("MF_BATCH_SYNC");
        flagSync_ = !(e != nullptr && std::strcmp(e, "stream") == 0);
        return BM_OK;
    }

    bool Supports(CopyDirection dir, const ExtOptions &opt) const override
    {
        return dir < DIR_AUTO && opt.srcDeviceVisible && opt.dstDeviceVisible;
    }

    int DataCopy(const CopyParams &p, CopyDirection dir, const ExtOptions &opt) override
    {
        if (!Supports(dir, opt)) {
            return BM_NOT_SUPPORTED;
        }
        cudaStream_t s = opt.stream != nullptr ? (cudaStream_t)opt.stream : cu::ThreadStream(device_);
        int rc = mf_k_xcopy(p.dest, p.src, p.dataSize, 0, (mf_stream_t)s);
        if (rc != MF_K_OK) {
            MF_ERROR("kernel engine: xcopy launch failed");
            return BM_ERROR;
        }
        if (opt.flags & FLAG_ASYNC_COPY) {
            return BM_OK;
        }
        return BoundedStreamSync(device_, s, DefaultSyncTimeoutMs());
    }

    int BatchDataCopy(const BatchCopyParams &p, CopyDirection dir, const ExtOptions &opt) override
    {
        if (!Supports(dir, opt)) {
            return BM_NOT_SUPPORTED;
        }
        ThreadCtx *ctx = Ctx();
        MF_CHECK_RET(ctx != nullptr, BM_ERROR, "kernel engine: cannot set up the per-thread batch context");
        cudaStream_t s = opt.stream != nullptr ? (cudaStream_t)opt.stream : cu::ThreadStream(device_);
        // 1. Coalesce runs that are contiguous on both sides, split anything too long for a 32-bit length.
        std::vector<mf_copy_desc_t> &d = ctx->scratch;
        d.clear();
        constexpr uint64_t kMaxLen = 1ull << 31;
        uint32_t chunks = 0;
        auto push = [&](uint64_t src, uint64_t dst, uint64_t len) {
            while (len > 0) {
                uint64_t part = std::min(len, kMaxLen);
                d.push_back(mf_copy_desc_t{src, dst, (uint32_t)part, 0});
                src += part;
                dst += part;
                len -= part;
            }
        };
        uint64_t curS = 0, curD = 0, curL = 0;
        for (uint32_t i = 0; i < p.batchSize; i++) {
            uint64_t sa = (uint64_t)p.sources[i], da = (uint64_t)p.destinations[i], len = p.dataSizes[i];
            if (len == 0) {
                continue;
            }
            if (curL != 0 && sa == curS + curL && da == curD + curL) {
                curL += len;
                continue;
            }
            if (curL != 0) {
                push(curS, curD, curL);
            }
            curS = sa;
            curD = da;
            curL = len;
        }
        if (curL != 0) {
            push(curS, curD, curL);
        }
        if (d.empty()) {
            return BM_OK;
        }
        for (auto &e : d) {
            e.chunkStart = chunks;
            chunks += (e.len + MF_BATCH_CHUNK_BYTES - 1) / MF_BATCH_CHUNK_BYTES;
        }
        const bool sync = !(opt.flags & FLAG_ASYNC_COPY);
        const bool useFlag = sync && flagSync_ && opt.stream == nullptr;
        const mf_copy_desc_t *devTable = nullptr;
        uint64_t stagedOff = 0;
        if (d.size() > MF_BATCH_INLINE_MAX) {
            // 2. Large tables: stage in pinned memory and copy to the device ahead of the kernel, on the same stream.
            // Table layout: descriptors, then one uint32 per chunk naming its descriptor.
            const size_t descBytes = d.size() * sizeof(mf_copy_desc_t);
            const size_t bytes = descBytes + (size_t)chunks * sizeof(uint32_t);
            int arc = StageAlloc(ctx->arena, bytes, s, &stagedOff);
            if (arc != BM_OK) {
                return arc;
            }
            char *host = ctx->arena.host + stagedOff;
            std::memcpy(host, d.data(), descBytes);
            uint32_t *map = reinterpret_cast<uint32_t *>(host + descBytes);
            for (uint32_t i = 0; i < d.size(); i++) {
                const uint32_t n = (d[i].len + MF_BATCH_CHUNK_BYTES - 1) / MF_BATCH_CHUNK_BYTES;
                for (uint32_t c = 0; c < n; c++) {
                    map[d[i].chunkStart + c] = i;
                }
            }
            MF_CUDA_CHECK_RET(cudaMemcpyAsync(ctx->arena.dev + stagedOff, host, bytes, cudaMemcpyHostToDevice, s), BM_ERROR);
            devTable = reinterpret_cast<const mf_copy_desc_t *>(ctx->arena.dev + stagedOff);
        }
        uint32_t seq = ++ctx->seq;
        int rc = mf_k_batch_xcopy(d.data(), devTable, (uint32_t)d.size(), chunks, useFlag ? ctx->counter : nullptr,
                                  useFlag ? ctx->flag : nullptr, seq, 0, (mf_stream_t)s);
        if (stagedOff != 0) {
            StageRetire(ctx->arena, stagedOff, s);  // the range is free again once this kernel has run
        }
        if (rc != MF_K_OK) {
            MF_ERROR("kernel engine: batch launch failed");
            return BM_ERROR;
        }
        if (!sync) {
            return BM_OK;
        }
        if (useFlag) {
            // 3. Completion word written by the last CTA; bounded poll, then fall back to the stream for the verdict.
            uint64_t deadline = NowNs() + (uint64_t)DefaultSyncTimeoutMs() * 1000000ull;
            uint32_t spins = 0;
            while (*ctx->flag != seq) {
                if ((++spins & 0x3ff) == 0 && NowNs() > deadline) {
                    MF_ERROR("kernel engine: batch completion word not seen in time");
                    return BM_TIMEOUT;
                }
            }
            return BM_OK;
        }
        return BoundedStreamSync(device_, s, DefaultSyncTimeoutMs());
    }

    int Wait() override { return BoundedStreamSync(device_, nullptr, DefaultSyncTimeoutMs()); }

private:
    // Hands back the ranges whose kernels have finished; with `block` it waits for the oldest one.
    static void StageReclaim(StageArena &a, bool block)
    {
        while (!a.inflight.empty()) {
            StageArena::InFlight &f = a.inflight.front();
            cudaError_t q = block ? cudaEventSynchronize(f.ev) : cudaEventQuery(f.ev);
            if (q != cudaSuccess) {
                (void)cudaGetLastError();
                return;
            }
            a.pool->Release(f.off);
            a.freeEvents.push_back(f.ev);
            a.inflight.pop_front();
            block = false;
        }
    }

    int StageAlloc(StageArena &a, size_t bytes, cudaStream_t s, uint64_t *off)
    {
        if (a.pool) {
            StageReclaim(a, false);
        }
        if (!a.pool || bytes + kArenaBase > a.cap) {
            // First use, or a table larger than the whole arena: (re)build it. Tables in flight still read the old blocks.
            if (a.pool) {
                cudaStreamSynchronize(s);
                while (!a.inflight.empty()) {
                    StageReclaim(a, true);
                }
                cudaFreeHost(a.host);
                cudaFree(a.dev);
                a.host = a.dev = nullptr;
            }
            size_t cap = kArenaDefault;
            while (cap < 2 * bytes + kArenaBase) {
                cap *= 2;
            }
            MF_CUDA_CHECK_RET(cudaHostAlloc((void **)&a.host, cap, cudaHostAllocDefault), BM_MALLOC_FAILED);
            MF_CUDA_CHECK_RET(cudaMalloc((void **)&a.dev, cap), BM_MALLOC_FAILED);
            a.cap = cap;
            a.pool.reset(new RangePool(kArenaBase, cap - kArenaBase, 256));
        }
        uint64_t o = a.pool->Allocate(bytes);
        while (o == 0 && !a.inflight.empty()) {
            StageReclaim(a, true);  // full: wait for the oldest table to be consumed
            o = a.pool->Allocate(bytes);
        }
        MF_CHECK_RET(o != 0, BM_MALLOC_FAILED, "kernel engine: no staging space for a table of " << bytes << " bytes");
        *off = o;
        return BM_OK;
    }

    static void StageRetire(StageArena &a, uint64_t off, cudaStream_t s)
    {
        cudaEvent_t ev = nullptr;
        if (!a.freeEvents.empty()) {
            ev = a.freeEvents.back();
            a.freeEvents.pop_back();
        } else if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) {
            (void)cudaGetLastError();
            cudaStreamSynchronize(s);  // no event to be had: wait right here and free the range
            a.pool->Release(off);
            return;
        }
        cudaEventRecord(ev, s);
        a.inflight.push_back(StageArena::InFlight{off, ev});
    }

    ThreadCtx *Ctx()
    {
        thread_local std::unordered_map<const KernelDataOp *, ThreadCtx> ctxs;
        ThreadCtx &c = ctxs[this];
        if (c.flag == nullptr) {
            cudaSetDevice(device_);
            void *hp = nullptr;
            if (cudaHostAlloc(&hp, 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
                (void)cudaGetLastError();
                return nullptr;
            }
            std::memset(hp, 0, 64);
            void *dp = nullptr;
            if (cudaMalloc(&dp, 64) != cudaSuccess || cudaMemset(dp, 0, 64) != cudaSuccess) {
                (void)cudaGetLastError();
                cudaFreeHost(hp);
                return nullptr;
            }
            c.flag = (volatile uint32_t *)hp;
            c.counter = (uint32_t *)dp;
        }
        return &c;
    }

    int device_;
    bool flagSync_{true};
};

// =============================================================================================== copy engine

class CopyEngineDataOp : public DataOperator {
public:
    explicit CopyEngineDataOp(int device) : device_(device) {}
    uint32_t Type() const override { return OP_COPY_ENGINE; }
    const char *Name() const override { return "copy_engine"; }
    int Initialize() override
    {
        MF_CHECK_RET(cu::Available() && device_ >= 0, BM_NOT_SUPPORTED, "copy engine: no GPU");
        return BM_OK;
    }
    bool Supports(CopyDirection dir, const ExtOptions &) const override { return dir < DIR_AUTO; }

    int DataCopy(const CopyParams &p, CopyDirection, const ExtOptions &opt) override
    {
        cudaStream_t s = opt.stream != nullptr ? (cudaStream_t)opt.stream : cu::ThreadStream(device_);
        MF_CUDA_CHECK_RET(cudaMemcpyAsync(p.dest, p.src, p.dataSize, cudaMemcpyDefault, s), BM_ERROR);
        if (opt.flags & FLAG_ASYNC_COPY) {
            return BM_OK;
        }
        return BoundedStreamSync(device_, s, DefaultSyncTimeoutMs());
    }

    int BatchDataCopy(const BatchCopyParams &p, CopyDirection, const ExtOptions &opt) override
    {
        cudaStream_t s = opt.stream != nullptr ? (cudaStream_t)opt.stream : cu::ThreadStream(device_);
        // One cudaMemcpyAsync per coalesced run.
        uint64_t curS = 0, curD = 0, curL = 0;
        auto flush = [&]() -> int {
            if (curL == 0) {
                return BM_OK;
            }
            MF_CUDA_CHECK_RET(cudaMemcpyAsync((void *)curD, (const void *)curS, curL, cudaMemcpyDefault, s), BM_ERROR);
            return BM_OK;
        };
        for (uint32_t i = 0; i < p.batchSize; i++) {
            uint64_t sa = (uint64_t)p.sources[i], da = (uint64_t)p.destinations[i], len = p.dataSizes[i];
            if (len == 0) {
                continue;
            }
            if (curL != 0 && sa == curS + curL && da == curD + curL) {
                curL += len;
                continue;
            }
            int rc = flush();
            if (rc != BM_OK) {
                return rc;
            }
            curS = sa;
            curD = da;
            curL = len;
        }
        int rc = flush();
        if (rc != BM_OK) {
            return rc;
        }
        if (opt.flags & FLAG_ASYNC_COPY) {
            return BM_OK;
        }
        return BoundedStreamSync(device_, s, DefaultSyncTimeoutMs());
    }

    int Wait() override { return BoundedStreamSync(device_, nullptr, DefaultSyncTimeoutMs()); }

private:
    int device_;
};

// =============================================================================================== CPU engine

// A few helper threads that stay around for large host copies and for batches of them: spawning threads per call costs more
// than a 4 MiB copy takes. One job at a time; a caller that finds the pool busy (or in a forked child, where the threads do
// not exist) copies on its own thread.
class CopyPool {
public:
    static CopyPool &Get()
    {
        static CopyPool *pool = new CopyPool();  // never destroyed: its threads may outlive static destruction order
        return *pool;
    }
    unsigned Width() const { return helpers_ + 1; }
    // Runs fn(0..parts-1) on the helpers and the caller. False: nothing ran (pool busy or unusable), the caller does the work.
    bool Run(unsigned parts, const std::function<void(unsigned)> &fn)
    {
        if (helpers_ == 0 || parts < 2 || ownerPid_ != getpid()) {
            return false;
        }
        std::unique_lock<std::mutex> job(jobMu_, std::try_to_lock);
        if (!job.owns_lock()) {
            return false;
        }
        {
            std::lock_guard<std::mutex> g(mu_);
            fn_ = &fn;
            parts_ = parts;
            next_.store(0);
            pendingHelpers_ = helpers_;
            generation_++;
        }
        cv_.notify_all();
        Work();
        std::unique_lock<std::mutex> lk(mu_);
        doneCv_.wait(lk, [this]() { return pendingHelpers_ == 0; });
        fn_ = nullptr;
        return true;
    }

private:
    CopyPool()
    {
        unsigned hw = std::thread::hardware_concurrency();
        helpers_ = hw >= 4 ? std::min(3u, hw / 2 - 1) : 0;
        ownerPid_ = getpid();
        for (unsigned i = 0; i < helpers_; i++) {
            std::thread([this]() { HelperLoop(); }).detach();
        }
    }
    void Work()
    {
        for (unsigned i = next_.fetch_add(1); i < parts_; i = next_.fetch_add(1)) {
            (*fn_)(i);
        }
    }
    void HelperLoop()
    {
        uint64_t seen = 0;
        std::unique_lock<std::mutex> lk(mu_);
        while (true) {
            cv_.wait(lk, [&]() { return generation_ != seen; });
            seen = generation_;
            lk.unlock();
            Work();
            lk.lock();
            if (--pendingHelpers_ == 0) {
                doneCv_.notify_one();
            }
        }
    }
    std::mutex jobMu_, mu_;
    std::condition_variable cv_, doneCv_;
    const std::function<void(unsigned)> *fn_{nullptr};
    unsigned parts_{0}, helpers_{0}, pendingHelpers_{0};
    std::atomic<unsigned> next_{0};
    uint64_t generation_{0};
    pid_t ownerPid_{0};
};

void ParallelMemcpy(void *dst, const void *src, size_t n)
{
    constexpr size_t kParallelMin = 2ull << 20, kPiece = 512ull << 10;
    if (n >= kParallelMin) {
        const unsigned parts = (unsigned)((n + kPiece - 1) / kPiece);
        if (CopyPool::Get().Run(parts, [&](unsigned i) {
                const size_t off = (size_t)i * kPiece;
                std::memcpy((char *)dst + off, (const char *)src + off, std::min(kPiece, n - off));
            })) {
            return;
        }
    }
    std::memcpy(dst, src, n);
}

class CpuDataOp : public DataOperator {
public:
    uint32_t Type() const override { return OP_HOST_RDMA | OP_HOST_TCP | OP_HOST_URMA; }
    const char *Name() const override { return "cpu_memcpy"; }
    bool Supports(CopyDirection dir, const ExtOptions &) const override
    {
        // Host-to-host legs only: the CPU cannot dereference HBM.
        return dir == DIR_LH_TO_GH || dir == DIR_GH_TO_LH || dir == DIR_GH_TO_GH;
    }
    int DataCopy(const CopyParams &p, CopyDirection dir, const ExtOptions &opt) override
    {
        if (!Supports(dir, opt)) {
            return BM_NOT_SUPPORTED;
        }
        ParallelMemcpy(p.dest, p.src, p.dataSize);
        return BM_OK;
    }
    int BatchDataCopy(const BatchCopyParams &p, CopyDirection dir, const ExtOptions &opt) override
    {
        if (!Supports(dir, opt)) {
            return BM_NOT_SUPPORTED;
        }
        // Many small elements: spread the elements over the pool; few large ones: spread each of them.
        uint64_t total = 0;
        for (uint32_t i = 0; i < p.batchSize; i++) {
            total += p.dataSizes[i];
        }
        if (p.batchSize >= 8 && total >= (4ull << 20) &&
            CopyPool::Get().Run(p.batchSize, [&](unsigned i) { std::memcpy(p.destinations[i], p.sources[i], p.dataSizes[i]); })) {
            return BM_OK;
        }
        for (uint32_t i = 0; i < p.batchSize; i++) {
            ParallelMemcpy(p.destinations[i], p.sources[i], p.dataSizes[i]);
        }
        return BM_OK;
    }
};

}  // namespace

std::shared_ptr<DataOperator> MakeKernelDataOp(int device) { return std::make_shared<KernelDataOp>(device); }
std::shared_ptr<DataOperator> MakeCopyEngineDataOp(int device) { return std::make_shared<CopyEngineDataOp>(device); }
std::shared_ptr<DataOperator> MakeCpuDataOp() { return std::make_shared<CpuDataOp>(); }

// =============================================================================================== compose

namespace {
std::atomic<uint64_t> g_served[6];
std::atomic<uint64_t> g_batchGroupsLast{0};
std::atomic<uint64_t> g_remote[2];

void NoteServed(uint32_t type, uint64_t elems)
{
    const int slot = type == OP_KERNEL_LDST ? 0 : (type == OP_COPY_ENGINE ? 1 : 2);
    g_served[2 * slot].fetch_add(1, std::memory_order_relaxed);
    g_served[2 * slot + 1].fetch_add(elems, std::memory_order_relaxed);
}
}  // namespace

DataOpStats GetDataOpStats()
{
    DataOpStats s;
    s.kernelCalls = g_served[0].load();
    s.kernelElems = g_served[1].load();
    s.copyEngineCalls = g_served[2].load();
    s.copyEngineElems = g_served[3].load();
    s.cpuCalls = g_served[4].load();
    s.cpuElems = g_served[5].load();
    s.batchGroupsLast = g_batchGroupsLast.load();
    s.remoteCalls = g_remote[0].load();
    s.remoteElems = g_remote[1].load();
    return s;
}

void NoteBatchGroups(uint32_t groups) { g_batchGroupsLast.store(groups, std::memory_order_relaxed); }

void NoteRemoteCopy(uint64_t elems)
{
    g_remote[0].fetch_add(1, std::memory_order_relaxed);
    g_remote[1].fetch_add(elems, std::memory_order_relaxed);
}

ComposeDataOp::ComposeDataOp(int device, uint32_t allowedOps, std::shared_ptr<TagInfo> tags)
    : device_(device), allowed_(allowedOps), tags_(std::move(tags))
{
}

int ComposeDataOp::Initialize()
{
    engines_.clear();
    const bool gpu = cu::Available() && device_ >= 0;
    if (gpu && (allowed_ & (OP_KERNEL_LDST | OP_DEVICE_RDMA | OP_COPY_ENGINE))) {
        // The two GPU engines back each other up: whichever the caller asked for, a failure of one falls through to
        // the other (reference: SDMA → DEVICE_RDMA → … fall-through, hybm_compose_data_op.cpp:94-111).
        auto k = MakeKernelDataOp(device_);
        if (k->Initialize() == BM_OK) {
            engines_.push_back(k);
        }
        auto c = MakeCopyEngineDataOp(device_);
        if (c->Initialize() == BM_OK) {
            engines_.push_back(c);
        }
    }
    engines_.push_back(MakeCpuDataOp());
    return BM_OK;
}

static bool HostOnly(CopyDirection d) { return d == DIR_LH_TO_GH || d == DIR_GH_TO_LH || d == DIR_GH_TO_GH; }
static bool TouchesHost(CopyDirection d)
{
    PtrClass s = SrcClassOf(d), t = DstClassOf(d);
    return s == PC_LOCAL_HOST || s == PC_GLOBAL_HOST || t == PC_LOCAL_HOST || t == PC_GLOBAL_HOST;
}

static uint64_t PeerCopyEngineMin()
{
    static const uint64_t v = []() -> uint64_t {
        const char *e = getenv("MF_PEER_COPY_ENGINE_MIN_MB");
        if (e == nullptr || e[0] == '\0') {
            return 0;
        }
        char *end = nullptr;
        unsigned long long mb = std::strtoull(e, &end, 10);
        return (end != nullptr && *end == '\0' && mb > 0 && mb < (1ull << 30)) ? mb << 20 : 0;
    }();
    return v;
}

std::vector<std::shared_ptr<DataOperator>> ComposeDataOp::Candidates(CopyDirection dir, const ExtOptions &opt, uint64_t bytes, bool batch) const
{
    uint32_t mask = allowed_;
    if (tags_) {
        mask = tags_->AllowedOps(opt.srcRank, opt.dstRank, allowed_);
    }
    // Rank order of preference for this call.
    std::vector<uint32_t> order;
    constexpr uint32_t kCpuBits = OP_HOST_RDMA | OP_HOST_TCP | OP_HOST_URMA;
    constexpr uint64_t kCopyEngineMin = 1ull << 20;
    if (HostOnly(dir)) {
        order = {kCpuBits, OP_COPY_ENGINE, OP_KERNEL_LDST};
    } else if (opt.flags & FLAG_COPY_KERNEL) {
        order = {OP_KERNEL_LDST, OP_COPY_ENGINE, kCpuBits};
    } else if (!opt.srcDeviceVisible || !opt.dstDeviceVisible) {
        order = {OP_COPY_ENGINE, kCpuBits};
    } else if (TouchesHost(dir) && !batch && bytes >= kCopyEngineMin) {
        order = {OP_COPY_ENGINE, OP_KERNEL_LDST, kCpuBits};  // big host legs: DMA engines saturate PCIe without SMs
    } else if (!batch && opt.srcRank != opt.dstRank && PeerCopyEngineMin() != 0 && bytes >= PeerCopyEngineMin()) {
        // Opt-in (MF_PEER_COPY_ENGINE_MIN_MB): large single transfers between GPUs ride the copy engine, whose packets
        // carry about a tenth more payload over NVLink than writes issued by SMs can; the SMs stay free for compute.
        order = {OP_COPY_ENGINE, OP_KERNEL_LDST, kCpuBits};
    } else {
        order = {OP_KERNEL_LDST, OP_COPY_ENGINE, kCpuBits};
    }
    std::vector<std::shared_ptr<DataOperator>> out;
    for (uint32_t want : order) {
        for (auto &e : engines_) {
            uint32_t t = e->Type();
            bool isCpu = (t & kCpuBits) != 0;
            // DEVICE_RDMA shares the kernel engine; host engines are always admissible for host-only legs.
            bool permitted = isCpu ? (HostOnly(dir) || (mask & kCpuBits)) : ((mask & t) || (t == OP_KERNEL_LDST && (mask & OP_DEVICE_RDMA)));
            if ((t & want) && permitted && e->Supports(dir, opt) && std::find(out.begin(), out.end(), e) == out.end()) {
                out.push_back(e);
            }
        }
    }
    return out;
}

int ComposeDataOp::DataCopy(const CopyParams &p, CopyDirection dir, const ExtOptions &opt)
{
    int ret = BM_NOT_SUPPORTED;
    MF_TRACE_SCOPE(MF_TP(TM_DATAOP, (int)dir), DirectionName(dir), &ret);
    auto cands = Candidates(dir, opt, p.dataSize, false);
    for (auto &e : cands) {
        ret = e->DataCopy(p, dir, opt);
        if (ret == BM_OK) {
            NoteServed(e->Type(), 1);
            return ret;
        }
        MF_WARN("data op: engine " << e->Name() << " failed (" << ret << ") for " << DirectionName(dir) << ", trying the next one");
    }
    if (cands.empty()) {
        MF_ERROR("data op: no engine can serve " << DirectionName(dir) << " between ranks " << opt.srcRank << " and " << opt.dstRank);
    }
    return ret;
}

int ComposeDataOp::BatchDataCopy(const BatchCopyParams &p, CopyDirection dir, const ExtOptions &opt)
{
    int ret = BM_NOT_SUPPORTED;
    MF_TRACE_SCOPE(MF_TP(TM_DATAOP, 32 + (int)dir), "BATCH_COPY", &ret);
    uint64_t bytes = 0;
    for (uint32_t i = 0; i < p.batchSize; i++) {
        bytes += p.dataSizes[i];
    }
    auto cands = Candidates(dir, opt, bytes, true);
    for (auto &e : cands) {
        ret = e->BatchDataCopy(p, dir, opt);
        if (ret == BM_OK) {
            NoteServed(e->Type(), p.batchSize);
            return ret;
        }
        MF_WARN("data op: engine " << e->Name() << " failed (" << ret << ") for batch " << DirectionName(dir) << ", trying the next one");
    }
    if (cands.empty()) {
        MF_ERROR("data op: no engine can serve batch " << DirectionName(dir));
    }
    return ret;
}

int ComposeDataOp::Wait()
{
    int ret = BM_OK;
    for (auto &e : engines_) {
        if (e->Type() == OP_KERNEL_LDST) {  // both GPU engines share the calling thread's stream
            ret = e->Wait();
            break;
        }
    }
    return ret;
}

}  // namespace hybm
}  // namespace mf
