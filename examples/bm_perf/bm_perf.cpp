// bm_perf: bandwidth of the Big Memory copy directions, one forked process per rank (one GPU each), through the public C API.
//
//   ./bm_perf -bw -t all -s 2097152 -bs 32 -cc 20 -ws 2 -lrs 2 -ip tcp://127.0.0.1:8570 [-d 0] [-ot sdma] [-pin]
//
// Counterpart of the reference's bm_perf_benchmark (example/bm/BmBenchmark/band_width_calculator.cpp:368-407 for the process
// model, :423-600 for the ten directions, README.md:60-96 for the command line): every rank issues `-cc` synchronous
// mf_bm_copy_batch calls of `-bs` blocks of `-s` bytes between rank barriers, wall-clock timed, GB/s = bytes / microseconds
// / 1000 (1 GB = 1e9 B), followed by a byte check of what arrived and a table per rank.
// Directions, seen from the issuing rank (its "remote" is the next rank):
//   h2d  local host -> own pooled HBM      d2h  own pooled HBM -> local host
//   h2rd local host -> remote pooled HBM   h2rh local host -> remote pooled DRAM
//   d2rd local device -> remote pooled HBM d2rh local device -> remote pooled DRAM
//   rh2d remote pooled DRAM -> local device   rh2h remote pooled DRAM -> local host
//   rd2d remote pooled HBM -> local device    rd2h remote pooled HBM -> local host
// All ranks of a run live on this host (-ws == -lrs); the rank barrier lives in memory shared by the forked ranks.
#include <cuda_runtime.h>
#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "mf/mf.h"
#include "mf/mf_bm.h"

namespace {

struct Options {
    std::string type{"all"}, opType{"sdma"}, url{"tcp://127.0.0.1:8570"};
    uint64_t blockSize{2ull << 20};
    uint32_t batch{32}, copyCount{10}, world{2}, localRanks{2}, rankStart{0}, deviceStart{0};
    bool pinned{false};
};

// Rank barrier in memory shared by the forked ranks. A rank that fails raises `failed`, which releases everybody else: no
// rank is left waiting for one that has gone.
struct Shared {
    std::atomic<uint32_t> arrived;
    std::atomic<uint32_t> generation;
    std::atomic<int> failed;
    uint32_t ranks;
};

bool BarrierWait(Shared *sh)
{
    const uint32_t gen = sh->generation.load();
    if (sh->arrived.fetch_add(1) + 1 == sh->ranks) {
        sh->arrived.store(0);
        sh->generation.fetch_add(1);
        return sh->failed.load() == 0;
    }
    for (uint64_t spins = 0; sh->generation.load() == gen; spins++) {
        if (sh->failed.load() != 0 || spins > 120ull * 20000) {  // about two minutes
            sh->failed.store(1);
            return false;
        }
        usleep(50);
    }
    return sh->failed.load() == 0;
}

struct Row {
    const char *name;
    double us;
    double gbps;
    bool checked;
    bool ok;
};

const char *kAll[] = {"h2d", "d2h", "h2rd", "h2rh", "d2rd", "d2rh", "rh2d", "rh2h", "rd2d", "rd2h"};

unsigned char PatternByte(uint32_t rank, int dir, uint64_t i) { return (unsigned char)((i * 2654435761u + rank * 97u + (uint32_t)dir * 13u) >> 7); }

void Fill(std::vector<unsigned char> &v, uint32_t rank, int dir)
{
    for (uint64_t i = 0; i < v.size(); i++) {
        v[i] = PatternByte(rank, dir, i);
    }
}

uint64_t Mismatches(const unsigned char *p, uint64_t n, uint32_t rank, int dir)
{
    uint64_t bad = 0;
    for (uint64_t i = 0; i < n; i++) {
        bad += p[i] != PatternByte(rank, dir, i);
    }
    return bad;
}

void Usage(const char *argv0)
{
    std::printf("usage: %s -bw [-ot sdma|device_rdma|host_rdma|host_tcp] [-t h2d|d2h|h2rd|h2rh|d2rd|d2rh|rh2d|rh2h|rd2d|rd2h|all]\n"
                "          [-s BLOCK_SIZE] [-bs BATCH_SIZE] [-cc COPY_COUNT] [-ws WORLD_SIZE] [-lrs LOCAL_RANK_SIZE] [-rs RANK_START]\n"
                "          [-d DEVICE_START] [-ip tcp://IP:PORT] [-pin]\n",
                argv0);
}

int RunRank(const Options &o, uint32_t rank, Shared *sh)
{
    const uint32_t next = (rank + 1) % o.world, prev = (rank + o.world - 1) % o.world;
    const uint64_t total = o.blockSize * o.batch;
    const uint64_t window = (total + (2ull << 20) - 1) / (2ull << 20) * (2ull << 20) * 2;  // two regions per pool window
    auto barrier = [&]() {
        if (!BarrierWait(sh)) {
            std::fprintf(stderr, "rank %u: another rank failed or did not arrive; leaving\n", rank);
            _exit(1);
        }
    };
    auto fail = [&](const char *what) {
        std::fprintf(stderr, "rank %u: %s: %s\n", rank, what, mf_get_last_err_msg());
        sh->failed.store(1);
        return 1;
    };
    mf_bm_config_t cfg;
    mf_bm_config_init(&cfg);
    cfg.autoRanking = false;
    cfg.rankId = (uint16_t)rank;
    if (mf_bm_init(o.url.c_str(), o.world, (uint16_t)(o.deviceStart + rank - o.rankStart), &cfg) != MF_OK) {
        return fail("mf_bm_init");
    }
    mf_bm_data_op_type op = o.opType == "host_rdma" ? MF_BM_DATA_OP_HOST_RDMA
                            : o.opType == "host_tcp" ? MF_BM_DATA_OP_HOST_TCP
                            : o.opType == "device_rdma" ? MF_BM_DATA_OP_DEVICE_RDMA
                                                        : MF_BM_DATA_OP_SDMA;
    mf_bm_t bm = mf_bm_create(0, o.world, op, window, window, MF_BM_FLAG_NUMA_MASK);
    if (bm == nullptr || mf_bm_join(bm, 0) != MF_OK) {
        return fail("mf_bm_create / mf_bm_join");
    }
    while (mf_bm_get_joined_size(bm) != o.world) {
        usleep(1000);
    }
    barrier();
    unsigned char *myHbm = (unsigned char *)mf_bm_ptr_by_mem_type(bm, MF_MEM_TYPE_DEVICE, (uint16_t)rank);
    unsigned char *myDram = (unsigned char *)mf_bm_ptr_by_mem_type(bm, MF_MEM_TYPE_HOST, (uint16_t)rank);
    unsigned char *nextHbm = (unsigned char *)mf_bm_ptr_by_mem_type(bm, MF_MEM_TYPE_DEVICE, (uint16_t)next);
    unsigned char *nextDram = (unsigned char *)mf_bm_ptr_by_mem_type(bm, MF_MEM_TYPE_HOST, (uint16_t)next);
    // local buffers: host (pageable, or pinned with -pin) and device
    unsigned char *lh = nullptr, *ld = nullptr;
    if (o.pinned) {
        cudaHostAlloc((void **)&lh, total, cudaHostAllocDefault);
    } else {
        lh = (unsigned char *)std::malloc(total);
    }
    if (lh == nullptr || cudaMalloc((void **)&ld, total) != cudaSuccess) {
        return fail("local buffers");
    }
    std::vector<unsigned char> pattern(total), back(total);
    std::vector<Row> rows;
    std::vector<void *> srcs(o.batch), dsts(o.batch);
    std::vector<uint64_t> sizes(o.batch, o.blockSize);

    auto timed = [&](unsigned char *src, unsigned char *dst, mf_bm_copy_type type) -> double {
        for (uint32_t b = 0; b < o.batch; b++) {
            srcs[b] = src + (uint64_t)b * o.blockSize;
            dsts[b] = dst + (uint64_t)b * o.blockSize;
        }
        mf_batch_copy_params p{srcs.data(), dsts.data(), sizes.data(), o.batch};
        if (mf_bm_copy_batch(bm, &p, type, 0) != MF_OK) {  // warm-up, and the copy whose result is checked
            fail("mf_bm_copy_batch");
            return -1.0;
        }
        barrier();
        auto t0 = std::chrono::steady_clock::now();
        for (uint32_t c = 0; c < o.copyCount; c++) {
            if (mf_bm_copy_batch(bm, &p, type, 0) != MF_OK) {
                fail("mf_bm_copy_batch");
                return -1.0;
            }
        }
        auto t1 = std::chrono::steady_clock::now();
        barrier();
        return std::chrono::duration<double, std::micro>(t1 - t0).count();
    };
    auto record = [&](const char *name, double us, bool checked, uint64_t bad) {
        Row r{name, us, us > 0 ? (double)total * o.copyCount / us / 1000.0 : 0.0, checked, bad == 0};
        rows.push_back(r);
        if (bad != 0) {
            sh->failed.store(1);
        }
    };
    auto stage = [&](unsigned char *poolAddr, mf_bm_copy_type type) {  // seeded bytes into a pool region of this rank
        mf_copy_params c{pattern.data(), poolAddr, total};
        return mf_bm_copy(bm, &c, type, 0) == MF_OK;
    };
    auto fetch = [&](unsigned char *poolAddr, mf_bm_copy_type type) {  // a pool region of this rank back into `back`
        mf_copy_params c{poolAddr, back.data(), total};
        return mf_bm_copy(bm, &c, type, 0) == MF_OK;
    };

    for (int d = 0; d < 10; d++) {
        const std::string name = kAll[d];
        if (o.type != "all" && o.type != name) {
            continue;
        }
        Fill(pattern, rank, d);
        std::memcpy(lh, pattern.data(), total);
        cudaMemcpy(ld, pattern.data(), total, cudaMemcpyHostToDevice);
        uint64_t bad = 0;
        double us = -1;
        if (name == "h2d") {
            us = timed(lh, myHbm, MF_BM_COPY_H2G);
            bad = fetch(myHbm, MF_BM_COPY_G2H) ? Mismatches(back.data(), total, rank, d) : 1;
        } else if (name == "d2h") {
            stage(myHbm, MF_BM_COPY_H2G);
            std::memset(lh, 0, total);
            us = timed(myHbm, lh, MF_BM_COPY_G2H);
            bad = Mismatches(lh, total, rank, d);
        } else if (name == "h2rd" || name == "d2rd" || name == "h2rh" || name == "d2rh") {
            const bool toHbm = name[name.size() - 1] == 'd';
            unsigned char *src = name[0] == 'h' ? lh : ld;
            unsigned char *dst = (toHbm ? nextHbm : nextDram) + window / 2;
            us = timed(src, dst, name[0] == 'h' ? (toHbm ? MF_BM_COPY_H2G : MF_BM_COPY_H2GH) : (toHbm ? MF_BM_COPY_L2G : MF_BM_COPY_L2GH));
            // what the previous rank wrote into MY window is checked by me
            bad = fetch((toHbm ? myHbm : myDram) + window / 2, toHbm ? MF_BM_COPY_G2H : MF_BM_COPY_GH2H) ? Mismatches(back.data(), total, prev, d) : 1;
        } else {  // rh2d, rh2h, rd2d, rd2h: the remote side first publishes its bytes in its own window
            const bool fromHbm = name[1] == 'd';
            const bool toDev = name[name.size() - 1] == 'd';
            stage(fromHbm ? myHbm : myDram, fromHbm ? MF_BM_COPY_H2G : MF_BM_COPY_H2GH);
            barrier();
            unsigned char *src = fromHbm ? nextHbm : nextDram;
            if (toDev) {
                cudaMemset(ld, 0, total);
                us = timed(src, ld, fromHbm ? MF_BM_COPY_G2L : MF_BM_COPY_GH2L);
                cudaMemcpy(back.data(), ld, total, cudaMemcpyDeviceToHost);
                bad = Mismatches(back.data(), total, next, d);
            } else {
                std::memset(lh, 0, total);
                us = timed(src, lh, fromHbm ? MF_BM_COPY_G2H : MF_BM_COPY_GH2H);
                bad = Mismatches(lh, total, next, d);
            }
        }
        record(kAll[d], us, true, us < 0 ? 1 : bad);
        barrier();
    }
    // per-rank table, one rank after the other
    for (uint32_t r = o.rankStart; r < o.rankStart + o.localRanks; r++) {
        if (r == rank) {
            std::printf("rank %u (GPU %u)  block %llu B x batch %u x count %u\n", rank, o.deviceStart + rank - o.rankStart, (unsigned long long)o.blockSize,
                        o.batch, o.copyCount);
            std::printf("  %-6s %14s %12s %8s\n", "type", "time(us)", "GB/s", "check");
            for (const Row &row : rows) {
                std::printf("  %-6s %14.1f %12.2f %8s\n", row.name, row.us, row.gbps, row.ok ? "ok" : "FAILED");
            }
            std::fflush(stdout);
        }
        barrier();
    }
    cudaFree(ld);
    if (o.pinned) {
        cudaFreeHost(lh);
    } else {
        std::free(lh);
    }
    barrier();
    mf_bm_destroy(bm);
    mf_bm_uninit(0);
    return sh->failed.load();
}

}  // namespace

int main(int argc, char **argv)
{
    Options o;
    bool bw = false;
    for (int i = 1; i < argc; i++) {
        std::string a = argv[i];
        auto val = [&]() -> const char * { return i + 1 < argc ? argv[++i] : ""; };
        if (a == "-h" || a == "--help") {
            Usage(argv[0]);
            return 0;
        } else if (a == "-bw") {
            bw = true;
        } else if (a == "-pin") {
            o.pinned = true;
        } else if (a == "-ot") {
            o.opType = val();
        } else if (a == "-t") {
            o.type = val();
        } else if (a == "-s") {
            o.blockSize = std::strtoull(val(), nullptr, 10);
        } else if (a == "-bs") {
            o.batch = (uint32_t)std::strtoul(val(), nullptr, 10);
        } else if (a == "-cc") {
            o.copyCount = (uint32_t)std::strtoul(val(), nullptr, 10);
        } else if (a == "-ws") {
            o.world = (uint32_t)std::strtoul(val(), nullptr, 10);
        } else if (a == "-lrs") {
            o.localRanks = (uint32_t)std::strtoul(val(), nullptr, 10);
        } else if (a == "-rs") {
            o.rankStart = (uint32_t)std::strtoul(val(), nullptr, 10);
        } else if (a == "-d") {
            o.deviceStart = (uint32_t)std::strtoul(val(), nullptr, 10);
        } else if (a == "-ip") {
            o.url = val();
        } else if (a == "-rdma") {
            (void)val();  // accepted for command-line compatibility: there is no separate RDMA NIC inside one NVSwitch domain
        } else {
            std::fprintf(stderr, "unknown option %s\n", a.c_str());
            Usage(argv[0]);
            return 2;
        }
    }
    bool known = o.type == "all";
    for (const char *n : kAll) {
        known = known || o.type == n;
    }
    if (!bw || !known || o.blockSize == 0 || o.batch == 0 || o.copyCount == 0 || o.world == 0 || o.localRanks == 0) {
        Usage(argv[0]);
        return 2;
    }
    if (o.world != o.localRanks || o.rankStart != 0) {
        std::fprintf(stderr, "bm_perf: all ranks of a run must be on this host (-ws == -lrs, -rs 0)\n");
        return 2;
    }
    Shared *sh = (Shared *)mmap(nullptr, sizeof(Shared), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0);
    if (sh == MAP_FAILED) {
        return 1;
    }
    new (sh) Shared();
    sh->arrived.store(0);
    sh->generation.store(0);
    sh->failed.store(0);
    sh->ranks = o.localRanks;
    std::vector<pid_t> kids;
    for (uint32_t r = 0; r < o.localRanks; r++) {  // fork BEFORE anything touches CUDA
        pid_t pid = fork();
        if (pid == 0) {
            _exit(RunRank(o, o.rankStart + r, sh));
        }
        kids.push_back(pid);
    }
    int rc = 0;
    for (pid_t pid : kids) {
        int st = 0;
        waitpid(pid, &st, 0);
        rc |= (WIFEXITED(st) ? WEXITSTATUS(st) : 1);
    }
    std::printf("bm_perf: %s\n", rc == 0 && sh->failed.load() == 0 ? "all directions verified" : "FAILED");
    return rc != 0 || sh->failed.load() != 0;
}
