// Control-plane latency of the UNMODIFIED reference library (its config store and group engine), for comparison with the same
// measurement on this repository's store (benchmarks/store_bench.cpp). The reference's data plane cannot run on a CUDA machine,
// its control plane can: it is plain C++ over TCP.
//
// N forked processes on loopback; rank 0 also hosts the store server. Each rank times `iters` group barriers and `iters`
// set + get round trips; the maximum over ranks of the mean is printed as one JSON line by rank 0.
// Built by baseline/build_ref.sh against the reference's own headers and its libmf_smem.so; nothing of it is part of the product.
#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "smem_net_common.h"
#include "smem_net_group_engine.h"
#include "smem_store_factory.h"

using namespace ock::smem;

struct Shared {
    double barrierUs[64];
    double setGetUs[64];
    double allGatherUs[64];
    int failed;
};

static int RunRank(int rank, int world, int port, int iters, Shared *sh)
{
    if (rank != 0) {
        usleep(500 * 1000);  // the server of rank 0 comes up first
    }
    UrlExtraction url;  // the public entry points parse the URL first; that registers the address family of the port
    if (url.ExtractIpPortFromUrl("tcp://127.0.0.1:" + std::to_string(port)) != 0) {
        fprintf(stderr, "rank %d: bad url\n", rank);
        return 1;
    }
    StorePtr base = StoreFactory::CreateStore(url.ip, url.port, rank == 0, (uint32_t)world, rank, 60);
    if (base == nullptr) {
        std::fprintf(stderr, "rank %d: cannot create the store\n", rank);
        sh->failed = 1;
        return 1;
    }
    StorePtr store = StoreFactory::PrefixStore(base, "bench_");
    SmemGroupOption opt{};
    opt.rankSize = (uint32_t)world;
    opt.rank = (uint32_t)rank;
    opt.timeoutMs = 30000;
    opt.dynamic = false;
    SmemGroupEnginePtr group = SmemNetGroupEngine::Create(store, opt);
    if (group == nullptr) {
        sh->failed = 1;
        return 1;
    }
    for (int i = 0; i < 5; i++) {
        if (group->GroupBarrier() != 0) {
            sh->failed = 1;
            return 1;
        }
    }
    auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < iters; i++) {
        if (group->GroupBarrier() != 0) {
            sh->failed = 1;
            return 1;
        }
    }
    auto t1 = std::chrono::steady_clock::now();
    sh->barrierUs[rank] = std::chrono::duration<double, std::micro>(t1 - t0).count() / iters;
    const std::string key = "k" + std::to_string(rank);
    std::string value(64, 'x'), got;
    t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < iters; i++) {
        if (store->Set(key, value) != 0 || store->Get(key, got, 1000) != 0) {
            sh->failed = 1;
            return 1;
        }
    }
    t1 = std::chrono::steady_clock::now();
    sh->setGetUs[rank] = std::chrono::duration<double, std::micro>(t1 - t0).count() / iters;
    // all-gather of one 64-byte record per rank (what the memory layers exchange when they publish slices and entities)
    std::string mine(64, (char)('a' + rank % 26)), all((size_t)world * 64, '\0');
    t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < iters; i++) {
        if (group->GroupAllGather(mine.data(), 64, &all[0], (uint32_t)all.size()) != 0 || all[(size_t)(world - 1) * 64] != (char)('a' + (world - 1) % 26)) {
            sh->failed = 1;
            return 1;
        }
    }
    t1 = std::chrono::steady_clock::now();
    sh->allGatherUs[rank] = std::chrono::duration<double, std::micro>(t1 - t0).count() / iters;
    group->GroupBarrier();
    if (rank != 0) {
        return 0;
    }
    usleep(200 * 1000);  // the server's host leaves last
    return 0;
}

int main(int argc, char **argv)
{
    const int world = argc > 1 ? std::atoi(argv[1]) : 4;
    const int port = argc > 2 ? std::atoi(argv[2]) : 28655;
    const int iters = argc > 3 ? std::atoi(argv[3]) : 200;
    if (world < 1 || world > 64) {
        return 2;
    }
    Shared *sh = (Shared *)mmap(nullptr, sizeof(Shared), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0);
    std::memset(sh, 0, sizeof(*sh));
    pid_t kids[64];
    for (int r = 0; r < world; r++) {
        kids[r] = fork();
        if (kids[r] == 0) {
            _exit(RunRank(r, world, port, iters, sh));
        }
    }
    int rc = 0;
    for (int r = 0; r < world; r++) {
        int st = 0;
        waitpid(kids[r], &st, 0);
        rc |= WIFEXITED(st) ? WEXITSTATUS(st) : 1;
    }
    double b = 0, s = 0, ag = 0;
    for (int r = 0; r < world; r++) {
        b = sh->barrierUs[r] > b ? sh->barrierUs[r] : b;
        s = sh->setGetUs[r] > s ? sh->setGetUs[r] : s;
        ag = sh->allGatherUs[r] > ag ? sh->allGatherUs[r] : ag;
    }
    if (rc != 0 || sh->failed) {
        std::printf("{\"impl\": \"reference\", \"error\": \"store benchmark failed\"}\n");
        return 1;
    }
    std::printf("{\"impl\": \"reference\", \"ranks\": %d, \"iters\": %d, \"group_barrier_us\": %.1f, \"set_get_us\": %.1f, \"group_allgather_us\": %.1f}\n",
                world, iters, b, s, ag);
    return 0;
}
