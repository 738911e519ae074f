// Control-plane micro-benchmark: N forked ranks on one host share a config store (rank 0 hosts the server) and a static
// group engine over it; the program times the group barrier and a set followed by a get of a 64-byte value, and prints one
// JSON line with the slowest rank's mean of each. baseline/ref_store_bench.cpp runs the same workload against the reference's
// TcpConfigStore and SmemNetGroupEngine, so the two lines compare like for like (same host, same rank count, same loop).
//
// usage: store_bench [ranks=4] [port=28755] [iters=200]
#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "group/mf_group.h"
#include "store/mf_store_client.h"

using namespace mf;

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
    net::Endpoint ep;
    if (!net::ParseUrl("tcp://127.0.0.1:" + std::to_string(port), &ep)) {
        return 1;
    }
    store::StorePtr base = store::StoreFactory::CreateStore(ep, rank == 0, (uint32_t)world, rank, 60);
    if (base == nullptr) {
        std::fprintf(stderr, "rank %d: cannot create the store\n", rank);
        sh->failed = 1;
        return 1;
    }
    store::StorePtr st = std::make_shared<store::PrefixStore>(base, "bench_");
    group::GroupOption opt;
    opt.rankSize = (uint32_t)world;
    opt.rank = (uint32_t)rank;
    opt.timeoutMs = 30000;
    auto grp = group::GroupEngine::Create(st, opt);
    if (grp == nullptr) {
        sh->failed = 1;
        return 1;
    }
    for (int i = 0; i < 5; i++) {
        if (grp->GroupBarrier() != 0) {
            sh->failed = 1;
            return 1;
        }
    }
    auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < iters; i++) {
        if (grp->GroupBarrier() != 0) {
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
        if (st->Set(key, value) != 0 || st->Get(key, &got, 1000) != 0) {
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
        if (grp->GroupAllGather(mine.data(), 64, &all[0], (uint32_t)all.size()) != 0 || all[(size_t)(world - 1) * 64] != (char)('a' + (world - 1) % 26)) {
            sh->failed = 1;
            return 1;
        }
    }
    t1 = std::chrono::steady_clock::now();
    sh->allGatherUs[rank] = std::chrono::duration<double, std::micro>(t1 - t0).count() / iters;
    grp->GroupBarrier();
    if (rank == 0) {
        usleep(200 * 1000);  // the server's host leaves last
    }
    return 0;
}

int main(int argc, char **argv)
{
    const int world = argc > 1 ? std::atoi(argv[1]) : 4;
    const int port = argc > 2 ? std::atoi(argv[2]) : 28755;
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
        int status = 0;
        waitpid(kids[r], &status, 0);
        rc |= WIFEXITED(status) ? WEXITSTATUS(status) : 1;
    }
    double b = 0, s = 0, ag = 0;
    for (int r = 0; r < world; r++) {
        b = sh->barrierUs[r] > b ? sh->barrierUs[r] : b;
        s = sh->setGetUs[r] > s ? sh->setGetUs[r] : s;
        ag = sh->allGatherUs[r] > ag ? sh->allGatherUs[r] : ag;
    }
    if (rc != 0 || sh->failed) {
        std::printf("{\"impl\": \"memfabric_hybrid_b200\", \"error\": \"store benchmark failed\"}\n");
        return 1;
    }
    std::printf("{\"impl\": \"memfabric_hybrid_b200\", \"ranks\": %d, \"iters\": %d, \"group_barrier_us\": %.1f, \"set_get_us\": %.1f, \"group_allgather_us\": %.1f}\n",
                world, iters, b, s, ag);
    return 0;
}
