// Big Memory from C++: every rank contributes HBM (and DRAM), pushes a seeded buffer host → own HBM → next rank's HBM →
// next rank's DRAM, then everybody verifies what landed in its own windows. One process per GPU:
//     ./bm_example <rank> <world> tcp://127.0.0.1:7788
// (counterpart of the reference's example/bm/BmCpp/main.cpp:142-201)
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <unistd.h>
#include <vector>

#include "mf/mf.h"
#include "mf/mf_bm.h"

static unsigned char Pattern(int rank, size_t i) { return (unsigned char)((i * 131 + rank * 17) & 0xff); }

int main(int argc, char **argv)
{
    if (argc < 4) {
        fprintf(stderr, "usage: %s <rank> <world> <store-url>\n", argv[0]);
        return 2;
    }
    const int rank = atoi(argv[1]), world = atoi(argv[2]);
    const size_t pool = 64ull << 20, n = 8ull << 20;
    mf_bm_config_t cfg;
    mf_bm_config_init(&cfg);
    cfg.rankId = (uint16_t)rank;
    if (mf_bm_init(argv[3], (uint32_t)world, (uint16_t)rank /* GPU ordinal */, &cfg) != MF_OK) {
        fprintf(stderr, "init failed: %s\n", mf_get_last_err_msg());
        return 1;
    }
    mf_bm_t bm = mf_bm_create(0, (uint32_t)world, MF_BM_DATA_OP_SDMA, pool, pool, 0);
    if (bm == nullptr || mf_bm_join(bm, 0) != MF_OK) {
        fprintf(stderr, "create/join failed: %s\n", mf_get_last_err_msg());
        return 1;
    }
    while (mf_bm_get_joined_size(bm) != (uint32_t)world) {
        usleep(1000);
    }
    const int next = (rank + 1) % world, prev = (rank + world - 1) % world;
    char *myHbm = (char *)mf_bm_ptr_by_mem_type(bm, MF_MEM_TYPE_DEVICE, (uint16_t)rank);
    char *nextHbm = (char *)mf_bm_ptr_by_mem_type(bm, MF_MEM_TYPE_DEVICE, (uint16_t)next);
    char *nextDram = (char *)mf_bm_ptr_by_mem_type(bm, MF_MEM_TYPE_HOST, (uint16_t)next);
    std::vector<unsigned char> host(n), back(n);
    for (size_t i = 0; i < n; i++) {
        host[i] = Pattern(rank, i);
    }
    mf_copy_params h2g{host.data(), myHbm, n};                 // host → own pooled HBM
    mf_copy_params g2g{myHbm, nextHbm + n, n};                 // own HBM → next rank's HBM (NVLink)
    mf_copy_params g2gh{myHbm, nextDram, n};                   // own HBM → next rank's pooled DRAM
    int rc = mf_bm_copy(bm, &h2g, MF_BM_COPY_H2G, 0) | mf_bm_copy(bm, &g2g, MF_BM_COPY_G2G, 0) | mf_bm_copy(bm, &g2gh, MF_BM_COPY_G2G, 0);
    if (rc != MF_OK) {
        fprintf(stderr, "copy failed: %s\n", mf_get_last_err_msg());
        return 1;
    }
    sleep(1);  // a real program synchronises through its own channel; the pool itself needs none for one-sided writes
    mf_copy_params g2h{myHbm + n, back.data(), n};             // what the previous rank left in my HBM → host
    rc = mf_bm_copy(bm, &g2h, MF_BM_COPY_G2H, 0);
    size_t bad = 0;
    const unsigned char *dram = (const unsigned char *)mf_bm_ptr_by_mem_type(bm, MF_MEM_TYPE_HOST, (uint16_t)rank);
    for (size_t i = 0; i < n; i++) {
        bad += back[i] != Pattern(prev, i);
        bad += dram[i] != Pattern(prev, i);  // pooled DRAM is ordinary memory for the CPU
    }
    printf("rank %d: rc=%d mismatches=%zu\n", rank, rc, bad);
    sleep(1);
    mf_bm_destroy(bm);
    mf_bm_uninit(0);
    return rc != MF_OK || bad != 0;
}
