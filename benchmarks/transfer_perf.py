#!/usr/bin/env python
"""Point-to-point latency/throughput table in the shape of the reference's transfer_perf
(example/trans/perf/transfer_perf.cpp:126-171, results example/trans/perf/README.md:61-70): rank 0 → rank 1, block sizes
32 KiB … 16 MiB; latency = mean wall-clock of 10 blocking single copies, throughput = 10 batches of 32 blocks.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/transfer_perf.py [--out FILE.json]

The reference's published Atlas A3 numbers (SDMA dev0 → dev1) are printed alongside.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

REF_LAT_US = [12.5, 12.1, 10.2, 11.3, 13.6, 15.9, 23.7, 35.5, 57.8, 102.5]
REF_GBPS = [9.70, 19.33, 39.98, 76.26, 151.83, 179.72, 179.87, 184.24, 183.11, 186.61]


def main():
    import torch
    import torch.distributed as dist

    import memfabric_hybrid_b200 as mf
    from memfabric_hybrid_b200.parallel.pool import env_rank_world, open_pool

    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank, local, world = env_rank_world()
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peer = 1 % world
    top = 16 << 20
    pool = open_pool(rank, world, local, 2 * 32 * top + (4 << 20))
    if world > 1:
        dist.barrier()
    T = mf.bm.BmCopyType.G2G
    me, dst = pool.hbm(rank), pool.hbm(peer) + 32 * top
    mf.native.fill_pattern(me, 32 * top, 9, 0)
    torch.cuda.synchronize()
    rows = []
    if rank == 0:
        for i, lg in enumerate(range(15, 25)):
            n = 1 << lg
            for _ in range(3):
                pool.handle.copy_data(me, dst, n, T, 0)
            t0 = time.perf_counter()
            for _ in range(10):
                assert pool.handle.copy_data(me, dst, n, T, 0) == 0
            lat = (time.perf_counter() - t0) / 10 * 1e6
            srcs = [me + k * n for k in range(32)]
            dsts = [dst + k * n for k in range(32)]
            sizes = [n] * 32
            pool.handle.copy_data_batch(srcs, dsts, sizes, 32, T, 0)
            t0 = time.perf_counter()
            for _ in range(10):
                assert pool.handle.copy_data_batch(srcs, dsts, sizes, 32, T, 0) == 0
            dt = time.perf_counter() - t0
            gbps = 10 * 32 * n / dt / 1e9
            rows.append({"block": n, "latency_us": round(lat, 1), "batch32_GBps": round(gbps, 1), "reference_a3_latency_us": REF_LAT_US[i],
                         "reference_a3_GBps": REF_GBPS[i]})
            print(json.dumps(rows[-1]), flush=True)
        if args.out:
            os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
            with open(args.out, "w") as f:
                json.dump({"world": world, "rows": rows}, f, indent=1)
    if world > 1:
        dist.barrier()
    pool.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
