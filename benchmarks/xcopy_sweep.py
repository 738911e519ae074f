#!/usr/bin/env python
"""Bandwidth sweep of xcopy over the GVA: D2D (local or rank r → r+1), H2D, D2H, GH→GD, sizes 4 KiB – 2 GiB in powers of two,
against cudaMemcpyAsync on the same buffers. Device-timed (CUDA events), max over ranks, seeded data, GB = 1e9 B.

    python benchmarks/xcopy_sweep.py [--max-log2 31] [--out FILE.json]
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/xcopy_sweep.py

Mirrors the reference's bm_perf_benchmark directions (example/bm/BmBenchmark/band_width_calculator.cpp:423-600).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch

    import memfabric_hybrid_b200 as mf
    from memfabric_hybrid_b200.parallel.pool import env_rank_world, open_pool

    ap = argparse.ArgumentParser()
    ap.add_argument("--min-log2", type=int, default=12)
    ap.add_argument("--max-log2", type=int, default=30)
    ap.add_argument("--out", default="")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--ctas", default="", help="comma list of CTA counts to try with the raw kernel at the largest size")
    args = ap.parse_args()

    rank, local, world = env_rank_world()
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()

    def maxr(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    top = 1 << args.max_log2
    host_cap = min(top, 1 << 30)
    pool = open_pool(rank, world, local, 2 * top + (4 << 20), dram_bytes=host_cap + (2 << 20))
    barrier()
    T = mf.bm.BmCopyType
    h = pool.handle
    stream = torch.cuda.current_stream()
    sh = stream.cuda_stream
    me, peer = pool.hbm(rank), pool.hbm((rank + 1) % world)
    mf.native.fill_pattern(me, top, 7 + rank, sh)
    pinned = torch.empty(host_cap, dtype=torch.uint8).pin_memory()
    pinned.random_(0, 256, generator=torch.Generator().manual_seed(rank))
    plain_src = torch.empty(top, dtype=torch.uint8, device="cuda")
    plain_dst = torch.empty(top, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    barrier()

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(iters):
            fn()
        b.record(stream)
        torch.cuda.synchronize()
        return maxr(a.elapsed_time(b)) / iters

    rows = []
    for lg in range(args.min_log2, args.max_log2 + 1):
        n = 1 << lg
        iters = args.iters if n <= (64 << 20) else max(5, args.iters // 4)
        row = {"bytes": n}
        cases = {
            "d2d": lambda: h.copy_data_on_stream(me, peer + top, n, T.G2G, sh, 0),
            "d2d_pull": lambda: h.copy_data_on_stream(peer, me + top, n, T.G2G, sh, 0),
            "d2d_ldst_kernel": lambda: mf.native.xcopy(peer + top, me, n, -1, sh),
            "d2d_copy_engine": lambda: mf.native.copy_engine(peer + top, me, n, sh),
            "cudaMemcpy_local": lambda: plain_dst[:n].copy_(plain_src[:n], non_blocking=True),
        }
        if n <= host_cap:
            cases.update({
                "h2d": lambda: h.copy_data_on_stream(pinned.data_ptr(), me + top, n, T.H2G, sh, 0),
                "d2h": lambda: h.copy_data_on_stream(me, pinned.data_ptr(), n, T.G2H, sh, 0),
                "gh2gd": lambda: h.copy_data_on_stream(pool.dram(rank), me + top, n, T.G2G, sh, 0),
                "gd2gh": lambda: h.copy_data_on_stream(me, pool.dram(rank), n, T.G2G, sh, 0),
                "h2d_kernel": lambda: h.copy_data_on_stream(pinned.data_ptr(), me + top, n, T.H2G, sh, 2),
                "d2h_kernel": lambda: h.copy_data_on_stream(me, pinned.data_ptr(), n, T.G2H, sh, 2),
            })
        for name, fn in cases.items():
            if fn is None:
                continue
            ms = timed(fn, iters)
            row[name + "_us"] = round(ms * 1e3, 2)
            row[name + "_GBps"] = round(n / (ms * 1e-3) / 1e9, 2)
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)

    cta_rows = []
    if args.ctas:
        n = min(top, 1 << 30)
        for c in [int(x) for x in args.ctas.split(",")]:
            ms = timed(lambda: mf.native.xcopy(peer + top, me, n, c, sh), 5)
            cta_rows.append({"ctas": c, "bytes": n, "GBps": round(n / (ms * 1e-3) / 1e9, 2)})
            if rank == 0:
                print(json.dumps(cta_rows[-1]), flush=True)

    # correctness of the last D2D
    out = torch.zeros(1, dtype=torch.int64, device="cuda")
    barrier()
    h.copy_data_on_stream(me, peer + top, top, T.G2G, sh, 0)
    torch.cuda.synchronize()
    barrier()
    mf.native.check_pattern(me + top, top, 7 + (rank - 1) % world, out.data_ptr(), sh)
    torch.cuda.synchronize()
    ok = int(out[0]) == 0
    if rank == 0:
        if args.out:
            os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
            with open(args.out, "w") as f:
                json.dump({"world": world, "rows": rows, "cta_rows": cta_rows, "bit_exact": ok}, f, indent=1)
        print("bit_exact", ok)
    barrier()
    pool.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
