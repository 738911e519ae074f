#!/usr/bin/env python
"""KV-cache block transfer: one request = 122 discrete blocks (61 × 128 KiB + 61 × 16 KiB = 8784 KiB, the DeepSeek-R1 KV
shape the reference quotes in README.md:110-112) at random 4 KiB-aligned offsets, moved with ONE batch-copy call per
batch of 1 / 8 / 32 requests. Directions: GD→GD (to the next rank's pooled HBM), GD→GH (offload to the pooled DRAM), GH→GD
(reload). Reported per direction and batch size: p50 / p99 of the blocking call's wall latency (what a serving engine
sees), the device time of the same work enqueued on a stream, and GB/s (1e9), all as the max over ranks.

    python benchmarks/kv_blocks.py [--pool-gib 8] [--dram-gib 4] [--iters 50] [--out gpurun_out/kv_blocks.json]
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/kv_blocks.py

Baseline columns: the same blocks moved with one cudaMemcpyAsync per block (what a copy-engine implementation does).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

KiB = 1024
BLOCKS_PER_REQUEST = [128 * KiB] * 61 + [16 * KiB] * 61
REQUEST_BYTES = sum(BLOCKS_PER_REQUEST)


def make_requests(nreq: int, span: int, seed: int):
    """Non-overlapping 4 KiB-aligned offsets inside [0, span): one 128 KiB slot per block, slots shuffled."""
    rng = np.random.default_rng(seed)
    nblocks = nreq * len(BLOCKS_PER_REQUEST)
    slots = span // (128 * KiB)
    if slots < nblocks:
        raise ValueError("pool too small for the requested batch")
    pick = rng.choice(slots, size=nblocks, replace=False)
    sizes = np.array(BLOCKS_PER_REQUEST * nreq, dtype=np.int64)
    room = (128 * KiB - sizes) // (4 * KiB)  # small blocks float inside their slot in 4 KiB steps
    jitter = (rng.random(nblocks) * (room + 1)).astype(np.int64)
    offs = (pick * 128 * KiB + jitter * 4 * KiB).astype(np.int64)
    return offs, sizes


def percentile(xs, p):
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(round(p / 100.0 * (len(xs) - 1))))]


def measure(handle, srcs, dsts, sizes, copy_type, stream, iters, maxr, native=None):
    import torch

    n = len(sizes)
    total = int(sum(sizes))
    # blocking latency through the public API
    for _ in range(3):
        assert handle.copy_data_batch(srcs, dsts, sizes, n, copy_type, 0) == 0
    lat = []
    for _ in range(iters):
        t0 = time.perf_counter()
        rc = handle.copy_data_batch(srcs, dsts, sizes, n, copy_type, 0)
        lat.append((time.perf_counter() - t0) * 1e6)
        assert rc == 0
    # device time of the enqueued work
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record(stream)
    for _ in range(iters):
        handle.copy_data_batch_on_stream(srcs, dsts, sizes, copy_type, stream.cuda_stream, 0)
    b.record(stream)
    torch.cuda.synchronize()
    dev_us = a.elapsed_time(b) * 1e3 / iters
    out = {
        "p50_us": round(maxr(percentile(lat, 50)), 1),
        "p99_us": round(maxr(percentile(lat, 99)), 1),
        "device_us": round(maxr(dev_us), 1),
    }
    out["GBps_p50"] = round(total / (out["p50_us"] * 1e-6) / 1e9, 1)
    out["GBps_device"] = round(total / (out["device_us"] * 1e-6) / 1e9, 1)
    if native is not None:
        # per-block cudaMemcpyAsync on the same stream, then one synchronize: the copy-engine way
        for _ in range(2):
            for s, d, z in zip(srcs, dsts, sizes):
                native.copy_engine(d, s, z, stream.cuda_stream)
            stream.synchronize()
        lat2 = []
        for _ in range(max(5, iters // 4)):
            t0 = time.perf_counter()
            for s, d, z in zip(srcs, dsts, sizes):
                native.copy_engine(d, s, z, stream.cuda_stream)
            stream.synchronize()
            lat2.append((time.perf_counter() - t0) * 1e6)
        out["per_block_memcpy_p50_us"] = round(maxr(percentile(lat2, 50)), 1)
    return out


def kv_latency_quick(pool, rank, world, stream, iters: int = 30):
    """Small variant used by bench.py on the pool it already has: GD→GD, batch of 1 and 8 requests."""
    import torch

    import memfabric_hybrid_b200 as mf

    def maxr(v):
        if world == 1:
            return v
        import torch.distributed as dist

        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    span = 1 << 30
    me, peer = pool.hbm(rank), pool.hbm((rank + 1) % world)
    res = {}
    for nreq in (1, 8):
        so, sizes = make_requests(nreq, span, 11 + nreq)
        do, _ = make_requests(nreq, span, 29 + nreq)
        srcs = [int(me + o) for o in so]
        dsts = [int(peer + span + o) for o in do]
        res[f"gd2gd_batch{nreq}"] = measure(pool.handle, srcs, dsts, [int(s) for s in sizes], mf.bm.BmCopyType.G2G, stream, iters, maxr)
    return res


def main():
    import torch

    import memfabric_hybrid_b200 as mf
    from memfabric_hybrid_b200.parallel.pool import env_rank_world, open_pool

    ap = argparse.ArgumentParser()
    ap.add_argument("--pool-gib", type=float, default=8.0, help="pooled HBM per rank (the full-size configuration is 64)")
    ap.add_argument("--dram-gib", type=float, default=4.0, help="pooled DRAM per rank (the full-size configuration is 256 in total)")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--out", default="gpurun_out/kv_blocks.json")
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

    hbm = int(args.pool_gib * (1 << 30))
    dram = int(args.dram_gib * (1 << 30))
    pool = open_pool(rank, world, local, hbm, dram_bytes=dram)
    barrier()
    stream = torch.cuda.current_stream()
    me, peer = pool.hbm(rank), pool.hbm((rank + 1) % world)
    half = hbm // 2
    mf.native.fill_pattern(me, half, 1000 + rank, stream.cuda_stream)  # bf16-agnostic seeded bytes in the source half
    torch.cuda.synchronize()
    barrier()
    G2G = mf.bm.BmCopyType.G2G
    results = {}
    for nreq in (1, 8, 32):
        so, sizes = make_requests(nreq, half, 3 + nreq)
        do, _ = make_requests(nreq, half, 5 + nreq)
        ho, _ = make_requests(nreq, dram, 7 + nreq)
        sizes_l = [int(s) for s in sizes]
        gd_src = [int(me + o) for o in so]
        gd_dst = [int(peer + half + o) for o in do]
        gh = [int(pool.dram(rank) + o) for o in ho]
        back = [int(me + half + o) for o in do]
        results[f"gd2gd_batch{nreq}"] = measure(pool.handle, gd_src, gd_dst, sizes_l, G2G, stream, args.iters, maxr, mf.native)
        barrier()
        results[f"gd2gh_batch{nreq}"] = measure(pool.handle, gd_src, gh, sizes_l, G2G, stream, args.iters, maxr, mf.native)
        results[f"gh2gd_batch{nreq}"] = measure(pool.handle, gh, back, sizes_l, G2G, stream, args.iters, maxr, mf.native)
        barrier()
        # bit-exactness of offload + reload: the reloaded blocks equal the source blocks
        if world == 1:
            from memfabric_hybrid_b200.utils.tensors import device_tensor_from_gva

            ok = all(torch.equal(device_tensor_from_gva(s, z), device_tensor_from_gva(b, z)) for s, b, z in zip(gd_src[:16], back[:16], sizes_l[:16]))
            results[f"roundtrip_exact_batch{nreq}"] = bool(ok)
        if rank == 0:
            print(json.dumps({k: v for k, v in results.items() if k.endswith(f"batch{nreq}")}), flush=True)
    if rank == 0:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            json.dump({"world": world, "request_bytes": REQUEST_BYTES, "blocks_per_request": len(BLOCKS_PER_REQUEST), "results": results}, f, indent=1)
    barrier()
    pool.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
