#!/usr/bin/env python
"""KV-cache block transfer: one request = 122 discrete blocks (61 × 128 KiB + 61 × 16 KiB = 8784 KiB, the DeepSeek-R1 KV
shape the reference quotes in README.md:110-112) at random 4 KiB-aligned offsets, moved with ONE batch-copy call per
batch of 1 / 8 / 32 requests. Directions: GD→GD (to the next rank's pooled HBM), GD→GH (offload to the pooled DRAM), GH→GD
(reload). Reported per direction and batch size: p50 / p99 of the blocking call's wall latency (what a serving engine
sees), the device time of the same work enqueued on a stream, and GB/s (1e9), all as the max over ranks.

    python benchmarks/kv_blocks.py [--pool-gib 64] [--dram-gib-total 256] [--iters 50] [--out kv_blocks.json]
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


def kv_latency_quick(pool, rank, world, stream, iters: int = 30, span: int = 1 << 30, base_off: int = 0, with_host: bool = False):
    """Short variant used by bench.py on a pool it already has. Blocks live in [base_off, base_off + span) of this rank's HBM
    window (sources) and in the next `span` bytes (destinations). GD→GD for batches of 1 / 8 / 32 requests; with a DRAM pool
    also GD→GH and GH→GD."""
    import memfabric_hybrid_b200 as mf
    from benchmarks.workloads import kv_measure

    me, peer = pool.hbm(rank), pool.hbm((rank + 1) % world)
    G2G = mf.bm.BmCopyType.G2G
    res = {}
    for nreq in (1, 8, 32):
        so, sizes = make_requests(nreq, span, 11 + nreq)
        do, _ = make_requests(nreq, span, 29 + nreq)
        sizes_l = [int(s) for s in sizes]
        srcs = [int(me + base_off + o) for o in so]
        dsts = [int(peer + base_off + span + o) for o in do]
        res[f"gd2gd_batch{nreq}"] = kv_measure(pool.handle, srcs, dsts, sizes_l, G2G, stream, iters, mf.native)
        if with_host and pool.dram_bytes >= nreq * len(BLOCKS_PER_REQUEST) * 128 * KiB:
            ho, _ = make_requests(nreq, pool.dram_bytes, 7 + nreq)
            gh = [int(pool.dram(rank) + o) for o in ho]
            back = [int(me + base_off + span + o) for o in do]
            res[f"gd2gh_batch{nreq}"] = kv_measure(pool.handle, srcs, gh, sizes_l, G2G, stream, max(5, iters // 3), mf.native)
            res[f"gh2gd_batch{nreq}"] = kv_measure(pool.handle, gh, back, sizes_l, G2G, stream, max(5, iters // 3), mf.native)
    return res


def main():
    import torch

    import memfabric_hybrid_b200 as mf
    from benchmarks.workloads import kv_measure
    from memfabric_hybrid_b200.parallel.pool import env_rank_world, open_pool

    ap = argparse.ArgumentParser()
    ap.add_argument("--pool-gib", type=float, default=64.0, help="pooled HBM per rank (the benchmark configuration: 64 GiB per GPU)")
    ap.add_argument("--dram-gib-total", type=float, default=256.0,
                    help="pooled host DRAM over all ranks (the benchmark configuration: 256 GiB); every rank contributes an equal share")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--out", default="", help="also write the result to this JSON file")
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
    dram = int(args.dram_gib_total * (1 << 30)) // world // (2 << 20) * (2 << 20)
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
        results[f"gd2gd_batch{nreq}"] = kv_measure(pool.handle, gd_src, gd_dst, sizes_l, G2G, stream, args.iters, mf.native)
        barrier()
        results[f"gd2gh_batch{nreq}"] = kv_measure(pool.handle, gd_src, gh, sizes_l, G2G, stream, args.iters, mf.native)
        results[f"gh2gd_batch{nreq}"] = kv_measure(pool.handle, gh, back, sizes_l, G2G, stream, args.iters, mf.native)
        barrier()
        # bit-exactness of offload + reload: the reloaded blocks equal the source blocks
        if world == 1:
            from memfabric_hybrid_b200.utils.tensors import device_tensor_from_gva

            ok = all(torch.equal(device_tensor_from_gva(s, z), device_tensor_from_gva(b, z)) for s, b, z in zip(gd_src[:16], back[:16], sizes_l[:16]))
            results[f"roundtrip_exact_batch{nreq}"] = bool(ok)
        if rank == 0:
            print(json.dumps({k: v for k, v in results.items() if k.endswith(f"batch{nreq}")}), flush=True)
    summary = {"world": world, "request_bytes": REQUEST_BYTES, "blocks_per_request": len(BLOCKS_PER_REQUEST),
               "hbm_pool_bytes_per_rank": hbm, "dram_pool_bytes_per_rank": dram, "dram_pool_bytes_total": dram * world, "results": results}
    if rank == 0:
        print(json.dumps({k: v for k, v in summary.items() if k != "results"}), flush=True)
    if rank == 0 and args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            json.dump(summary, f, indent=1)
    barrier()
    pool.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
