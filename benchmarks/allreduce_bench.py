#!/usr/bin/env python
"""In-kernel all-reduce fused with residual add + RMSNorm (hidden 8192, eps 1e-6, bf16 N(0,1)) versus NCCL all-reduce
followed by separate add and norm kernels. Sizes 16 KiB – 1 GiB of x per rank (whole rows of 8192 bf16), device-timed, max over ranks.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/allreduce_bench.py [--max-log2 30]

Per size: fused µs for each algorithm that applies, baseline µs, speed-up, and the achieved fraction of the NVLink roofline
(bytes that must cross NVLink per direction = 2 (R-1)/R x size for P2P, ~1 x size for NVLS; 770 GB/s measured per direction).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

NVLINK_GBPS = 770.0


def main():
    import torch
    import torch.distributed as dist

    from benchmarks import workloads
    from memfabric_hybrid_b200.parallel.heap import SymmetricHeap
    from memfabric_hybrid_b200.parallel.pool import env_rank_world

    ap = argparse.ArgumentParser()
    ap.add_argument("--min-log2", type=int, default=14)
    ap.add_argument("--max-log2", type=int, default=28)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--nvls", type=int, default=1)
    ap.add_argument("--out", default="", help="also write the rows to this JSON file")
    args = ap.parse_args()
    rank, local, world = env_rank_world()
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    H = args.hidden
    max_bytes = 1 << args.max_log2
    max_T = max(1, max_bytes // (H * 2))
    # two alternating input buffers and the residual of the large instance, the same for the small (CUDA-graph) instance
    heap = SymmetricHeap(rank, world, local, 3 * max_T * H * 2 + (64 << 20), nvls=bool(args.nvls))
    sizes = [1 << lg for lg in range(args.min_log2, args.max_log2 + 1) if (1 << lg) >= H * 2]
    rows = workloads.allreduce_sizes(heap, sizes, hidden=H, iters=args.iters)
    if rank == 0:
        for row in rows:
            print(json.dumps(row), flush=True)
    if rank == 0 and args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            json.dump({"world": world, "hidden": H, "nvls": bool(heap.multicast_ptr), "rows": rows}, f, indent=1)
    dist.barrier()
    heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
