#!/usr/bin/env python
"""In-kernel all-reduce fused with residual add + RMSNorm (hidden 8192, eps 1e-6, bf16 N(0,1)) versus NCCL all-reduce
followed by separate add and norm kernels. Sizes 1 KiB – 1 GiB of x per rank, device-timed, max over ranks.

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

    from memfabric_hybrid_b200.ops.allreduce import AllReduceRMSNorm, reference
    from memfabric_hybrid_b200.parallel.heap import SymmetricHeap
    from memfabric_hybrid_b200.parallel.pool import env_rank_world

    ap = argparse.ArgumentParser()
    ap.add_argument("--min-log2", type=int, default=10)
    ap.add_argument("--max-log2", type=int, default=28)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--nvls", type=int, default=1)
    ap.add_argument("--out", default="gpurun_out/allreduce_bench.json")
    args = ap.parse_args()
    rank, local, world = env_rank_world()
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    H = args.hidden
    max_bytes = 1 << args.max_log2
    max_T = max(1, max_bytes // (H * 2))
    heap = SymmetricHeap(rank, world, local, 2 * max_T * H * 2 + (8 << 20), nvls=bool(args.nvls))
    ar = AllReduceRMSNorm(heap, max_T, H, eps=1e-6)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    gc = torch.Generator(device="cuda").manual_seed(7)  # residual and weight are replicated across tensor-parallel ranks
    w = (1.0 + 0.1 * torch.randn(H, generator=gc, device="cuda")).to(torch.bfloat16)
    stream = torch.cuda.current_stream()

    def maxr(v):
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(iters):
            fn()
        b.record(stream)
        torch.cuda.synchronize()
        return maxr(a.elapsed_time(b)) * 1e3 / iters  # µs

    rows = []
    for lg in range(args.min_log2, args.max_log2 + 1):
        nbytes = 1 << lg
        if nbytes < H * 2:
            Hc, T = nbytes // 2, 1  # sub-row sizes: one short row
            if Hc % 8:
                continue
            arc = AllReduceRMSNorm(heap, 1, Hc, eps=1e-6) if Hc != H else ar
            wc = w[:Hc].contiguous()
        else:
            Hc, T, arc, wc = H, nbytes // (H * 2), ar, w
        x = torch.randn(T, Hc, generator=g, device="cuda").to(torch.bfloat16)
        res = torch.randn(T, Hc, generator=gc, device="cuda").to(torch.bfloat16)
        arc.x[:T].copy_(x)
        torch.cuda.synchronize()
        dist.barrier()
        row = {"bytes": nbytes, "T": T, "H": Hc}
        algos = ["oneshot"] if nbytes <= (4 << 20) else []
        algos += ["twoshot"]
        if heap.multicast_ptr:
            algos.append("nvls")
        iters = args.iters if nbytes <= (64 << 20) else 5
        for algo in algos:
            row[algo + "_us"] = round(timed(lambda: arc(T, res, wc, algo=algo), iters), 2)
        torch.cuda.synchronize()
        status = arc.check_status()
        # baseline: NCCL all-reduce, then add + norm as separate torch kernels
        xb = x.clone()

        def baseline():
            y = xb.clone()
            dist.all_reduce(y)
            h = y + res
            hf = h.float()
            return (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16) * wc, h

        row["nccl_unfused_us"] = round(timed(baseline, iters), 2)
        xb2 = x.clone()
        row["nccl_allreduce_only_us"] = round(timed(lambda: dist.all_reduce(xb2), iters), 2)
        best = min(row[a + "_us"] for a in algos)
        row["speedup_vs_nccl_unfused"] = round(row["nccl_unfused_us"] / best, 2)
        link_bytes = nbytes * (1.0 if "nvls" in algos else 2.0 * (world - 1) / world)
        row["roofline_us"] = round(link_bytes / (NVLINK_GBPS * 1e3), 2)
        row["frac_of_roofline"] = round(row["roofline_us"] / best, 3)
        row["status"] = status
        # correctness at this size (first call's output)
        out, h = arc(T, res, wc, algo=algos[-1])
        torch.cuda.synchronize()
        xs = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(xs, x)
        ref_out, ref_h = reference(xs, res, wc, 1e-6)
        row["max_abs_err"] = float((out.float() - ref_out).abs().max())
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
        dist.barrier()
    if rank == 0:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            json.dump({"world": world, "hidden": H, "nvls": bool(heap.multicast_ptr), "rows": rows}, f, indent=1)
    dist.barrier()
    heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
