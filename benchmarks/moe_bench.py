#!/usr/bin/env python
"""MoE expert-parallel layer, DeepSeek-V3-shaped: hidden 7168, 256 routed experts (256/N per rank), top-8, SwiGLU expert FFN
with intermediate 2048, activations bf16 N(0,1) quantised on dispatch to e4m3 with 1x128 power-of-two scales, expert weights
random-init e4m3 with 128x128 power-of-two scales. Tokens per rank: 128 (decode) and 4096 (prefill). Router logits N(0,1) → softmax → top-k →
renormalised weights.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/moe_bench.py [--tokens 128,4096]

Ours: fused dispatch kernel → tcgen05 grouped FP8 GEMMs → fused combine kernel (memfabric_hybrid_b200.ops.moe.FusedMoE).
Baseline: NCCL all-to-all (bf16 tokens) + cuBLAS bf16 matmul per expert + NCCL all-to-all back + index_add reduction.
Device-timed with CUDA events, max over ranks; per phase and end to end.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch
    import torch.distributed as dist

    from benchmarks import workloads
    from memfabric_hybrid_b200.parallel.heap import SymmetricHeap
    from memfabric_hybrid_b200.parallel.pool import env_rank_world

    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="128,4096")
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--capacity-factor", type=float, default=2.0)
    ap.add_argument("--out", default="", help="also write the rows to this JSON file")
    args = ap.parse_args()
    rank, local, world = env_rank_world()
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    H, E, K, I = args.hidden, args.experts, args.topk, args.inter
    token_list = [int(t) for t in args.tokens.split(",")]
    heap = SymmetricHeap(rank, world, local, workloads.moe_heap_bytes(max(token_list), world, E, H, K, args.capacity_factor))
    rows = workloads.moe_layer(heap, token_list, hidden=H, experts_per_rank=E // world, topk=K, inter=I, iters=args.iters,
                               capacity_factor=args.capacity_factor)
    if rank == 0:
        for row in rows:
            print(json.dumps(row), flush=True)
    if rank == 0 and args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            json.dump({"world": world, "hidden": H, "experts": E, "topk": K, "inter": I, "rows": rows}, f, indent=1)
    dist.barrier()
    heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
