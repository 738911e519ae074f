#!/usr/bin/env python
"""RL weight reshard, Llama-3-8B-shaped (32 layers, hidden 4096, 32/8 heads, FFN 14336, vocab 128256), random-init bf16.
Source: FSDP flat shards over N ranks. Destination: TP = min(4, N) x DP = N / TP inference layout (column/row splits of
qkv/o/gate/up/down, vocab-parallel embeddings), bf16 and with the e4m3 128x128 cast.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/reshard_bench.py

Ours: one gather kernel that pulls this rank's sub-blocks from the owners' shards over the GVA and casts in flight.
Baseline: NCCL all_gather_into_tensor of the full flat vector, then slice (+ PyTorch block quantisation). Device-timed,
max over ranks. Roofline: bytes this rank must pull over NVLink ((N-1)/N of its destination's source bytes) / 770 GB/s.
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

    from memfabric_hybrid_b200.models import LLAMA3_8B, LlamaConfig, param_specs
    from benchmarks import workloads
    from memfabric_hybrid_b200.ops.reshard import ReshardPlan
    from memfabric_hybrid_b200.parallel.heap import SymmetricHeap
    from memfabric_hybrid_b200.parallel.pool import env_rank_world

    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--out", default="", help="also write the result to this JSON file")
    args = ap.parse_args()
    rank, local, world = env_rank_world()
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = LLAMA3_8B if args.layers == 32 else LlamaConfig(layers=args.layers)
    p = ReshardPlan(param_specs(cfg), world, 0, min(4, world))
    heap = SymmetricHeap(rank, world, local, p.shard_elems * 2 + (4 << 20))
    rows = workloads.reshard_llama(heap, layers=args.layers, iters=args.iters)
    if rank == 0:
        print(json.dumps(rows), flush=True)
        if args.out:
            os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
            with open(args.out, "w") as f:
                json.dump(rows, f, indent=1)
    dist.barrier()
    heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
