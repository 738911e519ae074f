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

NVLINK_GBPS = 770.0


def main():
    import torch
    import torch.distributed as dist

    from memfabric_hybrid_b200.models import LLAMA3_8B, LlamaConfig, param_specs
    from memfabric_hybrid_b200.ops.fp8_gemm import quant_weight_torch
    from memfabric_hybrid_b200.ops.reshard import Resharder, ReshardPlan, reference_reshard
    from memfabric_hybrid_b200.parallel.heap import SymmetricHeap
    from memfabric_hybrid_b200.parallel.pool import env_rank_world

    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--out", default="gpurun_out/reshard_bench.json")
    args = ap.parse_args()
    rank, local, world = env_rank_world()
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = LLAMA3_8B if args.layers == 32 else LlamaConfig(layers=args.layers)
    specs = param_specs(cfg)
    tp = min(4, world)
    plans = {fp8: ReshardPlan(specs, world, rank % tp, tp, fp8=fp8) for fp8 in (False, True)}
    p = plans[False]
    heap = SymmetricHeap(rank, world, local, p.shard_elems * 2 + (4 << 20))
    stream = torch.cuda.current_stream()
    rs = {fp8: Resharder(heap, plans[fp8]) for fp8 in (False,)}
    rs[True] = Resharder.__new__(Resharder)  # share the shard: build the second one by hand on the same heap buffer
    r8 = rs[True]
    r8.heap, r8.plan, r8.timeout_ns = heap, plans[True], 0
    r8.shard_off, r8.shard = rs[False].shard_off, rs[False].shard
    dev = torch.device("cuda", local)
    r8.dst = torch.empty(plans[True].dst_bytes, dtype=torch.uint8, device=dev)
    r8.scales = torch.empty(max(plans[True].scale_floats, 1), dtype=torch.float32, device=dev)
    r8.status = torch.zeros(1, dtype=torch.int32, device=dev)
    r8.table = torch.frombuffer(bytearray(plans[True].table_bytes()), dtype=torch.uint8).to(dev)
    from memfabric_hybrid_b200._loader import _pymf
    blob = _pymf.ops.pack_reshard_args(heap.meta_ptr, r8.shard.data_ptr(), r8.dst.data_ptr(), r8.scales.data_ptr(), r8.table.data_ptr(),
                                       r8.status.data_ptr(), plans[True].shard_elems, len(plans[True].entries), plans[True].total_tiles)
    r8.args = torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(dev)
    r8.launches = 0

    # random-init training shard of this rank (seeded per rank)
    g = torch.Generator(device="cuda").manual_seed(500 + rank)
    shard = rs[False].shard
    for lo in range(0, p.shard_elems, 1 << 26):
        n = min(1 << 26, p.shard_elems - lo)
        shard[lo:lo + n] = (torch.randn(n, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    torch.cuda.synchronize()
    dist.barrier()

    def maxr(v):
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, iters):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(iters):
            fn()
        b.record(stream)
        torch.cuda.synchronize()
        return maxr(a.elapsed_time(b)) / iters  # ms

    rows = {}
    for fp8 in (False, True):
        ms = timed(lambda: rs[fp8].launch(), args.iters)
        pulled = plans[fp8].bytes_pulled()
        rows["fp8" if fp8 else "bf16"] = {
            "fused_ms": round(ms, 3), "dest_GB": round(plans[fp8].dst_bytes / 1e9, 3), "pulled_GB": round(pulled / 1e9, 3),
            "pull_GBps": round(pulled / ms / 1e6, 1), "roofline_ms": round(pulled * (world - 1) / world / (NVLINK_GBPS * 1e6), 3),
            "status": rs[fp8].check_status(),
        }
    # baseline: all-gather everything, then slice (+ cast)
    full = torch.empty(p.shard_elems * world, dtype=torch.bfloat16, device="cuda")

    def base(fp8):
        dist.all_gather_into_tensor(full, shard)
        out = {}
        for e in plans[fp8].entries:
            w = full[e.src_off:e.src_off + e.spec.numel]
            if len(e.spec.shape) == 1:
                out[e.spec.name] = w.clone()
                continue
            blk = w.view(*e.spec.shape)[e.r0:e.r0 + e.nrows, e.c0:e.c0 + e.ncols].contiguous()
            out[e.spec.name] = quant_weight_torch(blk) if e.quant else blk
        return out

    rows["bf16"]["nccl_allgather_slice_ms"] = round(timed(lambda: base(False), max(2, args.iters // 2)), 3)
    rows["fp8"]["nccl_allgather_slice_ms"] = round(timed(lambda: base(True), 2), 3)
    rows["allgather_only_ms"] = round(timed(lambda: dist.all_gather_into_tensor(full, shard), max(2, args.iters // 2)), 3)
    for k in ("bf16", "fp8"):
        rows[k]["speedup"] = round(rows[k]["nccl_allgather_slice_ms"] / rows[k]["fused_ms"], 2)
        rows[k]["frac_of_roofline"] = round(rows[k]["roofline_ms"] / rows[k]["fused_ms"], 3)
    # correctness: bf16 result is bit-exact against the gathered vector
    dist.all_gather_into_tensor(full, shard)
    ref = reference_reshard(full, plans[False])
    views = rs[False]()
    torch.cuda.synchronize()
    exact = all(torch.equal(views[e.spec.name].reshape(-1), ref[e.spec.name].reshape(-1)) for e in plans[False].entries[:40])
    rows["bf16"]["bit_exact_first40"] = bool(exact)
    if rank == 0:
        print(json.dumps(rows), flush=True)
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            json.dump({"world": world, "tp": tp, "layers": cfg.layers, "params": p.total_elems, "rows": rows}, f, indent=1)
    dist.barrier()
    heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
