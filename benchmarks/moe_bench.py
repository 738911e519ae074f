#!/usr/bin/env python
"""MoE expert-parallel layer, DeepSeek-V3-shaped: hidden 7168, 256 routed experts (256/N per rank), top-8, SwiGLU expert FFN
with intermediate 2048, activations bf16 N(0,1) quantised on dispatch to e4m3 with 1x128 scales, expert weights random-init
e4m3 with 128x128 scales. Tokens per rank: 128 (decode) and 4096 (prefill). Router logits N(0,1) → softmax → top-k →
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

NVLINK_GBPS = 770.0


def main():
    import torch
    import torch.distributed as dist

    from memfabric_hybrid_b200.ops import fp8_gemm as F
    from memfabric_hybrid_b200.ops.moe import FusedMoE, capacity_rows, route
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
    ap.add_argument("--out", default="gpurun_out/moe_bench.json")
    args = ap.parse_args()
    rank, local, world = env_rank_world()
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    H, E, K, I = args.hidden, args.experts, args.topk, args.inter
    EL = E // world
    dev = "cuda"
    token_list = [int(t) for t in args.tokens.split(",")]
    Tmax = max(token_list)

    # random-init expert weights of this rank, quantised expert by expert to bound temporaries
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    w13_q = torch.empty(EL, 2 * I, H, dtype=torch.float8_e4m3fn, device=dev)
    w13_s = torch.empty(EL, 2 * I // 128, H // 128, dtype=torch.float32, device=dev)
    w2_q = torch.empty(EL, H, I, dtype=torch.float8_e4m3fn, device=dev)
    w2_s = torch.empty(EL, H // 128, I // 128, dtype=torch.float32, device=dev)
    for e in range(EL):
        wg = torch.randn(I, H, generator=g, device=dev) * H ** -0.5
        wu = torch.randn(I, H, generator=g, device=dev) * H ** -0.5
        w13_q[e], w13_s[e] = F.quant_weight_mx_torch(F.interleave_gate_up(wg, wu))
        w2_q[e], w2_s[e] = F.quant_weight_mx_torch(torch.randn(H, I, generator=g, device=dev) * I ** -0.5)
    del wg, wu

    cap = capacity_rows(Tmax, K, world, EL, args.capacity_factor)
    heap_bytes = world * E * 4 + cap * (H + H // 128 * 4 + 16) + Tmax * K * H * 2 + (16 << 20)
    heap = SymmetricHeap(rank, world, local, heap_bytes)
    layer = FusedMoE(heap, Tmax, H, E, K, I, w13_q, w13_s, w2_q, w2_s, capacity_factor=args.capacity_factor)
    stream = torch.cuda.current_stream()

    def maxr(v):
        t = torch.tensor([v], dtype=torch.float64, device=dev)
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

    # dequantised bf16 weights for the library baseline (de-interleaved once)
    w13_bf = torch.empty(EL, 2 * I, H, dtype=torch.bfloat16, device=dev)
    w2_bf = torch.empty(EL, H, I, dtype=torch.bfloat16, device=dev)
    for e in range(EL):
        w13_bf[e] = F.dequant_weight(w13_q[e], w13_s[e]).to(torch.bfloat16)
        w2_bf[e] = F.dequant_weight(w2_q[e], w2_s[e]).to(torch.bfloat16)

    def baseline(x, idx, w):
        T = x.shape[0]
        flat_e = idx.reshape(-1).long()
        order = torch.argsort(flat_e, stable=True)
        src_tok = order // K
        send = x[src_tok]
        counts = torch.bincount(flat_e, minlength=E)
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts)
        in_split = counts.view(world, EL).sum(1).tolist()
        out_split = recv_counts.view(world, EL).sum(1).tolist()
        recv = torch.empty(sum(out_split), H, dtype=torch.bfloat16, device=dev)
        dist.all_to_all_single(recv, send, out_split, in_split)
        # received rows are ordered by (source rank, local expert): regroup by expert
        rc = recv_counts.view(world, EL)
        exp_of_row = torch.repeat_interleave(torch.arange(EL, device=dev).repeat(world), rc.reshape(-1))
        perm = torch.argsort(exp_of_row, stable=True)
        xs = recv[perm]
        per_e = rc.sum(0).tolist()
        y = torch.empty_like(xs)
        lo = 0
        for e in range(EL):
            n = per_e[e]
            if n:
                h = xs[lo:lo + n] @ w13_bf[e].T
                h = h.view(n, 2 * I // 64, 2, 32)
                h = (torch.nn.functional.silu(h[:, :, 0]) * h[:, :, 1]).reshape(n, I)
                y[lo:lo + n] = h @ w2_bf[e].T
            lo += n
        back = torch.empty_like(y)
        back[perm] = y
        ret = torch.empty(T * K, H, dtype=torch.bfloat16, device=dev)
        dist.all_to_all_single(ret, back, in_split, out_split)
        out = torch.zeros(T, H, dtype=torch.float32, device=dev)
        out.index_add_(0, src_tok, ret.float() * w.reshape(-1)[order].unsqueeze(1))
        return out.to(torch.bfloat16)

    rows = []
    for T in token_list:
        gi = torch.Generator(device=dev).manual_seed(77 + rank)
        x = torch.randn(T, H, generator=gi, device=dev).to(torch.bfloat16)
        idx, w = route(torch.randn(T, E, generator=gi, device=dev), K)
        iters = args.iters if T <= 512 else max(3, args.iters // 2)
        row = {"tokens_per_rank": T, "world": world}
        row["fused_total_us"] = round(timed(lambda: layer(x, idx, w), iters), 1)
        row["dispatch_us"] = round(timed(lambda: layer.dispatch(x, idx, w), iters), 1)
        row["experts_us"] = round(timed(lambda: layer.experts(), iters), 1)
        layer.dispatch(x, idx, w)
        layer.experts()
        row["combine_us"] = round(timed(lambda: (layer.dispatch(x, idx, w), layer.combine(T)), iters) - row["dispatch_us"], 1)
        row["status"] = layer.check_status()
        ours = layer(x, idx, w).clone()
        row["nccl_cublas_total_us"] = round(timed(lambda: baseline(x, idx, w), iters), 1)
        ref = baseline(x, idx, w)
        torch.cuda.synchronize()
        scale = float(ref.float().abs().max()) + 1e-6
        row["max_err_vs_bf16_baseline_rel"] = round(float((ours.float() - ref.float()).abs().max()) / scale, 4)
        row["speedup"] = round(row["nccl_cublas_total_us"] / row["fused_total_us"], 2)
        # roofline: bytes that must cross NVLink per direction per rank, and the GEMM FLOPs at the measured fp8-capable peak
        remote = (world - 1) / world
        disp_bytes = T * K * remote * (H + H // 128 * 4 + 16)
        comb_bytes = T * K * remote * H * 2
        flops = 2.0 * T * K * (H * 2 * I + I * H)
        row["nvlink_floor_us"] = round((disp_bytes + comb_bytes) / (NVLINK_GBPS * 1e3), 1)
        row["gemm_tflops"] = round(flops / (row["experts_us"] * 1e-6) / 1e12, 1)
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
        dist.barrier()
    if rank == 0:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            json.dump({"world": world, "hidden": H, "experts": E, "topk": K, "inter": I, "rows": rows}, f, indent=1)
    dist.barrier()
    heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
