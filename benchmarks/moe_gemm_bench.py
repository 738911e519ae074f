#!/usr/bin/env python
"""Grouped block-scaled FP8 expert GEMM (tcgen05 kernel) versus cuBLAS bf16 matmuls on the same dequantised operands.
DeepSeek-V3 expert shapes per rank at EP=8: 32 experts, FFN1 [rows, 7168] x [4096, 7168]^T with the SwiGLU epilogue and
FFN2 [rows, 2048] x [7168, 2048]^T; rows per expert 32 (decode: 128 tokens/rank) and 1024 (prefill: 4096 tokens/rank).

    python benchmarks/moe_gemm_bench.py [--out FILE.json] [--small]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch

    from memfabric_hybrid_b200.ops import fp8_gemm as F

    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--small", action="store_true", help="one small case (for profiler captures)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--tile-n", type=int, default=0, help="0 = let the launcher choose; 128, 224 (bf16 epilogue only) or 256")
    ap.add_argument("--cases", default="", help="comma list of case names to run (default: all)")
    ap.add_argument("--packed", action="store_true", help="weights in the 4 KiB-block layout of ops.fp8_gemm.pack_weight_mx")
    ap.add_argument("--ctas", type=int, default=0, help="persistent CTAs of the GEMM (0 = one per SM)")
    ap.add_argument("--no-baseline", action="store_true", help="skip the cuBLAS comparison")
    args = ap.parse_args()
    torch.cuda.set_device(0)
    dev = "cuda"
    G = 32
    cases = [("ffn1_decode", 32, 4096, 7168, "swiglu"), ("ffn2_decode", 32, 7168, 2048, "bf16"),
             ("ffn1_prefill", 1024, 4096, 7168, "swiglu"), ("ffn2_prefill", 1024, 7168, 2048, "bf16")]
    if args.small:
        G, cases = 8, [("ffn1_small", 256, 4096, 7168, "swiglu")]
    if args.cases:
        cases = [c for c in cases if c[0] in args.cases.split(",")]
    rows_out = []
    stream = torch.cuda.current_stream()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for name, per, N, K, mode in cases:
        g = torch.Generator(device=dev).manual_seed(N + K + per)
        counts = [per] * G
        offs, cur = [], 0
        for c in counts:
            offs.append(cur)
            cur += (c + 127) // 128 * 128
        offs.append(cur)
        offs_t = torch.tensor(offs, dtype=torch.int32, device=dev)
        cnts_t = torch.tensor(counts, dtype=torch.int32, device=dev)
        a = torch.randn(cur, K, generator=g, device=dev)
        a_q, a_s = F.quant_act_mx_torch(a)
        del a
        w_q = torch.empty(G, N, K, dtype=torch.float8_e4m3fn, device=dev)
        w_s = torch.empty(G, N // 128, K // 128, dtype=torch.float32, device=dev)
        for e in range(G):  # random-init expert by expert to bound the fp32 temporaries
            q, s_ = F.quant_weight_mx_torch(torch.randn(N, K, generator=g, device=dev) * 0.02)
            w_q[e], w_s[e] = q, s_
        w_ref = w_q
        if args.packed:
            w_q = F.pack_weight_mx(w_q)
        out = torch.empty(cur, N // 2 if mode == "swiglu" else N, dtype=torch.bfloat16, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)

        out_q = torch.empty(cur, N // 2, dtype=torch.float8_e4m3fn, device=dev) if mode == "swiglu" else None
        out_sf = torch.empty(cur, N // 64, dtype=torch.uint8, device=dev) if mode == "swiglu" else None

        def run():
            # the layer's configuration: SwiGLU + 1x32 quantisation fused into the first GEMM, bf16 out of the second
            if mode == "swiglu":
                F.grouped_gemm_mx(a_q, a_s, w_q, w_s, offs_t, cnts_t, mode="swiglu_fp8", out=out_q, out_sf=out_sf, status=status, tile_n=args.tile_n, ctas=args.ctas)
            else:
                F.grouped_gemm_mx(a_q, a_s, w_q, w_s, offs_t, cnts_t, mode="bf16", out=out, status=status, tile_n=args.tile_n, ctas=args.ctas)

        for _ in range(3):
            run()
        torch.cuda.synchronize()
        times = []
        for _ in range(args.iters):
            flush.fill_(1)  # cold L2 between timed iterations
            a_ev, b_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a_ev.record(stream)
            run()
            b_ev.record(stream)
            torch.cuda.synchronize()
            times.append(a_ev.elapsed_time(b_ev))
        ms = sorted(times)[len(times) // 2]
        flops = 2.0 * sum(counts) * N * K
        # baseline: cuBLAS bf16, one matmul per expert on dequantised operands (what a library implementation does)
        a_bf = F.dequant_act_mx(a_q, a_s).to(torch.bfloat16)
        w_bf = torch.empty(G, N, K, dtype=torch.bfloat16, device=dev)
        for e in range(G):
            w_bf[e] = F.dequant_weight(w_ref[e], w_s[e]).to(torch.bfloat16)

        def base():
            for e in range(G):
                y = a_bf[offs[e]:offs[e] + counts[e]] @ w_bf[e].T
                if mode == "swiglu":
                    y = y.view(counts[e], N // 64, 2, 32)
                    y = torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]
            return y

        for _ in range(0 if args.no_baseline else 2):
            base()
        torch.cuda.synchronize()
        bt = [0.0] if args.no_baseline else []
        for _ in range(0 if args.no_baseline else max(3, args.iters // 2)):
            flush.fill_(1)
            a_ev, b_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a_ev.record(stream)
            base()
            b_ev.record(stream)
            torch.cuda.synchronize()
            bt.append(a_ev.elapsed_time(b_ev))
        bms = sorted(bt)[len(bt) // 2]
        # correctness on one expert
        ref = F.grouped_gemm_mx_reference(a_q[:offs[1]], a_s[:offs[1]], w_ref[:1], w_s[:1], offs_t[:2], cnts_t[:1], mode=mode)
        got = F.dequant_act_mx(out_q[:counts[0]], out_sf[:counts[0]]) if mode == "swiglu" else out[:counts[0]].float()
        err = float((got - ref[:counts[0]]).abs().max() / (ref[:counts[0]].abs().max() + 1e-9))
        weight_bytes = G * N * K
        row = {"case": name, "G": G, "rows_per_expert": per, "N": N, "K": K, "mode": mode, "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1),
               "weight_GBps": round(weight_bytes / ms / 1e6, 1), "cublas_bf16_ms": round(bms, 4), "speedup": round(bms / ms, 2) if bms else None,
               "rel_err": round(err, 5), "status": int(status)}
        rows_out.append(row)
        print(json.dumps(row), flush=True)
        row["tile_n"] = args.tile_n
        del a_bf, w_bf, w_q, w_ref, w_s, a_q, a_s, out
        torch.cuda.empty_cache()
    if args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            json.dump(rows_out, f, indent=1)


if __name__ == "__main__":
    main()
