#!/usr/bin/env python
"""Small, self-ending single-GPU cases for profiler captures: each runs ONE kernel of the library a few times on inputs that
are larger than L2 (126 MB) where DRAM figures matter but hold at most a few GB on the device.

    python benchmarks/profile_cases.py xcopy | peer | batch | gemm | gemm_2sm | gemm2 | allreduce | dispatch | reshard

`peer` needs two GPUs in ONE process (no second rank): GPU 0 pushes 256 MiB into GPU 1's memory over NVLink, so the link's byte
counters (nvltx__bytes / nvlrx__bytes) can be read next to the kernel's duration.

Capture (after the same command has exited 0 without the profiler), e.g.:
    ncu --set full --clock-control none -k regex:mf_moe_grouped_gemm -c 2 -o <report> python benchmarks/profile_cases.py gemm
"""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def case_xcopy():
    import torch
    import memfabric_hybrid_b200 as mf

    n = 256 << 20
    a = torch.empty(n, dtype=torch.uint8, device="cuda")
    b = torch.empty(n, dtype=torch.uint8, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    mf.native.fill_pattern(a.data_ptr(), n, 1, s)
    for _ in range(3):
        assert mf.native.xcopy(b.data_ptr(), a.data_ptr(), n, 0, s) == 0    # bulk-copy (TMA) variant
    for _ in range(3):
        assert mf.native.xcopy(b.data_ptr(), a.data_ptr(), n, -1, s) == 0   # load/store variant
    torch.cuda.synchronize()
    assert torch.equal(a, b)


def case_peer():
    import torch
    import memfabric_hybrid_b200 as mf

    assert torch.cuda.device_count() >= 2, "the peer case needs two GPUs in this process"
    n = 256 << 20
    a = torch.empty(n, dtype=torch.uint8, device="cuda:0")
    b = torch.zeros(n, dtype=torch.uint8, device="cuda:1")
    b.copy_(a)  # the first cross-device copy makes torch enable peer access both ways
    torch.cuda.synchronize(0)
    torch.cuda.synchronize(1)
    s = torch.cuda.current_stream().cuda_stream
    mf.native.fill_pattern(a.data_ptr(), n, 1, s)
    for _ in range(3):
        assert mf.native.xcopy(b.data_ptr(), a.data_ptr(), n, 0, s) == 0    # bulk-copy (TMA) variant, stores cross the link
    for _ in range(3):
        assert mf.native.xcopy(b.data_ptr(), a.data_ptr(), n, -1, s) == 0   # load/store variant
    torch.cuda.synchronize(0)
    assert torch.equal(a, b.to("cuda:0"))


def case_batch():
    import numpy as np
    import torch
    import memfabric_hybrid_b200 as mf

    from benchmarks.kv_blocks import make_requests

    span = 1 << 30
    a = torch.empty(span, dtype=torch.uint8, device="cuda")
    b = torch.empty(span, dtype=torch.uint8, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    so, sizes = make_requests(1, span, 3)
    do, _ = make_requests(1, span, 4)
    srcs = [int(a.data_ptr() + o) for o in so]
    dsts = [int(b.data_ptr() + o) for o in do]
    for _ in range(4):
        assert mf.native.batch_xcopy_inline(srcs, dsts, [int(x) for x in sizes], 0, s) == 0
    torch.cuda.synchronize()


def case_gemm(tile_n: int = 0):
    import torch
    from memfabric_hybrid_b200.ops import fp8_gemm as F

    G, per, N, K = 8, 512, 4096, 7168
    g = torch.Generator(device="cuda").manual_seed(1)
    rows = G * per
    a_q, a_s = F.quant_act_mx_torch(torch.randn(rows, K, generator=g, device="cuda"))
    w_q = torch.empty(G, N, K, dtype=torch.float8_e4m3fn, device="cuda")
    w_s = torch.empty(G, N // 128, K // 128, dtype=torch.float32, device="cuda")
    for e in range(G):
        w_q[e], w_s[e] = F.quant_weight_mx_torch(torch.randn(N, K, generator=g, device="cuda") * 0.02)
    offs = torch.arange(0, rows + 1, per, dtype=torch.int32, device="cuda")
    cnts = torch.full((G,), per, dtype=torch.int32, device="cuda")
    out = torch.empty(rows, N // 2, dtype=torch.float8_e4m3fn, device="cuda")
    out_sf = torch.empty(rows, N // 64, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    for _ in range(3):
        F.grouped_gemm_mx(a_q, a_s, w_q, w_s, offs, cnts, mode="swiglu_fp8", out=out, out_sf=out_sf, tile_n=tile_n)
    torch.cuda.synchronize()


def case_gemm_2sm():
    """The `gemm` case on the two-SM kernel (256 x 256 tiles by CTA pairs)."""
    case_gemm(tile_n=512)


def case_gemm2():
    """The second FFN GEMM of the expert layer: short K, bf16 epilogue (12 experts x 512 rows, N 7168, K 2048; weights 176 MB)."""
    import torch
    from memfabric_hybrid_b200.ops import fp8_gemm as F

    G, per, N, K = 12, 512, 7168, 2048
    g = torch.Generator(device="cuda").manual_seed(1)
    rows = G * per
    a_q, a_s = F.quant_act_mx_torch(torch.randn(rows, K, generator=g, device="cuda"), block=32)
    w_q = torch.empty(G, N, K, dtype=torch.float8_e4m3fn, device="cuda")
    w_s = torch.empty(G, N // 128, K // 128, dtype=torch.float32, device="cuda")
    for e in range(G):
        w_q[e], w_s[e] = F.quant_weight_mx_torch(torch.randn(N, K, generator=g, device="cuda") * 0.02)
    offs = torch.arange(0, rows + 1, per, dtype=torch.int32, device="cuda")
    cnts = torch.full((G,), per, dtype=torch.int32, device="cuda")
    out = torch.empty(rows, N, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    for _ in range(3):
        F.grouped_gemm_mx(a_q, a_s, w_q, w_s, offs, cnts, mode="bf16", out=out)
    torch.cuda.synchronize()


def case_allreduce():
    import torch
    from memfabric_hybrid_b200.ops.allreduce import emulated_allreduce
    from memfabric_hybrid_b200.parallel.heap import EmulatedHeap

    world, T, H = 4, 2048, 8192   # 32 MiB per rank, 128 MiB over the four emulated ranks
    heap = EmulatedHeap(world, 2 * T * H * 2 + 8192)
    x_off, r_off = heap.alloc(T * H * 2), heap.alloc(T * H * 2)
    res = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    w = torch.ones(H, dtype=torch.bfloat16, device="cuda")
    for r in range(world):
        heap.tensor(r, x_off, (T, H), torch.bfloat16).normal_()
    for _ in range(3):
        outs, status = emulated_allreduce(heap, x_off, r_off, [res] * world, w, T, H, 1e-6, "twoshot")
        assert status == [0] * world


def case_dispatch():
    import torch
    from memfabric_hybrid_b200.ops import fp8_gemm as F
    from memfabric_hybrid_b200.ops.moe import EmulatedMoE, route
    from memfabric_hybrid_b200.parallel.heap import EmulatedHeap

    world, T, H, E, K, I = 4, 1024, 7168, 32, 8, 256
    g = torch.Generator(device="cuda").manual_seed(2)
    weights = []
    for _ in range(world):
        el = E // world
        w13 = F.quant_weight_mx_torch(torch.randn(el, 2 * I, H, generator=g, device="cuda") * 0.01)
        w2 = F.quant_weight_mx_torch(torch.randn(el, H, I, generator=g, device="cuda") * 0.02)
        weights.append((w13[0], w13[1], w2[0], w2[1]))
    xs = [torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
    routed = [route(torch.randn(T, E, generator=g, device="cuda"), K) for _ in range(world)]
    cap = T * K * 2 + (E // world) * 128
    heap = EmulatedHeap(world, world * E * 4 + cap * (H + H // 128 * 4 + 16 + 56) + T * K * H * 2 + (4 << 20))
    layer = EmulatedMoE(heap, T, H, E, K, I, weights, capacity_factor=2.0)
    for _ in range(2):
        outs, status = layer(xs, [r[0] for r in routed], [r[1] for r in routed])
        assert status == [0] * world, status


def case_reshard():
    import torch
    from memfabric_hybrid_b200.models import LlamaConfig, param_specs
    from memfabric_hybrid_b200.ops.reshard import ReshardPlan, emulated_reshard
    from memfabric_hybrid_b200.parallel.heap import EmulatedHeap

    world, tp = 4, 4
    cfg = LlamaConfig(layers=2, hidden=4096, heads=32, kv_heads=8, ffn=14336, vocab=16384)
    specs = param_specs(cfg)
    plans = [ReshardPlan(specs, world, r % tp, tp, fp8=True) for r in range(world)]
    p0 = plans[0]
    heap = EmulatedHeap(world, p0.shard_elems * 2 + 4096)
    off = heap.alloc(p0.shard_elems * 2)
    for r in range(world):
        heap.tensor(r, off, (p0.shard_elems,), torch.bfloat16).normal_(0, 0.02)
    for _ in range(2):
        res = emulated_reshard(heap, plans, off)
        assert all(st == 0 for _, _, st in res)


if __name__ == "__main__":
    import torch

    torch.cuda.set_device(0)
    {"xcopy": case_xcopy, "peer": case_peer, "batch": case_batch, "gemm": case_gemm, "gemm_2sm": case_gemm_2sm, "gemm2": case_gemm2, "allreduce": case_allreduce, "dispatch": case_dispatch, "reshard": case_reshard}[sys.argv[1]]()
    print("ok", sys.argv[1])
