"""Short, importable measurements of every workload of the benchmark configuration, shared by bench.py (which reports them
next to its headline number at every GPU count) and by the per-workload scripts in this folder.

All times are device times (CUDA events on the launching stream, synchronised on both sides, after warm-up), reduced with
MAX over ranks. Every function takes an already opened heap or pool and leaves it open. With one rank the collectives
degenerate (no peer traffic) but the same kernels run; the NCCL baselines then skip their collective call.
"""
from __future__ import annotations

import time
from typing import Dict, List

NVLINK_GBPS = 770.0  # measured peer-copy rate per direction on this platform (copy engine)


def _dist():
    import torch.distributed as dist

    return dist if dist.is_available() and dist.is_initialized() else None


def max_over_ranks(v: float) -> float:
    import torch

    d = _dist()
    if d is None:
        return v
    t = torch.tensor([v], dtype=torch.float64, device="cuda")
    d.all_reduce(t, op=d.ReduceOp.MAX)
    return float(t.item())


def barrier() -> None:
    d = _dist()
    if d is not None:
        d.barrier()


def timed_us(fn, iters: int, warmup: int = 3, stream=None) -> float:
    """Mean device time of fn in microseconds, max over ranks."""
    import torch

    stream = stream or torch.cuda.current_stream()
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(iters):
        fn()
    b.record(stream)
    torch.cuda.synchronize()
    return max_over_ranks(a.elapsed_time(b)) * 1e3 / iters


# ---------------------------------------------------------------------------------------------- all-reduce + residual + RMSNorm


def _graph_us(call, prepare, iters: int, calls_per_graph: int = 10, check=None) -> float:
    """Microseconds per call when `calls_per_graph` calls are captured into one CUDA graph and the graph is replayed `iters`
    times. call(stream) issues one call on the capture stream; prepare() runs before capture (fills inputs)."""
    import torch

    prepare()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            call(side)  # warm-up outside the graph: argument blocks uploaded, both input buffers seen
    torch.cuda.synchronize()
    barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(calls_per_graph):
                call(side)
    torch.cuda.synchronize()
    barrier()
    graph.replay()  # one replay on its own first: a replay that cannot complete must not be repeated iters times
    torch.cuda.synchronize()
    if check is not None and check() != 0:
        raise RuntimeError(f"status {check()} after the first replay")
    return timed_us(graph.replay, iters) / calls_per_graph


def allreduce_sizes(heap, sizes: List[int], hidden: int = 8192, iters: int = 20, baselines: bool = True) -> List[Dict]:
    """Fused all-reduce + residual add + RMSNorm (bf16, eps 1e-6) for each x size in bytes, every algorithm that applies,
    against NCCL all-reduce + separate add and norm kernels and against NCCL all-reduce alone."""
    import torch

    from memfabric_hybrid_b200.ops.allreduce import AllReduceRMSNorm, reference

    d = _dist()
    world, rank = heap.world, heap.rank
    H = hidden
    max_T = max(1, max(sizes) // (H * 2))
    ar = AllReduceRMSNorm(heap, max_T, H, eps=1e-6)
    # Small inputs are also timed as a replayed CUDA graph (ten calls per graph), which is how a decode step runs them: the
    # launch overhead of the host loop disappears from the figure. Needs the device-resident epochs and its own signal channel.
    graph_max = 4 << 20
    small_T = max([max(1, n // (H * 2)) for n in sizes if n <= graph_max], default=0)
    ar_g = AllReduceRMSNorm(heap, small_T, H, eps=1e-6, channel=1, device_epochs=True, timeout_ns=200_000_000) if small_T else None
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    gc = torch.Generator(device="cuda").manual_seed(7)  # residual and weight are replicated across tensor-parallel ranks
    w = (1.0 + 0.1 * torch.randn(H, generator=gc, device="cuda")).to(torch.bfloat16)
    rows = []
    for nbytes in sizes:
        T = max(1, nbytes // (H * 2))
        x = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16)
        res = torch.randn(T, H, generator=gc, device="cuda").to(torch.bfloat16)
        for buf in ar._xs:  # the same addend in both input buffers: timed calls alternate between them
            buf[:T].copy_(x)
        torch.cuda.synchronize()
        barrier()
        row = {"bytes": T * H * 2, "T": T, "H": H}
        algos = (["oneshot"] if nbytes <= (4 << 20) else []) + ["twoshot"] + (["nvls"] if heap.multicast_ptr else [])
        it = iters if nbytes <= (64 << 20) else max(3, iters // 4)
        for algo in algos:
            row[algo + "_us"] = round(timed_us(lambda: ar(T, res, w, algo=algo), it), 2)
        row["auto_us"] = round(timed_us(lambda: ar(T, res, w), it), 2)
        row["status"] = ar.check_status()
        if ar_g is not None and nbytes <= graph_max:
            try:
                row["auto_graph_us"] = round(_graph_us(lambda s: ar_g(T, res, w, stream=s), lambda: [b[:T].copy_(x) for b in ar_g._xs], it,
                                                       check=ar_g.check_status), 2)
            except Exception as e:  # noqa: BLE001
                row["graph_error"] = repr(e)[:160]
        best = min(row[a + "_us"] for a in algos)
        if baselines:
            xb = x.clone()

            def unfused():
                y = xb.clone()
                if d is not None:
                    d.all_reduce(y)
                h = y + res
                hf = h.float()
                return (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16) * w, h

            row["nccl_unfused_us"] = round(timed_us(unfused, it), 2)
            if d is not None:
                xb2 = x.clone()
                row["nccl_allreduce_only_us"] = round(timed_us(lambda: d.all_reduce(xb2), it), 2)
                if nbytes <= graph_max:
                    try:
                        row["nccl_allreduce_only_graph_us"] = round(_graph_us(lambda s: d.all_reduce(xb2), lambda: None, it), 2)
                    except Exception as e:  # noqa: BLE001 - a library that refuses capture must not take the row down
                        row["nccl_graph_error"] = repr(e)[:120]
            row["speedup_vs_nccl_unfused"] = round(row["nccl_unfused_us"] / best, 2)
        if world > 1:
            link_bytes = row["bytes"] * (1.0 if "nvls" in algos else 2.0 * (world - 1) / world)
            row["nvlink_floor_us"] = round(link_bytes / (NVLINK_GBPS * 1e3), 2)
            row["frac_of_nvlink_floor"] = round(row["nvlink_floor_us"] / best, 3)
        out, _ = ar(T, res, w)
        torch.cuda.synchronize()
        xs = [x]
        if d is not None:
            xs = [torch.empty_like(x) for _ in range(world)]
            d.all_gather(xs, x)
        ref_out, _ = reference(xs, res, w, 1e-6)
        row["max_abs_err"] = round(float((out.float() - ref_out).abs().max()), 5)
        rows.append(row)
        barrier()
    return rows


# ---------------------------------------------------------------------------------------------- MoE dispatch + experts + combine


def make_moe_weights(el: int, hidden: int, inter: int, seed: int):
    """Random-init expert weights of one rank, quantised expert by expert (bounds the fp32 temporaries)."""
    import torch

    from memfabric_hybrid_b200.ops import fp8_gemm as F

    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(seed)
    w13_q = torch.empty(el, 2 * inter, hidden, dtype=torch.float8_e4m3fn, device=dev)
    w13_s = torch.empty(el, 2 * inter // 128, hidden // 128, dtype=torch.float32, device=dev)
    w2_q = torch.empty(el, hidden, inter, dtype=torch.float8_e4m3fn, device=dev)
    w2_s = torch.empty(el, hidden // 128, inter // 128, dtype=torch.float32, device=dev)
    for e in range(el):
        wg = torch.randn(inter, hidden, generator=g, device=dev) * hidden ** -0.5
        wu = torch.randn(inter, hidden, generator=g, device=dev) * hidden ** -0.5
        w13_q[e], w13_s[e] = F.quant_weight_mx_torch(F.interleave_gate_up(wg, wu))
        w2_q[e], w2_s[e] = F.quant_weight_mx_torch(torch.randn(hidden, inter, generator=g, device=dev) * inter ** -0.5)
    return w13_q, w13_s, w2_q, w2_s


def moe_heap_bytes(tokens: int, world: int, experts: int, hidden: int, topk: int, factor: float) -> int:
    from memfabric_hybrid_b200.ops.moe import capacity_rows

    cap = capacity_rows(tokens, topk, world, experts // world, factor)
    return world * experts * 4 + cap * (hidden + hidden // 128 * 4 + 16 + 56) + tokens * topk * hidden * 2 + (16 << 20)


def moe_layer(heap, token_list: List[int], hidden: int = 7168, experts_per_rank: int = 32, topk: int = 8, inter: int = 2048, iters: int = 10,
              capacity_factor: float = 2.0, baselines: bool = True) -> List[Dict]:
    """Expert-parallel MoE layer (DeepSeek-V3 shapes: 32 experts per rank, i.e. 256 at 8 ranks): fused dispatch → block-scaled
    tcgen05 grouped GEMMs → fused combine, per phase and in total, against NCCL all-to-all + cuBLAS bf16 matmul per expert."""
    import torch

    from memfabric_hybrid_b200.ops import fp8_gemm as F
    from memfabric_hybrid_b200.ops.moe import FusedMoE, route

    d = _dist()
    world, rank = heap.world, heap.rank
    H, K, I, EL = hidden, topk, inter, experts_per_rank
    E = EL * world
    dev = "cuda"
    Tmax = max(token_list)
    w13_q, w13_s, w2_q, w2_s = make_moe_weights(EL, H, I, 1000 + rank)
    # device-resident epochs, so that the layer can also be replayed from a CUDA graph (eager calls work the same way)
    layer = FusedMoE(heap, Tmax, H, E, K, I, w13_q, w13_s, w2_q, w2_s, capacity_factor=capacity_factor, device_epochs=True)
    w13_bf = w2_bf = None
    if baselines:
        w13_bf = torch.empty(EL, 2 * I, H, dtype=torch.bfloat16, device=dev)
        w2_bf = torch.empty(EL, H, I, dtype=torch.bfloat16, device=dev)
        for e in range(EL):
            w13_bf[e] = F.dequant_weight(w13_q[e], w13_s[e]).to(torch.bfloat16)
            w2_bf[e] = F.dequant_weight(w2_q[e], w2_s[e]).to(torch.bfloat16)

    def a2a(out, inp, out_split=None, in_split=None):
        if d is not None:
            d.all_to_all_single(out, inp, out_split, in_split)
        else:
            out.copy_(inp)

    def baseline(x, idx, w):
        T = x.shape[0]
        flat_e = idx.reshape(-1).long()
        order = torch.argsort(flat_e, stable=True)
        src_tok = order // K
        send = x[src_tok]
        counts = torch.bincount(flat_e, minlength=E)
        recv_counts = torch.empty_like(counts)
        a2a(recv_counts, counts)
        in_split = counts.view(world, EL).sum(1).tolist()
        out_split = recv_counts.view(world, EL).sum(1).tolist()
        recv = torch.empty(sum(out_split), H, dtype=torch.bfloat16, device=dev)
        a2a(recv, send, out_split, in_split)
        rc = recv_counts.view(world, EL)  # received rows are ordered by (source rank, local expert): regroup by expert
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
        a2a(ret, back, in_split, out_split)
        out = torch.zeros(T, H, dtype=torch.float32, device=dev)
        out.index_add_(0, src_tok, ret.float() * w.reshape(-1)[order].unsqueeze(1))
        return out.to(torch.bfloat16)

    rows = []
    for T in token_list:
        gi = torch.Generator(device=dev).manual_seed(77 + rank)
        x = torch.randn(T, H, generator=gi, device=dev).to(torch.bfloat16)
        idx, w = route(torch.randn(T, E, generator=gi, device=dev), K)
        it = iters if T <= 512 else max(3, iters // 2)
        row = {"tokens_per_rank": T, "world": world, "experts": E}
        row["fused_total_us"] = round(timed_us(lambda: layer(x, idx, w), it), 1)
        if T <= 512:
            # decode-sized call: four calls of the layer captured into one CUDA graph, replayed
            row["fused_total_graph_us"] = round(_graph_us(lambda s_: layer(x, idx, w, stream=s_), lambda: None, it, calls_per_graph=4,
                                                          check=layer.check_status), 1)
        row["dispatch_us"] = round(timed_us(lambda: layer.dispatch(x, idx, w), it), 1)
        row["experts_us"] = round(timed_us(lambda: layer.experts(), it), 1)
        layer.dispatch(x, idx, w)
        layer.experts()
        row["combine_us"] = round(timed_us(lambda: (layer.dispatch(x, idx, w), layer.combine(T)), it) - row["dispatch_us"], 1)
        row["status"] = layer.check_status()
        # Arrival mode: no closing barrier in dispatch, the first GEMM starts each tile when its rows have landed. Only the whole
        # layer is timed in this mode (two dispatches must be separated by a consumer that waited for every tile).
        plain = layer(x, idx, w).clone()
        layer.overlap = True
        row["fused_total_overlap_us"] = round(timed_us(lambda: layer(x, idx, w), it), 1)
        row["overlap_max_abs_diff"] = float((layer(x, idx, w).float() - plain.float()).abs().max())
        row["overlap_status"] = layer.check_status()
        barrier()
        layer.overlap = False
        flops = 2.0 * T * K * (H * 2 * I + I * H)
        row["gemm_tflops_fp8"] = round(flops / (row["experts_us"] * 1e-6) / 1e12, 1)
        if world > 1:
            remote = (world - 1) / world
            disp_bytes = T * K * remote * (H + H // 128 * 4 + 16)
            comb_bytes = T * K * remote * H * 2
            row["nvlink_floor_us"] = round((disp_bytes + comb_bytes) / (NVLINK_GBPS * 1e3), 1)
        if baselines:
            ours = layer(x, idx, w).clone()
            row["nccl_cublas_total_us"] = round(timed_us(lambda: baseline(x, idx, w), it), 1)
            ref = baseline(x, idx, w)
            torch.cuda.synchronize()
            scale = float(ref.float().abs().max()) + 1e-6
            row["max_err_vs_bf16_baseline_rel"] = round(float((ours.float() - ref.float()).abs().max()) / scale, 4)
            row["speedup"] = round(row["nccl_cublas_total_us"] / row["fused_total_us"], 2)
        rows.append(row)
        barrier()
    return rows


# ---------------------------------------------------------------------------------------------- RL weight reshard


def reshard_llama(heap, layers: int = 32, iters: int = 5, baselines: bool = True) -> Dict:
    """Llama-3-8B-shaped FSDP flat shards over all ranks → TP = min(4, N) x DP inference layout, bf16 and with the e4m3
    128x128 cast, against NCCL all-gather + slice (+ PyTorch block quantisation)."""
    import torch

    from memfabric_hybrid_b200.models import LLAMA3_8B, LlamaConfig, param_specs
    from memfabric_hybrid_b200.ops.fp8_gemm import quant_weight_torch
    from memfabric_hybrid_b200.ops.reshard import Resharder, ReshardPlan, reference_reshard

    d = _dist()
    world, rank = heap.world, heap.rank
    cfg = LLAMA3_8B if layers == 32 else LlamaConfig(layers=layers)
    specs = param_specs(cfg)
    tp = min(4, world)
    plans = {fp8: ReshardPlan(specs, world, rank % tp, tp, fp8=fp8) for fp8 in (False, True)}
    p = plans[False]
    rs = {False: Resharder(heap, plans[False])}
    rs[True] = Resharder(heap, plans[True], shard=(rs[False].shard_off, rs[False].shard))
    g = torch.Generator(device="cuda").manual_seed(500 + rank)
    shard = rs[False].shard
    for lo in range(0, p.shard_elems, 1 << 26):
        n = min(1 << 26, p.shard_elems - lo)
        shard[lo:lo + n] = (torch.randn(n, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    torch.cuda.synchronize()
    barrier()
    out: Dict = {"world": world, "tp": tp, "layers": cfg.layers, "params": p.total_elems}
    for fp8 in (False, True):
        us = timed_us(lambda: rs[fp8].launch(), iters, warmup=2)
        pulled = plans[fp8].bytes_pulled()
        row = {"fused_ms": round(us / 1e3, 3), "dest_GB": round(plans[fp8].dst_bytes / 1e9, 3), "pulled_GB": round(pulled / 1e9, 3),
               "pull_GBps": round(pulled / us / 1e3, 1), "status": rs[fp8].check_status()}
        if world > 1:
            row["nvlink_floor_ms"] = round(pulled * (world - 1) / world / (NVLINK_GBPS * 1e6), 3)
            row["frac_of_nvlink_floor"] = round(row["nvlink_floor_ms"] / row["fused_ms"], 3)
        out["fp8" if fp8 else "bf16"] = row
    full = torch.empty(p.shard_elems * world, dtype=torch.bfloat16, device="cuda")

    def gather():
        if d is not None:
            d.all_gather_into_tensor(full, shard)
        else:
            full.copy_(shard)

    if baselines:
        def base(fp8):
            gather()
            res = {}
            for e in plans[fp8].entries:
                w = full[e.src_off:e.src_off + e.spec.numel]
                if len(e.spec.shape) == 1:
                    res[e.spec.name] = w.clone()
                    continue
                blk = w.view(*e.spec.shape)[e.r0:e.r0 + e.nrows, e.c0:e.c0 + e.ncols].contiguous()
                res[e.spec.name] = quant_weight_torch(blk) if e.quant else blk
            return res

        out["bf16"]["nccl_allgather_slice_ms"] = round(timed_us(lambda: base(False), max(2, iters // 2), warmup=1) / 1e3, 3)
        out["fp8"]["nccl_allgather_slice_ms"] = round(timed_us(lambda: base(True), 2, warmup=1) / 1e3, 3)
        for k in ("bf16", "fp8"):
            out[k]["speedup"] = round(out[k]["nccl_allgather_slice_ms"] / out[k]["fused_ms"], 2)
    gather()
    ref = reference_reshard(full, plans[False])
    views = rs[False]()
    torch.cuda.synchronize()
    out["bf16"]["bit_exact_first40"] = bool(all(torch.equal(views[e.spec.name].reshape(-1), ref[e.spec.name].reshape(-1)) for e in plans[False].entries[:40]))
    del full
    return out


# ---------------------------------------------------------------------------------------------- peer copy, single


def peer_copy_rates(pool, sizes: List[int], iters: int = 10) -> List[Dict]:
    """Rank r → r+1 copies through the Big Memory API (push: the source rank runs the kernel; pull: the destination rank does)
    next to cudaMemcpyAsync on the same addresses. Per-GPU GB/s (1e9), max-over-ranks time."""
    import torch

    import memfabric_hybrid_b200 as mf

    rank, world = pool.rank, pool.world
    G2G = mf.bm.BmCopyType.G2G
    stream = torch.cuda.current_stream()
    sh = stream.cuda_stream
    top = max(sizes)
    me, nxt = pool.hbm(rank), pool.hbm((rank + 1) % world)
    rows = []
    for n in sizes:
        it = iters if n <= (64 << 20) else max(3, iters // 3)
        row = {"bytes": n}
        cases = {
            "push": lambda: pool.handle.copy_data_on_stream(me, nxt + top, n, G2G, sh, 0),
            "pull": lambda: pool.handle.copy_data_on_stream(nxt, me + top, n, G2G, sh, 0),
            "copy_engine_push": lambda: mf.native.copy_engine(nxt + top, me, n, sh),
        }
        for name, fn in cases.items():
            us = timed_us(fn, it, stream=stream)
            row[name + "_us"] = round(us, 2)
            row[name + "_GBps"] = round(n / us / 1e3, 2)
        rows.append(row)
    return rows


# ---------------------------------------------------------------------------------------------- KV-cache block batches


def percentile(xs, p):
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(round(p / 100.0 * (len(xs) - 1))))]


def kv_measure(handle, srcs, dsts, sizes, copy_type, stream, iters, native=None) -> Dict:
    """One batch-copy call per batch: p50 / p99 wall latency of the blocking call, device time of the enqueued work, GB/s;
    with `native`, also one cudaMemcpyAsync per block (what a copy-engine implementation does)."""
    import torch

    n = len(sizes)
    total = int(sum(sizes))
    for _ in range(3):
        assert handle.copy_data_batch(srcs, dsts, sizes, n, copy_type, 0) == 0
    barrier()
    lat = []
    for _ in range(iters):
        t0 = time.perf_counter()
        rc = handle.copy_data_batch(srcs, dsts, sizes, n, copy_type, 0)
        lat.append((time.perf_counter() - t0) * 1e6)
        assert rc == 0
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record(stream)
    for _ in range(iters):
        handle.copy_data_batch_on_stream(srcs, dsts, sizes, copy_type, stream.cuda_stream, 0)
    b.record(stream)
    torch.cuda.synchronize()
    dev_us = a.elapsed_time(b) * 1e3 / iters
    out = {"p50_us": round(max_over_ranks(percentile(lat, 50)), 1), "p99_us": round(max_over_ranks(percentile(lat, 99)), 1),
           "device_us": round(max_over_ranks(dev_us), 1)}
    out["GBps_p50"] = round(total / (out["p50_us"] * 1e-6) / 1e9, 1)
    out["GBps_device"] = round(total / (out["device_us"] * 1e-6) / 1e9, 1)
    if native is not None:
        for _ in range(2):
            for s, d_, z in zip(srcs, dsts, sizes):
                native.copy_engine(d_, s, z, stream.cuda_stream)
            stream.synchronize()
        lat2 = []
        for _ in range(max(5, iters // 4)):
            t0 = time.perf_counter()
            for s, d_, z in zip(srcs, dsts, sizes):
                native.copy_engine(d_, s, z, stream.cuda_stream)
            stream.synchronize()
            lat2.append((time.perf_counter() - t0) * 1e6)
        out["per_block_memcpy_p50_us"] = round(max_over_ranks(percentile(lat2, 50)), 1)
    return out
