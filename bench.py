#!/usr/bin/env python
"""Headline benchmark: xcopy bandwidth over the global virtual address space (D2D, rank r → rank r+1), 1 GiB per copy.

    python bench.py --gpus N --steps K --warmup W            # N>1: launched by torch.distributed.run, one rank per GPU

The metric and its configuration follow the reference's published headline (RD2D/D2RD bandwidth at 1 GB per transfer,
README.md:119-126 of the reference; measured there as bytes/time around synchronous copies between rank barriers,
example/bm/BmBenchmark/band_width_calculator.cpp:368-407). One step = every rank copies 1 GiB of seeded random bf16 data
from its own pooled HBM to the next rank's pooled HBM through the public Big Memory API (`BigMemory.copy_data_on_stream`,
copy type G2G). With one GPU the destination is the second half of the same rank's window (a local HBM copy). The value
is the whole-job aggregate in GB/s (1 GB = 1e9 B), timed with CUDA events, max over ranks.

`--impl reference` would run the unmodified reference; its data plane only builds against Ascend CANN, so that arm reports
`unavailable` (plus, when baseline/build_ref.sh has been run, the reference's own config-store / group-barrier timings). `--impl baseline` runs the same step with stock CUDA/NCCL calls (cudaMemcpyAsync on one GPU, NCCL
send/recv ring on several) as the measured thing-to-beat on this hardware.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GiB = 1 << 30
MiB = 1 << 20
COPY_BYTES = 1 * GiB
E2E_BYTES = 64 * MiB          # per-step host→device input of the end-to-end variant
E2E_RESULT_BYTES = 4096       # per-step device→host read-back
BASELINE_GBPS = 166.47        # reference RD2D @ 1 GB (Atlas A3, README.md:123-124 of the reference)
KV_HBM_POOL = 64 * GiB        # pooled HBM per GPU of the KV-block workload
KV_DRAM_POOL_TOTAL = 256 * GiB  # pooled host DRAM of the KV-block workload, over all ranks
KV_DRAM_PER_RANK_CAP = 8 * GiB  # this script pins at most this much per rank (pinning 256 GiB takes minutes); benchmarks/kv_blocks.py runs the full size


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "baseline"])
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary measurements (KV blocks, host legs)")
    return ap.parse_args()


def reference_arm(args):
    reason = ("reference builds only against Ascend CANN (its XPU_TYPE=GPU build is a cudart memcpy shim that refuses "
              "device paths, src/smem/csrc/smem_bm/smem_bm.cpp:179-185); pip install into baseline/_ref failed")
    marker = os.path.join(ROOT, "baseline", "REFERENCE_INSTALL.txt")
    if os.path.exists(marker):
        with open(marker) as f:
            first = f.readline().strip()
        if first:
            reason = first
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    line = {"impl": "reference", "unavailable": reason}
    # What of the reference does build here is its C++ control plane (baseline/build_ref.sh); its barrier and store round
    # trips are timed with the same loop as ours (benchmarks/store_bench.cpp) so the two can be put side by side.
    ref = control_plane(os.path.join(ROOT, "baseline", "_ref", "cpp", "ref_store_bench"), max(args.gpus, 2))
    if ref is not None:
        line["control_plane"] = ref
    print(json.dumps(line))
    return 0


def control_plane(binary: str, ranks: int):
    """Runs a store micro-benchmark binary (ranks forked on this host) and returns its JSON line, or None."""
    import socket
    import subprocess

    if not os.path.exists(binary):
        return None
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    try:
        out = subprocess.run([binary, str(ranks), str(port), "200"], capture_output=True, text=True, timeout=120)
        for ln in reversed(out.stdout.strip().splitlines()):
            if ln.startswith("{"):
                rec = json.loads(ln)
                return None if "error" in rec else rec
    except (OSError, subprocess.SubprocessError, ValueError):
        pass
    return None


def max_over_ranks(value: float, world: int) -> float:
    if world == 1:
        return value
    import torch
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch

    from memfabric_hybrid_b200.parallel.pool import env_rank_world
    from memfabric_hybrid_b200.utils.timing import ClockSampler

    rank, local_rank, world = env_rank_world()
    if world != args.gpus:
        if args.gpus > 1 and world == 1:
            print(f"bench.py: --gpus {args.gpus} needs torch.distributed.run with that many ranks", file=sys.stderr)
            return 2
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist.barrier()

    steps, warmup = args.steps, max(args.warmup, 3)
    result = run_ours(args, rank, local_rank, world, steps, warmup) if args.impl == "ours" else run_baseline(args, rank, local_rank, world, steps, warmup)

    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(result))
    return 0


def seeded_bf16(nbytes: int, seed: int, out):
    """Fills `out` (uint8 CUDA tensor) with N(0,1) bf16 values from a seeded generator."""
    import torch

    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    view = out.view(torch.bfloat16)
    chunk = 64 * MiB
    for off in range(0, view.numel(), chunk):
        n = min(chunk, view.numel() - off)
        view[off:off + n] = torch.randn(n, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)


def run_ours(args, rank, local_rank, world, steps, warmup):
    import torch

    import memfabric_hybrid_b200 as mf
    from memfabric_hybrid_b200.parallel.pool import open_pool
    from memfabric_hybrid_b200.utils.tensors import device_tensor_from_gva
    from memfabric_hybrid_b200.utils.timing import ClockSampler

    bmod = mf.bm
    # Window: [0, 1 GiB) source, [1 GiB, 2 GiB) landing zone for the previous rank, then e2e staging; with the secondary
    # measurements the window is the 64 GiB pool of the KV-block workload and the blocks live in its upper part.
    hbm_bytes = 2 * COPY_BYTES + 2 * E2E_BYTES
    dram_bytes = 0
    if not args.no_extra:
        hbm_bytes = KV_HBM_POOL
        dram_bytes = min(KV_DRAM_POOL_TOTAL // world, KV_DRAM_PER_RANK_CAP)
    pool = open_pool(rank, world, local_rank, hbm_bytes, dram_bytes=dram_bytes)
    barrier(world)
    me, peer = pool.hbm(rank), pool.hbm((rank + 1) % world)
    src_addr, dst_addr = me, peer + COPY_BYTES
    src = device_tensor_from_gva(src_addr, COPY_BYTES)
    seeded_bf16(COPY_BYTES, 1234 + rank, src)
    torch.cuda.synchronize()
    barrier(world)

    stream = torch.cuda.current_stream()
    sh = stream.cuda_stream
    G2G = bmod.BmCopyType.G2G
    launches = 0

    def step():
        rc = pool.handle.copy_data_on_stream(src_addr, dst_addr, COPY_BYTES, G2G, sh, 0)
        if rc != 0:
            raise RuntimeError(f"copy failed ({rc}): {mf.get_last_err_msg()}")

    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # The clock sampler runs from the warm-up through the timed region: nvidia-smi cannot sample faster than every few tens
    # of milliseconds, so an untimed pre-load of the same copies keeps the GPU in the measured state long enough for it to
    # see the clocks this kernel runs at.
    with ClockSampler(local_rank, period_ms=50) as cs:
        for _ in range(warmup):
            step()
        t_pre = time.perf_counter()
        while time.perf_counter() - t_pre < 0.7:
            for _ in range(8):
                step()
            stream.synchronize()
        torch.cuda.synchronize()
        barrier(world)
        start.record(stream)
        for _ in range(steps):
            step()
            launches += 1
        end.record(stream)
        torch.cuda.synchronize()
        t_post = time.perf_counter()
        while time.perf_counter() - t_post < 0.15:  # let the sampler take one more reading under the same load
            step()
            stream.synchronize()
        barrier(world)
    clocks = cs.summary()
    ms = max_over_ranks(start.elapsed_time(end), world)
    ms_per_step = ms / steps
    value = world * COPY_BYTES / (ms_per_step * 1e-3) / 1e9

    # Bit-exact check of what landed here (written by rank-1) against a regenerated copy of its source.
    barrier(world)
    prev = (rank - 1) % world
    expect = torch.empty(COPY_BYTES, dtype=torch.uint8, device="cuda")
    seeded_bf16(COPY_BYTES, 1234 + prev, expect)
    landed = device_tensor_from_gva(me + COPY_BYTES, COPY_BYTES)
    exact = bool(torch.equal(landed, expect))
    del expect

    # End-to-end: pinned host input → own pool (H2G), pool → next rank's pool (G2G), 4 KiB result back to host (G2H).
    host_in = torch.empty(E2E_BYTES, dtype=torch.uint8).pin_memory()
    host_in.random_(0, 256, generator=torch.Generator().manual_seed(99 + rank))
    host_out = torch.empty(E2E_RESULT_BYTES, dtype=torch.uint8).pin_memory()
    stage = me + 2 * COPY_BYTES
    land = peer + 2 * COPY_BYTES + E2E_BYTES
    H2G, G2H = bmod.BmCopyType.H2G, bmod.BmCopyType.G2H

    def e2e_step():
        h = pool.handle
        rc = h.copy_data_on_stream(host_in.data_ptr(), stage, E2E_BYTES, H2G, sh, 0)
        rc |= h.copy_data_on_stream(stage, land, E2E_BYTES, G2G, sh, 0)
        rc |= h.copy_data_on_stream(land + E2E_BYTES - E2E_RESULT_BYTES, host_out.data_ptr(), E2E_RESULT_BYTES, G2H, sh, 0)
        if rc != 0:
            raise RuntimeError(f"e2e copy failed ({rc}): {mf.get_last_err_msg()}")
        stream.synchronize()  # the step's result is on the host before the next step starts

    for _ in range(3):
        e2e_step()
    barrier(world)
    e2e_steps = max(5, min(steps, 20))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    start.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    end.record(stream)
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks(max(start.elapsed_time(end), (time.perf_counter() - t0) * 1e3), world) / e2e_steps
    e2e_value = world * E2E_BYTES / (e2e_ms * 1e-3) / 1e9
    # What came back to this rank's host is the tail of the PREVIOUS rank's input (each rank lands its data on the next one).
    expect_in = torch.empty(E2E_BYTES, dtype=torch.uint8)
    expect_in.random_(0, 256, generator=torch.Generator().manual_seed(99 + (rank - 1) % world))
    barrier(world)
    pool.handle.copy_data_on_stream(me + 2 * COPY_BYTES + 2 * E2E_BYTES - E2E_RESULT_BYTES, host_out.data_ptr(), E2E_RESULT_BYTES, G2H, sh, 0)
    stream.synchronize()
    e2e_ok = bool(torch.equal(host_out, expect_in[-E2E_RESULT_BYTES:]))
    e2e_ok = bool(max_over_ranks(0.0 if e2e_ok else 1.0, world) == 0.0)

    # The same copy with stock calls, in the same process on the same addresses: cudaMemcpyAsync (copy engine), and for
    # several GPUs an NCCL send/recv ring.
    measured = {}

    def timed_ms(fn, n):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        barrier(world)
        start.record(stream)
        for _ in range(n):
            fn()
        end.record(stream)
        torch.cuda.synchronize()
        return max_over_ranks(start.elapsed_time(end), world) / n

    bsteps = max(3, min(steps, 10))
    ce_ms = timed_ms(lambda: mf.native.copy_engine(dst_addr, src_addr, COPY_BYTES, sh), bsteps)
    measured["cudaMemcpyAsync_GBps"] = round(world * COPY_BYTES / (ce_ms * 1e-3) / 1e9, 2)
    if world > 1:
        import torch.distributed as dist

        nbuf = torch.empty(COPY_BYTES, dtype=torch.uint8, device="cuda")

        def ring():
            ops = [dist.P2POp(dist.isend, src, (rank + 1) % world), dist.P2POp(dist.irecv, nbuf, (rank - 1) % world)]
            for wk in dist.batch_isend_irecv(ops):
                wk.wait()

        measured["nccl_sendrecv_ring_GBps"] = round(world * COPY_BYTES / (timed_ms(ring, bsteps) * 1e-3) / 1e9, 2)
        del nbuf
    measured_best = max(measured.values())

    extra = {}
    if not args.no_extra:
        extra = run_extras(pool, rank, local_rank, world, stream)
    else:
        barrier(world)
        pool.close()
    return {
        "metric": "xcopy_d2d_GBps_1GiB",
        "value": round(value, 2),
        "unit": "GB/s",
        "n_gpus": world,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": round(value / BASELINE_GBPS, 3),
        "vs_baseline_note": "whole-job aggregate over the reference's published single-pair RD2D rate on Atlas A3 (166.47 GB/s); with one GPU "
                            "the copy is local HBM to HBM, with several it crosses NVLink, so compare per-GPU figures from N=2 on",
        "per_gpu_GBps": round(value / world, 2),
        "measured_baseline": measured,
        "vs_measured_baseline": round(value / measured_best, 3),
        "dtype": "bf16",
        "data": "synthetic: seeded N(0,1) bf16 buffers, byte-compared after the run",
        "impl": "ours",
        "config": {
            "model": "xcopy D2D over GVA (BM API, copy type G2G), rank r -> r+1" if world > 1 else "xcopy D2D over GVA (BM API, copy type G2G), local HBM",
            "global_batch": world * COPY_BYTES,
            "seq_len": COPY_BYTES,
            "parallelism": f"ring{world}",
            "l2_policy": "inputs (1 GiB per copy) far exceed the 126 MB L2; no flush needed",
            "bit_exact": exact,
        },
        "clocks": {"sm_mhz": clocks.get("sm_mhz"), "sm_max_mhz": clocks.get("sm_max_mhz"), "reasons": clocks.get("reasons", [])},
        "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": E2E_BYTES, "d2h_bytes_per_step": E2E_RESULT_BYTES,
                "ms_per_step": round(e2e_ms, 4), "result_ok": e2e_ok},
        "gpu_launches": launches,
        "extra": extra,
    }


def run_extras(pool, rank, local_rank, world, stream):
    """Secondary measurements on every GPU count: peer-copy rates next to cudaMemcpyAsync, KV-block batches, then (on a symmetric
    heap) all-reduce + RMSNorm, the MoE layer and the weight reshard, each against its NCCL / cuBLAS baseline. A failure of one
    of them is recorded and never takes the headline number down. Closes the pool."""
    import torch

    from benchmarks import workloads
    from benchmarks.kv_blocks import kv_latency_quick

    extra = {}

    def guarded(name, fn):
        try:
            extra[name] = fn()
        except Exception as e:  # noqa: BLE001
            extra[name + "_error"] = repr(e)[:300]
        torch.cuda.synchronize()
        barrier(world)

    guarded("peer_copy", lambda: workloads.peer_copy_rates(pool, [64 << 10, 1 << 20, 64 << 20, 1 << 30], iters=10))
    kv_base = 4 * GiB
    guarded("kv_block", lambda: dict(kv_latency_quick(pool, rank, world, stream, iters=30, span=16 * GiB, base_off=kv_base, with_host=True),
                                     hbm_pool_bytes_per_rank=pool.hbm_bytes, dram_pool_bytes_per_rank=pool.dram_bytes,
                                     dram_pool_bytes_total=pool.dram_bytes * world))
    barrier(world)
    pool.close()
    torch.cuda.empty_cache()

    from memfabric_hybrid_b200.models import LLAMA3_8B, param_specs
    from memfabric_hybrid_b200.ops.reshard import ReshardPlan
    from memfabric_hybrid_b200.parallel.heap import SymmetricHeap

    shard_bytes = ReshardPlan(param_specs(LLAMA3_8B), world, 0, min(4, world)).shard_elems * 2
    heap_bytes = 3 * (256 << 20) + workloads.moe_heap_bytes(4096, world, 32 * world, 7168, 8, 2.0) + shard_bytes + (64 << 20)
    heap = None
    try:
        heap = SymmetricHeap(rank, world, local_rank, heap_bytes, nvls=world > 1)
    except Exception as e:  # noqa: BLE001
        extra["heap_error"] = repr(e)[:300]
        return extra
    guarded("allreduce_rmsnorm", lambda: workloads.allreduce_sizes(heap, [64 << 10, 4 << 20, 256 << 20], iters=20))
    guarded("moe_layer", lambda: workloads.moe_layer(heap, [128, 4096], iters=10))
    torch.cuda.empty_cache()
    guarded("reshard_llama3_8b", lambda: workloads.reshard_llama(heap, layers=32, iters=3))
    try:
        heap.close()
    except Exception as e:  # noqa: BLE001
        extra["heap_close_error"] = repr(e)[:200]
    if rank == 0:
        cp = control_plane(os.path.join(ROOT, "benchmarks", "store_bench"), max(world, 2))
        if cp is not None:
            extra["control_plane"] = cp
    return extra


def run_baseline(args, rank, local_rank, world, steps, warmup):
    """Same step with stock calls: torch copy_ (cudaMemcpyAsync D2D) on one GPU, an NCCL send/recv ring on several."""
    import torch

    from memfabric_hybrid_b200.utils.timing import ClockSampler

    src = torch.empty(COPY_BYTES, dtype=torch.uint8, device="cuda")
    dst = torch.empty(COPY_BYTES, dtype=torch.uint8, device="cuda")
    seeded_bf16(COPY_BYTES, 1234 + rank, src)
    stream = torch.cuda.current_stream()
    if world > 1:
        import torch.distributed as dist

        nxt, prv = (rank + 1) % world, (rank - 1) % world

        def step():
            ops = [dist.P2POp(dist.isend, src, nxt), dist.P2POp(dist.irecv, dst, prv)]
            for w in dist.batch_isend_irecv(ops):
                w.wait()
    else:
        def step():
            dst.copy_(src, non_blocking=True)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    barrier(world)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as cs:
        torch.cuda.synchronize()
        start.record(stream)
        for _ in range(steps):
            step()
        end.record(stream)
        torch.cuda.synchronize()
        barrier(world)
    clocks = cs.summary()
    ms_per_step = max_over_ranks(start.elapsed_time(end), world) / steps
    value = world * COPY_BYTES / (ms_per_step * 1e-3) / 1e9
    return {
        "metric": "xcopy_d2d_GBps_1GiB", "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": round(value / BASELINE_GBPS, 3),
        "dtype": "bf16", "data": "synthetic: seeded N(0,1) bf16 buffers", "impl": "baseline",
        "config": {"model": "cudaMemcpyAsync D2D" if world == 1 else "NCCL send/recv ring", "global_batch": world * COPY_BYTES,
                   "seq_len": COPY_BYTES, "parallelism": f"ring{world}", "l2_policy": "inputs exceed L2"},
        "clocks": {"sm_mhz": clocks.get("sm_mhz"), "sm_max_mhz": clocks.get("sm_max_mhz"), "reasons": clocks.get("reasons", [])},
        "gpu_launches": 0,
    }


if __name__ == "__main__":
    sys.exit(main())
