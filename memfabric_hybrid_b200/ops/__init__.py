"""Torch-facing wrappers of the fused kernels: allreduce (+residual+RMSNorm), MoE dispatch / grouped FP8 GEMM / combine, weight
reshard, and `smoke_all`, a quick self-check that launches every kernel of the library once on small inputs."""
from __future__ import annotations


def smoke_all(verbose: bool = False) -> dict:
    """Launches every kernel family on `cuda:<current>` with small inputs and checks each result against its PyTorch oracle:
    single copies through both copy kernels, the inline and the table batch copy, all-reduce + RMSNorm (one-shot and two-shot,
    four emulated ranks), MoE dispatch → block-scaled grouped GEMMs → combine (two emulated ranks), the fp32-scale grouped
    GEMM and the row quantiser, and the weight reshard (bf16 and fp8, four emulated ranks). Returns {name: True}; raises on
    the first mismatch."""
    import numpy as np
    import torch

    from .. import native
    from ..models import LlamaConfig, param_specs
    from ..parallel.heap import EmulatedHeap
    from . import fp8_gemm as F
    from .allreduce import emulated_allreduce, reference
    from .moe import EmulatedMoE, moe_reference, route
    from .reshard import ReshardPlan, emulated_reshard, reference_reshard

    done = {}
    s = torch.cuda.current_stream().cuda_stream
    dev = "cuda"

    def mark(name):
        done[name] = True
        if verbose:
            print("smoke:", name, "ok", flush=True)

    # ---- single copies: bulk-copy kernel (>= 4 MiB, congruent addresses), load/store kernel (misaligned), small copy
    n = 6 << 20
    a = torch.empty(n + 64, dtype=torch.uint8, device=dev)
    b = torch.zeros(n + 64, dtype=torch.uint8, device=dev)
    native.fill_pattern(a.data_ptr(), n + 64, 5, s)
    assert native.xcopy(b.data_ptr(), a.data_ptr(), n, 0, s) == 0
    torch.cuda.synchronize()
    assert torch.equal(a[:n], b[:n]) and int(b[n:].sum()) == 0
    mark("xcopy_bulk")
    b.zero_()
    assert native.xcopy(b.data_ptr() + 3, a.data_ptr() + 7, n, 0, s) == 0
    assert native.xcopy(b.data_ptr() + n + 8, a.data_ptr() + 1, 40, 0, s) == 0
    torch.cuda.synchronize()
    assert torch.equal(a[7:7 + n], b[3:3 + n]) and torch.equal(a[1:41], b[n + 8:n + 48])
    mark("xcopy_ldst")

    # ---- batch copies: 100 descriptors ride in the kernel parameters, 400 go through the staged table
    rng = np.random.default_rng(0)
    for count, name in ((100, "batch_inline"), (400, "batch_table")):
        blk = 8192
        src = torch.randint(0, 256, (count * blk,), dtype=torch.uint8, device=dev)
        dst = torch.zeros(count * blk, dtype=torch.uint8, device=dev)
        perm = rng.permutation(count)
        srcs = [src.data_ptr() + i * blk for i in range(count)]
        dsts = [dst.data_ptr() + int(p) * blk for p in perm]
        if count <= 168:
            assert native.batch_xcopy_inline(srcs, dsts, [blk] * count, 0, s) == 0
        else:
            assert native.batch_xcopy_noalloc(srcs, dsts, [blk] * count, s) == 0
        torch.cuda.synchronize()
        assert torch.equal(dst.view(count, blk)[torch.from_numpy(perm).to(dev)], src.view(count, blk))
        mark(name)

    # ---- all-reduce + residual + RMSNorm on four emulated ranks
    world, T, H = 4, 24, 4096
    g = torch.Generator(device=dev).manual_seed(1)
    xs = [torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16) for _ in range(world)]
    res = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn(H, generator=g, device=dev)).to(torch.bfloat16)
    ref_out, ref_h = reference(xs, res, w, 1e-6)
    for algo in ("oneshot", "twoshot"):
        heap = EmulatedHeap(world, 2 * T * H * 2 + 8192)
        x_off, r_off = heap.alloc(T * H * 2), heap.alloc(T * H * 2)
        for r in range(world):
            heap.tensor(r, x_off, (T, H), torch.bfloat16).copy_(xs[r])
        outs, status = emulated_allreduce(heap, x_off, r_off, [res] * world, w, T, H, 1e-6, algo)
        assert status == [0] * world, status
        for r in range(world):
            torch.testing.assert_close(outs[r].float(), ref_out, atol=2e-2, rtol=2e-2)
        mark("allreduce_" + algo)

    # ---- MoE layer on two emulated ranks: dispatch, block-scaled GEMMs (both tile widths are picked by size), combine
    world, T, H, E, K, I = 2, 48, 1024, 8, 4, 256
    weights = []
    for _ in range(world):
        el = E // world
        wg = torch.randn(el, I, H, generator=g, device=dev) * H ** -0.5
        wu = torch.randn(el, I, H, generator=g, device=dev) * H ** -0.5
        w2 = torch.randn(el, H, I, generator=g, device=dev) * I ** -0.5
        weights.append(F.quant_weight_mx_torch(F.interleave_gate_up(wg, wu)) + F.quant_weight_mx_torch(w2))
    xs = [torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16) for _ in range(world)]
    routed = [route(torch.randn(T, E, generator=g, device=dev), K) for _ in range(world)]
    idxs, ws = [r[0] for r in routed], [r[1] for r in routed]
    heap = EmulatedHeap(world, 32 << 20)
    layer = EmulatedMoE(heap, T, H, E, K, I, weights, capacity_factor=float(world))
    outs, status = layer(xs, idxs, ws)
    assert status == [0] * world, status
    for o, ref in zip(outs, moe_reference(xs, idxs, ws, weights, E, I)):
        scale = float(ref.abs().max()) + 1e-6
        assert float((o.float() - ref).abs().max()) <= 1e-1 * scale
        assert float((o.float() - ref).abs().mean()) <= 4e-3 * scale
    mark("moe_dispatch_gemm_mx_combine")

    # ---- wide-tile block-scaled GEMM (256 columns per tile), fp32-scale GEMM and the row quantiser
    rows, N, Kd = 256, 512, 512
    offs = torch.tensor([0, 128, 256], dtype=torch.int32, device=dev)
    cnts = torch.tensor([100, 128], dtype=torch.int32, device=dev)
    act = torch.randn(rows, Kd, generator=g, device=dev)
    wt = torch.randn(2, N, Kd, generator=g, device=dev) * 0.05
    a_q, a_sf = F.quant_act_mx_torch(act)
    w_q, w_s = F.quant_weight_mx_torch(wt)
    out = F.grouped_gemm_mx(a_q, a_sf, w_q, w_s, offs, cnts, tile_n=256)
    ref = F.grouped_gemm_mx_reference(a_q, a_sf, w_q, w_s, offs, cnts)
    torch.cuda.synchronize()
    torch.testing.assert_close(out[:100].float(), ref[:100], rtol=2e-2, atol=2e-2 * float(ref.abs().max()))
    torch.testing.assert_close(out[128:256].float(), ref[128:256], rtol=2e-2, atol=2e-2 * float(ref.abs().max()))
    mark("gemm_mx_tile256")
    xb = act.to(torch.bfloat16)
    q, sc = F.quant_rows_fp8(xb)
    w_q2, w_s2 = F.quant_weight_torch(wt)
    out2 = F.grouped_gemm(q, sc, w_q2, w_s2, offs, cnts)
    ref2 = F.grouped_gemm_reference(q, sc, w_q2, w_s2, offs, cnts)
    torch.cuda.synchronize()
    torch.testing.assert_close(out2[:100].float(), ref2[:100], rtol=2e-2, atol=2e-2 * float(ref2.abs().max()))
    mark("gemm_fp32_scales_and_row_quant")

    # ---- weight reshard on four emulated ranks, bf16 (bit-exact) and fp8
    world, tp = 4, 2
    cfg = LlamaConfig(layers=1, hidden=512, heads=4, kv_heads=2, ffn=1024, vocab=1024)
    specs = param_specs(cfg)
    for fp8 in (False, True):
        plans = [ReshardPlan(specs, world, r % tp, tp, fp8=fp8) for r in range(world)]
        p0 = plans[0]
        flat = torch.zeros(p0.shard_elems * world, dtype=torch.bfloat16, device=dev)
        flat[:p0.total_elems] = (torch.randn(p0.total_elems, generator=g, device=dev) * 0.1).to(torch.bfloat16)
        heap = EmulatedHeap(world, p0.shard_elems * 2 + 4096)
        off = heap.alloc(p0.shard_elems * 2)
        for r in range(world):
            heap.tensor(r, off, (p0.shard_elems,), torch.bfloat16).copy_(flat[r * p0.shard_elems:(r + 1) * p0.shard_elems])
        results = emulated_reshard(heap, plans, off)
        for r, (dst, scales, status) in enumerate(results):
            assert status == 0
            refd = reference_reshard(flat, plans[r])
            for e in plans[r].entries:
                nel = e.nrows * e.ncols
                if e.quant:
                    qd = dst[e.dst_off:e.dst_off + nel].view(torch.float8_e4m3fn).view(e.nrows, e.ncols)
                    assert float((qd.float() != refd[e.spec.name][0].float()).float().mean()) < 2e-3
                else:
                    assert torch.equal(dst[e.dst_off:e.dst_off + 2 * nel].view(torch.bfloat16), refd[e.spec.name].reshape(-1))
        mark("reshard_fp8" if fp8 else "reshard_bf16")
    return done
