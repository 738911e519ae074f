"""Device-side argument checks (the stand-in for a device memory checker): with the debug bit set in the heap's meta record, a
kernel whose heap arguments do not lie inside the heap reports MF_DEV_ERR_BOUNDS and touches no peer memory; with valid
arguments the checked run gives the same results as the unchecked one. The bad cases here never reach a peer access — the
check returns first — so nothing can fault."""
import pytest

pytestmark = pytest.mark.gpu

MF_DEV_ERR_BOUNDS = 2


def test_allreduce_rejects_input_outside_the_heap_and_accepts_valid_input():
    import torch

    from memfabric_hybrid_b200._loader import _pymf
    from memfabric_hybrid_b200.ops.allreduce import ALGOS, emulated_allreduce, reference
    from memfabric_hybrid_b200.parallel.heap import EmulatedHeap

    ops = _pymf.ops
    world, T, H = 4, 8, 2048
    heap = EmulatedHeap(world, 2 * T * H * 2 + 8192, check_bounds=True)
    x_off, r_off = heap.alloc(T * H * 2), heap.alloc(T * H * 2)
    g = torch.Generator(device="cuda").manual_seed(3)
    xs = [torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
    res = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16)
    w = torch.ones(H, dtype=torch.bfloat16, device="cuda")
    for r in range(world):
        heap.tensor(r, x_off, (T, H), torch.bfloat16).copy_(xs[r])
    # valid arguments: checked and correct
    for algo in ("oneshot", "twoshot"):
        outs, status = emulated_allreduce(heap, x_off, r_off, [res] * world, w, T, H, 1e-6, algo)
        assert status == [0] * world
        torch.testing.assert_close(outs[0].float(), reference(xs, res, w, 1e-6)[0], atol=2e-2, rtol=2e-2)
    # x given as an ordinary tensor (not heap memory): every rank reports the violation, outputs stay untouched
    stray = [torch.zeros(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    outs = [torch.full((T, H), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    status = torch.zeros(world, dtype=torch.int32, device="cuda")
    for algo in ("oneshot", "twoshot"):
        status.zero_()
        blob = b""
        for r in range(world):
            rk = heap.ranks[r]
            blob += ops.pack_allreduce_args(rk.meta_ptr, stray[r].data_ptr(), res.data_ptr(), w.data_ptr(), rk.addr(r_off), outs[r].data_ptr(),
                                            status.data_ptr() + 4 * r)
        args = torch.frombuffer(bytearray(blob), dtype=torch.uint8).cuda()
        rc = ops.allreduce_rmsnorm(args.data_ptr(), world, world, T, H, 1e-6, ALGOS[algo], 0, heap.next_epoch(0), 0, 0,
                                   torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert status.tolist() == [MF_DEV_ERR_BOUNDS] * world
        assert all(bool((o == 7.0).all()) for o in outs)
    # a size that runs past the end of the rank's window is caught as well
    status.zero_()
    blob = b""
    big_T = heap.size // (H * 2) + 1
    for r in range(world):
        rk = heap.ranks[r]
        blob += ops.pack_allreduce_args(rk.meta_ptr, rk.addr(x_off), 0, w.data_ptr(), rk.addr(r_off), outs[r].data_ptr(), status.data_ptr() + 4 * r)
    args = torch.frombuffer(bytearray(blob), dtype=torch.uint8).cuda()
    assert ops.allreduce_rmsnorm(args.data_ptr(), world, world, big_T, H, 1e-6, ALGOS["oneshot"], 0, heap.next_epoch(0), 0, 0,
                                 torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert status.tolist() == [MF_DEV_ERR_BOUNDS] * world


def test_reshard_and_moe_run_checked():
    """The checked mode is transparent for correct callers: the MoE layer and the reshard give their usual results."""
    import torch

    from memfabric_hybrid_b200.models import LlamaConfig, param_specs
    from memfabric_hybrid_b200.ops import fp8_gemm as F
    from memfabric_hybrid_b200.ops.moe import EmulatedMoE, moe_reference, route
    from memfabric_hybrid_b200.ops.reshard import ReshardPlan, emulated_reshard, reference_reshard
    from memfabric_hybrid_b200.parallel.heap import EmulatedHeap

    g = torch.Generator(device="cuda").manual_seed(9)
    world, T, H, E, K, I = 2, 16, 512, 4, 2, 128
    weights = []
    for _ in range(world):
        wg = torch.randn(E // world, I, H, generator=g, device="cuda") * H ** -0.5
        wu = torch.randn(E // world, I, H, generator=g, device="cuda") * H ** -0.5
        w2 = torch.randn(E // world, H, I, generator=g, device="cuda") * I ** -0.5
        weights.append(F.quant_weight_mx_torch(F.interleave_gate_up(wg, wu)) + F.quant_weight_mx_torch(w2))
    xs = [torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
    routed = [route(torch.randn(T, E, generator=g, device="cuda"), K) for _ in range(world)]
    heap = EmulatedHeap(world, 8 << 20, check_bounds=True)
    layer = EmulatedMoE(heap, T, H, E, K, I, weights, capacity_factor=float(world))
    outs, status = layer(xs, [r[0] for r in routed], [r[1] for r in routed])
    assert status == [0] * world
    refs = moe_reference(xs, [r[0] for r in routed], [r[1] for r in routed], weights, E, I)
    for o, ref in zip(outs, refs):
        assert float((o.float() - ref).abs().max()) <= 1e-1 * (float(ref.abs().max()) + 1e-6)

    cfg = LlamaConfig(layers=1, hidden=512, heads=4, kv_heads=2, ffn=1024, vocab=1024)
    plans = [ReshardPlan(param_specs(cfg), world, r, world) for r in range(world)]
    p0 = plans[0]
    flat = torch.zeros(p0.shard_elems * world, dtype=torch.bfloat16, device="cuda")
    flat[:p0.total_elems] = torch.randn(p0.total_elems, generator=g, device="cuda").to(torch.bfloat16)
    heap2 = EmulatedHeap(world, p0.shard_elems * 2 + 4096, check_bounds=True)
    off = heap2.alloc(p0.shard_elems * 2)
    for r in range(world):
        heap2.tensor(r, off, (p0.shard_elems,), torch.bfloat16).copy_(flat[r * p0.shard_elems:(r + 1) * p0.shard_elems])
    for r, (dst, _, st) in enumerate(emulated_reshard(heap2, plans, off)):
        assert st == 0
        ref = reference_reshard(flat, plans[r])
        e = plans[r].entries[1]
        n = e.nrows * e.ncols
        assert torch.equal(dst[e.dst_off:e.dst_off + 2 * n].view(torch.bfloat16), ref[e.spec.name].reshape(-1))
    # a shard that claims to be longer than the rank's window: caught before the first load
    plans_bad = [ReshardPlan(param_specs(cfg), world, r, world) for r in range(world)]
    for p in plans_bad:
        p.shard_elems = heap2.size  # elements, i.e. twice the window in bytes
    assert all(st == MF_DEV_ERR_BOUNDS for _, _, st in emulated_reshard(heap2, plans_bad, off))
