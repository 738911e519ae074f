"""Reshard kernel (FSDP flat shards → TP layout, optional fp8 cast) against the all-gather + slice + cast oracle."""
import pytest

pytestmark = pytest.mark.gpu


def _setup(world, tp, fp8, seed=3):
    import torch

    from memfabric_hybrid_b200.models import LlamaConfig, param_specs
    from memfabric_hybrid_b200.ops.reshard import ReshardPlan
    from memfabric_hybrid_b200.parallel.heap import EmulatedHeap

    cfg = LlamaConfig(layers=2, hidden=512, heads=4, kv_heads=2, ffn=1024, vocab=1024)
    specs = param_specs(cfg)
    plans = [ReshardPlan(specs, world, r % tp, tp, fp8=fp8) for r in range(world)]
    p0 = plans[0]
    g = torch.Generator(device="cuda").manual_seed(seed)
    flat = torch.zeros(p0.shard_elems * world, dtype=torch.bfloat16, device="cuda")
    flat[:p0.total_elems] = (torch.randn(p0.total_elems, generator=g, device="cuda") * 0.1).to(torch.bfloat16)
    heap = EmulatedHeap(world, p0.shard_elems * 2 + 4096)
    off = heap.alloc(p0.shard_elems * 2)
    for r in range(world):
        heap.tensor(r, off, (p0.shard_elems,), torch.bfloat16).copy_(flat[r * p0.shard_elems:(r + 1) * p0.shard_elems])
    return plans, flat, heap, off


@pytest.mark.parametrize("world,tp", [(8, 4), (2, 2), (4, 1)])
def test_bf16_reshard_is_bit_exact(world, tp):
    import torch

    from memfabric_hybrid_b200.ops.reshard import emulated_reshard, reference_reshard

    plans, flat, heap, off = _setup(world, tp, fp8=False)
    results = emulated_reshard(heap, plans, off)
    for r, (dst, _, status) in enumerate(results):
        assert status == 0
        ref = reference_reshard(flat, plans[r])
        for e in plans[r].entries:
            n = e.nrows * e.ncols
            got = dst[e.dst_off:e.dst_off + 2 * n].view(torch.bfloat16)
            assert torch.equal(got, ref[e.spec.name].reshape(-1)), f"rank {r} {e.spec.name}"


def test_fp8_reshard_matches_block_quantisation():
    import torch

    from memfabric_hybrid_b200.ops.fp8_gemm import dequant_weight
    from memfabric_hybrid_b200.ops.reshard import emulated_reshard, reference_reshard

    plans, flat, heap, off = _setup(8, 4, fp8=True)
    results = emulated_reshard(heap, plans, off)
    for r, (dst, scales, status) in enumerate(results):
        assert status == 0
        ref = reference_reshard(flat, plans[r])
        for e in plans[r].entries:
            n = e.nrows * e.ncols
            if not e.quant:
                assert torch.equal(dst[e.dst_off:e.dst_off + 2 * n].view(torch.bfloat16), ref[e.spec.name].reshape(-1))
                continue
            q = dst[e.dst_off:e.dst_off + n].view(torch.float8_e4m3fn).view(e.nrows, e.ncols)
            sc = scales[e.scale_off:e.scale_off + (e.nrows // 128) * (e.ncols // 128)].view(e.nrows // 128, e.ncols // 128)
            q_ref, sc_ref = ref[e.spec.name]
            torch.testing.assert_close(sc, sc_ref, rtol=1e-6, atol=0)
            assert float((q.float() != q_ref.float()).float().mean()) < 2e-3  # division vs reciprocal rounding
            blk = flat[e.src_off:e.src_off + e.spec.numel].view(*e.spec.shape)[e.r0:e.r0 + e.nrows, e.c0:e.c0 + e.ncols].float()
            err = (dequant_weight(q, sc) - blk).abs().max()
            assert float(err) <= float(sc.max()) * 32 + 1e-6  # within one e4m3 step of the source


def test_missing_rank_times_out_with_status():
    from memfabric_hybrid_b200.ops.reshard import emulated_reshard

    plans, flat, heap, off = _setup(4, 2, fp8=False)
    results = emulated_reshard(heap, plans, off, timeout_ns=50_000_000, participating=3)
    assert all(st & 0xFF == 1 and st >> 8 == 3 for _, _, st in results)


def _real_rank(rank, world, port, q):
    try:
        import torch

        from memfabric_hybrid_b200.models import LlamaConfig, param_specs
        from memfabric_hybrid_b200.ops.fp8_gemm import dequant_weight
        from memfabric_hybrid_b200.ops.reshard import Resharder, ReshardPlan, reference_reshard
        from memfabric_hybrid_b200.parallel.heap import SymmetricHeap

        torch.cuda.set_device(rank)
        tp = 4 if world % 4 == 0 else (2 if world % 2 == 0 else 1)
        cfg = LlamaConfig(layers=2, hidden=1024, heads=8, kv_heads=4, ffn=2048, vocab=4096)
        specs = param_specs(cfg)
        plans = {fp8: ReshardPlan(specs, world, rank % tp, tp, fp8=fp8) for fp8 in (False, True)}
        p = plans[False]
        heap = SymmetricHeap(rank, world, rank, p.shard_elems * 2 + (4 << 20), store_url=f"tcp://127.0.0.1:{port}")
        # the same seeded flat vector on every rank: each writes only its own shard, each can build the oracle
        g = torch.Generator(device="cuda").manual_seed(17)
        flat = torch.zeros(p.shard_elems * world, dtype=torch.bfloat16, device="cuda")
        flat[:p.total_elems] = (torch.randn(p.total_elems, generator=g, device="cuda") * 0.1).to(torch.bfloat16)
        rs = Resharder(heap, plans[False])
        rs8 = Resharder(heap, plans[True], shard=(rs.shard_off, rs.shard))
        rs.shard.copy_(flat[rank * p.shard_elems:(rank + 1) * p.shard_elems])
        torch.cuda.synchronize()
        heap.barrier()
        for it in range(2):
            views = rs()
            views8 = rs8()
            torch.cuda.synchronize()
            assert rs.check_status() == 0 and rs8.check_status() == 0
            ref, ref8 = reference_reshard(flat, plans[False]), reference_reshard(flat, plans[True])
            for e in plans[False].entries:
                assert torch.equal(views[e.spec.name].reshape(-1), ref[e.spec.name].reshape(-1)), f"rank {rank} {e.spec.name}"
            for e in plans[True].entries:
                if not e.quant:
                    assert torch.equal(views8[e.spec.name].reshape(-1), ref8[e.spec.name].reshape(-1))
                    continue
                qd, sc = views8[e.spec.name]
                q_ref, sc_ref = ref8[e.spec.name]
                torch.testing.assert_close(sc, sc_ref, rtol=1e-6, atol=0)
                assert float((qd.float() != q_ref.float()).float().mean()) < 2e-3
                assert float((dequant_weight(qd, sc) - dequant_weight(q_ref, sc_ref)).abs().max()) <= float(sc.max()) * 32 + 1e-6
            heap.barrier()
        heap.close()
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        import traceback

        traceback.print_exc()
        q.put((rank, repr(e)))


def test_real_ranks_one_per_gpu():
    import multiprocessing as mp

    import torch

    from conftest import free_port

    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    ps = [ctx.Process(target=_real_rank, args=(r, world, port, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = sorted(q.get(timeout=300) for _ in ps)
    for p in ps:
        p.join(timeout=60)
    assert res == [(r, "ok") for r in range(world)], res
