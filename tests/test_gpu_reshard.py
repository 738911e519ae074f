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
