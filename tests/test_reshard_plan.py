"""Reshard planning is pure host logic: shapes, offsets and coverage for the Llama-3-8B inventory (no GPU)."""
from memfabric_hybrid_b200.models import LLAMA3_8B, param_specs, tp_block


def test_llama3_8b_inventory():
    specs = param_specs(LLAMA3_8B)
    assert len(specs) == 1 + 32 * 9 + 2
    total = sum(s.numel for s in specs)
    assert 8.0e9 < total < 8.1e9  # 8.03 B parameters
    by = {s.name: s for s in specs}
    assert by["layers.0.k_proj"].shape == (1024, 4096) and by["layers.31.down_proj"].shape == (4096, 14336)


def test_tp_blocks_tile_every_parameter():
    for s in param_specs(LLAMA3_8B):
        if len(s.shape) == 1:
            assert tp_block(s, 3, 4) == (0, 0, 1, s.shape[0], s.shape[0])
            continue
        covered = 0
        for r in range(4):
            r0, c0, nr, nc, cf = tp_block(s, r, 4)
            assert cf == s.shape[1] and r0 + nr <= s.shape[0] and c0 + nc <= s.shape[1]
            covered += nr * nc
        assert covered == s.numel  # the four shards partition the matrix


def test_plan_offsets_and_sizes():
    from memfabric_hybrid_b200.ops.reshard import ReshardPlan

    specs = param_specs(LLAMA3_8B)
    bf = ReshardPlan(specs, 8, 1, 4, fp8=False)
    f8 = ReshardPlan(specs, 8, 1, 4, fp8=True)
    assert bf.shard_elems * 8 >= bf.total_elems and bf.shard_elems % 8 == 0
    assert bf.total_tiles == f8.total_tiles
    # bf16 destination: a quarter of the linears + all norms + a quarter of embed/head
    assert abs(bf.dst_bytes - bf.bytes_pulled()) < 1 << 20
    assert f8.dst_bytes < bf.dst_bytes * 0.65  # linears shrink to one byte per element
    q = [e for e in f8.entries if e.quant]
    assert len(q) == 32 * 7 and all(e.nrows % 128 == 0 and e.ncols % 128 == 0 for e in q)
    assert f8.scale_floats == sum((e.nrows // 128) * (e.ncols // 128) for e in q)
    # entries do not overlap in the destination
    spans = sorted((e.dst_off, e.dst_off + e.nrows * e.ncols * (1 if e.quant else 2)) for e in f8.entries)
    assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))
    assert len(f8.table_bytes()) == len(f8.entries) * 56
