"""Pure host logic: VA manager (first-fit windows, overlap rules, classification), slice handles, direction table, tag
rules, data-operator selection policy, range-pool allocator, tracer, logger hooks. Counterparts of the reference's logic
tests (test/ut/testcase/hybm/hybm_va_manager_test.cpp, hybm_entity_tag_info_test.cpp,
data_operator/hybm_compose_data_op_test.cpp, utils/*.cpp)."""
import pytest

TiB, GiB, MiB = 1 << 40, 1 << 30, 1 << 20
LH, LD, GH, GD = 0, 1, 2, 3


@pytest.fixture
def va(mf):
    mf.native.va_clear()
    yield mf.native
    mf.native.va_clear()


def test_va_first_fit_and_overlap(va):
    a = va.va_find_free_window(3 * MiB, 0)
    assert a == 32 * TiB
    assert va.va_add_reserved(a, GiB, 1, 1) == 0
    b = va.va_find_free_window(5 * GiB, 0)
    assert b == a + GiB  # windows are 1 GiB aligned and padded
    assert va.va_add_reserved(b, 5 * GiB, 2, 2) == 0
    assert va.va_add_reserved(b + GiB, GiB, 3, 1) != 0  # overlaps the second window
    assert va.va_add_reserved(a - GiB + 1, GiB, 3, 1) != 0  # not granule aligned
    assert va.va_find_free_window(GiB, b) == b + 5 * GiB  # a hint inside a taken window moves past it
    assert va.va_find_free_window(GiB, 40 * TiB) == 40 * TiB
    assert va.va_find_free_window(100 * TiB, 0) == 0  # does not fit the search window
    assert va.va_remove_reserved(a) == 0 and va.va_remove_reserved(a) != 0
    assert va.va_find_free_window(GiB, 0) == a  # the hole is found again


def test_va_allocated_lookup_and_classify(va):
    base = 32 * TiB
    assert va.va_add_allocated(base, 4 * MiB, 1, 0, 7, False) == 0             # local HBM slice of rank 0
    assert va.va_add_allocated(base + 64 * MiB, 4 * MiB, 1, 1, 7, True) == 0   # imported slice of rank 1
    assert va.va_add_allocated(64 * TiB, 2 * MiB, 2, 0, 7, False) == 0         # DRAM slice
    assert va.va_add_allocated(base + MiB, MiB, 1, 0, 7, False) != 0           # overlap
    assert va.va_add_allocated(base + 4 * MiB - 1, 2, 1, 0, 7, False) != 0
    assert va.va_find_allocated(base + 5, 10) == (base, 4 * MiB, 1, 0, 7, False)
    assert va.va_find_allocated(base + 64 * MiB + 4 * MiB - 1, 1)[3] == 1
    assert va.va_find_allocated(base + 4 * MiB - 1, 2) is None  # runs off the end
    assert va.va_find_allocated(base + 8 * MiB, 1) is None and va.va_find_allocated(5, 1) is None
    assert va.va_classify(base + 1) == GD and va.va_classify(64 * TiB) == GH and va.va_classify(12345) == 4
    assert "R" in va.va_info(base + 64 * MiB) and "not in pool" in va.va_info(1)
    assert "allocated(3)" in va.va_dump()
    assert va.va_remove_allocated(base) == 0 and va.va_find_allocated(base, 1) is None


def test_direction_table(mf):
    n = mf.native
    names = {(LH, GH): "LH_TO_GH", (LH, GD): "LH_TO_GD", (LD, GH): "LD_TO_GH", (LD, GD): "LD_TO_GD", (GH, LH): "GH_TO_LH", (GH, LD): "GH_TO_LD",
             (GD, LH): "GD_TO_LH", (GD, LD): "GD_TO_LD", (GH, GH): "GH_TO_GH", (GH, GD): "GH_TO_GD", (GD, GH): "GD_TO_GH", (GD, GD): "GD_TO_GD"}
    for (s, d), name in names.items():
        assert n.va_direction_name(n.va_direction(s, d)) == name
    for s, d in [(LH, LH), (LH, LD), (LD, LH), (LD, LD), (4, GD)]:
        assert n.va_direction_name(n.va_direction(s, d)) == "BUTT"  # local → local is not a pool operation


def test_slice_handles(mf):
    n = mf.native
    h = n.slice_handle(513, 2)
    assert n.slice_decode(h) == (513, 2)
    assert n.slice_decode(h ^ (1 << 40)) is None and n.slice_decode(0) is None and n.slice_decode(h & ~1) is None


def test_tag_rules(mf):
    T = mf.native.TagInfo
    KERNEL, COPY, DRDMA, HRDMA, HTCP = 1, 2, 4, 8, 16
    assert T.valid_tag("prefill_0") and not T.valid_tag("") and not T.valid_tag("a b") and not T.valid_tag("x" * 32)
    assert T.op_type_from_name("DEVICE_SDMA") == COPY and T.op_type_from_name("DEVICE_MTE") == KERNEL
    assert T.op_type_from_name("HOST_TCP") == HTCP and T.op_type_from_name("bogus") == 0
    t = T()
    assert t.init(0, "", "") == 0 and t.allowed_ops(0, 1, 99) == 99  # no rules: everything configured is allowed
    t = T()
    assert t.init(0, "prefill", "prefill:DEVICE_SDMA:decode,prefill:HOST_RDMA:store,prefill:DEVICE_MTE:decode") == 0
    assert t.add_rank_tag(1, "decode") == 0 and t.add_rank_tag(2, "store") == 0 and t.add_rank_tag(3, "other") == 0
    assert t.tag_of(1) == "decode" and t.tag_of(9) == ""
    assert t.allowed_ops(0, 1, 99) == COPY | KERNEL and t.allowed_ops(1, 0, 99) == COPY | KERNEL  # symmetric
    assert t.allowed_ops(0, 2, 99) == HRDMA
    assert t.allowed_ops(0, 3, 99) == 99 and t.allowed_ops(0, 7, 99) == 99  # no rule / unknown rank: fallback
    t.remove_rank_tag(1)
    assert t.allowed_ops(0, 1, 99) == 99
    for bad in ["a:DEVICE_SDMA", "a:NOPE:b", "a b:DEVICE_SDMA:c", "a:DEVICE_SDMA:b:c"]:
        assert T().init(0, "a", bad) != 0, bad
    assert T().init(0, "bad tag", "") != 0 and t.add_rank_tag(4, "no good") != 0


def test_compose_policy_without_gpu(mf):
    n = mf.native
    if n.cuda_available():
        pytest.skip("policy with a GPU is covered by the GPU tier")
    d = {name: i for i, name in enumerate(["LH_TO_GH", "LH_TO_GD", "LD_TO_GH", "LD_TO_GD", "GH_TO_LH", "GH_TO_LD", "GD_TO_LH", "GD_TO_LD", "GH_TO_GH",
                                            "GH_TO_GD", "GD_TO_GH", "GD_TO_GD"])}
    for name in ("LH_TO_GH", "GH_TO_LH", "GH_TO_GH"):
        assert n.compose_candidates(-1, 8, d[name], 4096, False, False, False, 0) == ["cpu_memcpy"]
    # host legs work even if the caller only asked for device engines; device legs have no engine on a CPU-only rank
    assert n.compose_candidates(-1, 3, d["GH_TO_GH"], 4096, True, False, False, 0) == ["cpu_memcpy"]
    assert n.compose_candidates(-1, 3, d["GD_TO_GD"], 4096, False, True, True, 0) == []


def test_range_pool(mf):
    P = mf.native.RangePool
    p = P(1 << 20, 1 << 16, 256)
    a = p.allocate(100)
    b = p.allocate(1000)
    c = p.allocate(300)
    assert (a, b, c) == (1 << 20, (1 << 20) + 256, (1 << 20) + 256 + 1024)
    assert p.in_use() == 256 + 1024 + 512 and p.free_blocks() == 1
    assert p.release(b) and not p.release(b) and not p.release(12345)
    assert p.free_blocks() == 2
    assert p.allocate(1024) == b  # best fit: the hole of exactly that size, not the big tail
    assert p.release(a) and p.release(b) and p.release(c)
    assert p.free_blocks() == 1 and p.largest_free() == 1 << 16 and p.in_use() == 0  # everything coalesced
    assert p.allocate((1 << 16) + 1) == 0 and p.allocate(0) == 0
    full = p.allocate(1 << 16)
    assert full == 1 << 20 and p.allocate(1) == 0 and p.release(full)


def test_tracer_aggregates(mf):
    assert mf.trace_enable() == 0
    mf.trace_dump(reset=True)
    tp = (7 << 8) | 5
    mf.native.trace_point(tp, "TEST_POINT", 0, 2000)
    mf.native.trace_point(tp, "TEST_POINT", 0, 4000)
    mf.native.trace_point(tp, "TEST_POINT", -1, 1000)
    begin, good, bad, total = mf.native.trace_query(tp)
    assert (begin, good, bad) == (3, 2, 1) and total >= 7000
    text = mf.trace_dump()
    assert "TEST_POINT" in text and "TP_NAME" in text
    mf.trace_dump(reset=True)
    assert mf.native.trace_query(tp)[:3] == (0, 0, 0)
    mf.trace_disable()


def test_logger_hook_and_last_error(mf):
    seen = []
    assert mf.set_extern_logger(lambda lv, msg: seen.append((lv, msg))) == 0
    assert mf.set_log_level(9) != 0 and mf.set_log_level(3) == 0
    assert mf.create_config_store("not a url") != 0
    assert any(lv == 3 and "not tcp://" in msg for lv, msg in seen)
    assert "not tcp://" in mf.get_last_err_msg()
    assert "not tcp://" in mf.get_and_clear_last_err_msg() and mf.get_last_err_msg() == ""
    assert mf.set_extern_logger(None) == 0
    assert mf.set_conf_store_tls(False) == 0 and mf.set_conf_store_tls(True, "x") != 0
    assert mf.version().startswith("memfabric-b200")


def test_reference_package_names_resolve():
    """Programs written against the reference import `memfabric_hybrid` (or the transfer-only `mf_adapter`)."""
    import memfabric_hybrid as ref_name
    import memfabric_hybrid_b200 as mf
    import mf_adapter

    for name in ("bm", "shm", "TransferEngine", "TransferOpcode", "create_config_store", "initialize", "uninitialize", "set_log_level",
                 "set_extern_logger", "get_last_err_msg", "set_conf_store_tls", "set_conf_store_tls_key", "get_and_clear_last_err_msg",
                 "get_include_path", "get_lib_path"):
        assert getattr(ref_name, name) is getattr(mf, name), name
    assert mf_adapter.TransferEngine is mf.TransferEngine and mf_adapter.create_config_store is mf.create_config_store
    import os

    assert os.path.isfile(os.path.join(mf.get_include_path(), "mf", "mf_bm.h"))
    assert os.path.isfile(os.path.join(mf.get_lib_path(), "libmf_core.so"))


def test_weight_packing_layout_round_trips():
    """pack_weight_mx: block (nb, kb) of the packed tensor holds rows 32 nb .. 32 nb + 31, K bytes 128 kb .. 128 kb + 127."""
    import torch

    from memfabric_hybrid_b200.ops import fp8_gemm as F

    G, N, K = 2, 96, 384
    w = torch.arange(G * N * K, dtype=torch.int64).remainder(251).to(torch.uint8).view(G, N, K).view(torch.float8_e4m3fn)
    p = F.pack_weight_mx(w)
    assert p.shape == (G, N // 32, K // 128, 32, 128) and p.is_contiguous()
    wb, pb = w.view(torch.uint8), p.view(torch.uint8)
    for g, nb, kb in [(0, 0, 0), (1, 2, 1), (0, 1, 2)]:
        assert torch.equal(pb[g, nb, kb], wb[g, 32 * nb:32 * nb + 32, 128 * kb:128 * kb + 128])
    assert torch.equal(F.unpack_weight_mx(p).view(torch.uint8), wb)
