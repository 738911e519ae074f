"""GPU tests of the xcopy data plane: every direction, odd sizes and alignments, batch copy (inline and table paths),
two ranks mapping each other's HBM and DRAM. Oracle: the bytes themselves (numpy on the CPU). Model: the reference's
direction-matrix test (test/python/hybm/data_op_all_path_test.py:32-110) and BmCpp's H2G→G2G→G2H check
(example/bm/BmCpp/main.cpp:142-201)."""
import multiprocessing as mp

import numpy as np
import pytest

from conftest import free_port

pytestmark = pytest.mark.gpu

MiB = 1 << 20


@pytest.fixture(scope="module")
def pool():
    import torch

    from memfabric_hybrid_b200.parallel.pool import open_pool

    torch.cuda.set_device(0)
    p = open_pool(0, 1, 0, 96 * MiB, dram_bytes=32 * MiB, store_url=f"tcp://127.0.0.1:{free_port()}")
    yield p
    p.close()


def _rand(n, seed):
    return np.random.default_rng(seed).integers(0, 256, n, dtype=np.uint8)


def test_native_module_is_loaded(mf):
    import sys

    assert mf.native.cuda_available()
    assert any("_pymf" in (getattr(m, "__file__", "") or "") for m in sys.modules.values())
    caps = mf.native.device_caps(0)
    assert caps["vmm"] and caps["posix_fd"]


@pytest.mark.parametrize("n", [1, 15, 16, 17, 255, 4096, 4097, 65535, 65536, 1 * MiB + 3, 2 * MiB + 1, 5 * MiB])
@pytest.mark.parametrize("soff,doff", [(0, 0), (1, 1), (3, 7), (8, 0), (4, 12), (2, 9)])
def test_g2g_alignments(mf, pool, n, soff, doff):
    import torch

    from memfabric_hybrid_b200.utils.tensors import device_tensor_from_gva

    base = pool.hbm()
    src_region = device_tensor_from_gva(base, 8 * MiB)
    dst_region = device_tensor_from_gva(base + 16 * MiB, 8 * MiB)
    data = torch.from_numpy(_rand(n, n + soff)).cuda()
    src_region[soff:soff + n] = data
    dst_region.fill_(0xA5)
    torch.cuda.synchronize()
    rc = pool.handle.copy_data(base + soff, base + 16 * MiB + 64 + doff, n, mf.bm.BmCopyType.G2G, 0)
    assert rc == 0, mf.get_last_err_msg()
    got = dst_region.cpu().numpy()
    lo = 64 + doff
    assert (got[lo:lo + n] == data.cpu().numpy()).all()
    # canaries on both sides of the destination stay untouched
    assert (got[:lo] == 0xA5).all() and (got[lo + n:lo + n + 256] == 0xA5).all()


def test_all_directions_roundtrip(mf, pool):
    """LH/LD/GH/GD sources into GH/GD and back out: the 12 directions of the pool."""
    import torch

    T = mf.bm.BmCopyType
    n = 3 * MiB + 11
    gd, gh = pool.hbm() + 32 * MiB, pool.dram()
    ref = _rand(n, 7)
    lh_page = ref.copy()                                   # pageable host
    lh_pin = torch.from_numpy(ref.copy()).pin_memory()     # pinned host
    ld = torch.from_numpy(ref).cuda()                      # local device
    h = pool.handle

    def back_gd(addr):
        out = np.zeros(n, dtype=np.uint8)
        assert h.copy_data(addr, out.ctypes.data, n, T.G2H, 0) == 0, mf.get_last_err_msg()
        return out

    def back_gh(addr):
        out = np.zeros(n, dtype=np.uint8)
        assert h.copy_data(addr, out.ctypes.data, n, T.GH2H, 0) == 0, mf.get_last_err_msg()
        return out

    # LH → GD (pageable and pinned), LD → GD
    assert h.copy_data(lh_page.ctypes.data, gd + 1, n, T.H2G, 0) == 0, mf.get_last_err_msg()
    assert (back_gd(gd + 1) == ref).all()
    assert h.copy_data(lh_pin.data_ptr(), gd + 5, n, T.H2G, 0) == 0, mf.get_last_err_msg()
    assert (back_gd(gd + 5) == ref).all()
    assert h.copy_data(ld.data_ptr(), gd + 9, n, T.L2G, 0) == 0, mf.get_last_err_msg()
    assert (back_gd(gd + 9) == ref).all()
    # LH → GH, LD → GH
    assert h.copy_data(lh_page.ctypes.data, gh + 3, n, T.H2GH, 0) == 0, mf.get_last_err_msg()
    assert (back_gh(gh + 3) == ref).all()
    assert h.copy_data(ld.data_ptr(), gh + 8 * MiB, n, T.L2GH, 0) == 0, mf.get_last_err_msg()
    assert (back_gh(gh + 8 * MiB) == ref).all()
    # GD → GH, GH → GD, GH → GH, GD → GD (G2G decides by where the pointers live)
    assert h.copy_data(gd + 9, gh + 16 * MiB, n, T.G2G, 0) == 0, mf.get_last_err_msg()
    assert (back_gh(gh + 16 * MiB) == ref).all()
    assert h.copy_data(gh + 16 * MiB, gd + 8 * MiB, n, T.G2G, 0) == 0, mf.get_last_err_msg()
    assert (back_gd(gd + 8 * MiB) == ref).all()
    assert h.copy_data(gh + 3, gh + 24 * MiB, n, T.G2G, 0) == 0, mf.get_last_err_msg()
    assert (back_gh(gh + 24 * MiB) == ref).all()
    # GD → LD, GH → LD, and AUTO classification
    out_ld = torch.zeros(n, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    assert h.copy_data(gd + 8 * MiB, out_ld.data_ptr(), n, T.G2L, 0) == 0, mf.get_last_err_msg()
    assert (out_ld.cpu().numpy() == ref).all()
    out_ld.zero_()
    torch.cuda.synchronize()  # the pool's synchronous copies run on the library's own stream, not on torch's
    assert h.copy_data(gh + 24 * MiB, out_ld.data_ptr(), n, T.GH2L, 0) == 0, mf.get_last_err_msg()
    assert (out_ld.cpu().numpy() == ref).all()
    out_ld.zero_()
    torch.cuda.synchronize()  # the pool's synchronous copies run on the library's own stream, not on torch's
    assert h.copy_data(gd + 8 * MiB, out_ld.data_ptr(), n, T.AUTO, 0) == 0, mf.get_last_err_msg()
    assert (out_ld.cpu().numpy() == ref).all()
    # local → local is not a pool operation
    assert h.copy_data(ld.data_ptr(), out_ld.data_ptr(), n, T.AUTO, 0) != 0
    # a range that leaves the pool is refused
    assert h.copy_data(ld.data_ptr(), pool.hbm() + pool.hbm_bytes - 16, 4096, T.L2G, 0) != 0


def test_batch_with_mixed_local_sides_is_split_by_placement(mf, pool):
    """One batch whose local sides are pageable host, pinned host, device and pooled memory: every element is placed on its
    own; the pageable ones go to the copy engine as their own group and the kernel engine never sees them (checked on the
    engine counters, not by provoking a fault), and every byte arrives."""
    import torch

    T = mf.bm.BmCopyType
    blk = 64 * 1024
    gd = pool.hbm() + 8 * MiB
    pageable = _rand(4 * blk, 1)
    pinned = torch.from_numpy(_rand(4 * blk, 2)).pin_memory()
    device = torch.from_numpy(_rand(4 * blk, 3)).cuda()
    pooled = pool.hbm() + 64 * MiB
    pooled_ref = _rand(4 * blk, 4)
    assert pool.handle.copy_data(pooled_ref.ctypes.data, pooled, 4 * blk, T.H2G, 0) == 0
    torch.cuda.synchronize()
    srcs, expect = [], []
    for i in range(4):  # interleaved on purpose: element 0 is pinned (device-visible), pageable elements come later
        srcs += [pinned.data_ptr() + i * blk, pageable.ctypes.data + i * blk, device.data_ptr() + i * blk, pooled + i * blk]
        expect += [pinned.numpy()[i * blk:(i + 1) * blk], pageable[i * blk:(i + 1) * blk], device.cpu().numpy()[i * blk:(i + 1) * blk],
                   pooled_ref[i * blk:(i + 1) * blk]]
    dsts = [gd + i * blk for i in range(16)]
    before = mf.native.data_op_stats()
    assert pool.handle.copy_data_batch(srcs, dsts, [blk] * 16, 16, T.AUTO, 0) == 0, mf.get_last_err_msg()
    after = mf.native.data_op_stats()
    assert after["batch_groups_last"] >= 2
    assert after["copy_engine_elems"] - before["copy_engine_elems"] == 4   # exactly the four pageable elements
    assert after["kernel_elems"] - before["kernel_elems"] == 12
    out = np.zeros(16 * blk, dtype=np.uint8)
    assert pool.handle.copy_data(gd, out.ctypes.data, 16 * blk, T.G2H, 0) == 0
    for i in range(16):
        assert (out[i * blk:(i + 1) * blk] == expect[i]).all(), f"element {i}"
    # the other way round: pooled sources into pageable, pinned and device destinations
    out_page = np.zeros(2 * blk, dtype=np.uint8)
    out_pin = torch.zeros(2 * blk, dtype=torch.uint8).pin_memory()
    out_dev = torch.zeros(2 * blk, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    dsts2 = [out_pin.data_ptr(), out_page.ctypes.data, out_dev.data_ptr(), out_page.ctypes.data + blk, out_pin.data_ptr() + blk, out_dev.data_ptr() + blk]
    srcs2 = [gd + i * blk for i in range(6)]
    before = mf.native.data_op_stats()
    assert pool.handle.copy_data_batch(srcs2, dsts2, [blk] * 6, 6, T.AUTO, 0) == 0, mf.get_last_err_msg()
    after = mf.native.data_op_stats()
    assert after["copy_engine_elems"] - before["copy_engine_elems"] == 2
    assert (out_pin.numpy()[:blk] == expect[0]).all() and (out_page[:blk] == expect[1]).all() and (out_dev.cpu().numpy()[:blk] == expect[2]).all()
    assert (out_page[blk:] == expect[3]).all() and (out_pin.numpy()[blk:] == expect[4]).all() and (out_dev.cpu().numpy()[blk:] == expect[5]).all()


@pytest.mark.parametrize("count", [1, 7, 122, 168, 169, 1000])
def test_batch_copy(mf, pool, count):
    import torch

    from memfabric_hybrid_b200.utils.tensors import device_tensor_from_gva

    rng = np.random.default_rng(count)
    base = pool.hbm()
    region = 40 * MiB
    src_t = device_tensor_from_gva(base, region)
    dst_t = device_tensor_from_gva(base + 48 * MiB, region)
    src_t.copy_(torch.from_numpy(_rand(region, 99 + count)).cuda())
    dst_t.zero_()
    torch.cuda.synchronize()
    src_np = src_t.cpu().numpy()
    slot = region // count // 64 * 64
    sizes = [int(rng.integers(1, min(slot - 64, 200_000))) for _ in range(count)]
    if count >= 7 and slot > 140_000:
        sizes[3] = 131072
        sizes[5] = 16384
    soffs = [i * slot + int(rng.integers(0, 16)) for i in range(count)]
    doffs = [i * slot + int(rng.integers(0, 16)) for i in range(count)]
    rc = pool.handle.copy_data_batch([base + o for o in soffs], [base + 48 * MiB + o for o in doffs], sizes, count, mf.bm.BmCopyType.G2G, 0)
    assert rc == 0, mf.get_last_err_msg()
    got = dst_t.cpu().numpy()
    expect = np.zeros(region, dtype=np.uint8)
    for s, d, n in zip(soffs, doffs, sizes):
        expect[d:d + n] = src_np[s:s + n]
    assert (got == expect).all()


def test_batch_coalesces_adjacent_runs(mf, pool):
    """Adjacent blocks on both sides are merged into one run; the result is the same bytes."""
    import torch

    from memfabric_hybrid_b200.utils.tensors import device_tensor_from_gva

    base = pool.hbm()
    n, blocks = 16384, 64
    src_t = device_tensor_from_gva(base, n * blocks)
    src_t.copy_(torch.from_numpy(_rand(n * blocks, 5)).cuda())
    srcs = [base + i * n for i in range(blocks)]
    dsts = [base + 48 * MiB + i * n for i in range(blocks)]
    assert pool.handle.copy_data_batch(srcs, dsts, [n] * blocks, blocks, mf.bm.BmCopyType.G2G, 0) == 0
    assert torch.equal(device_tensor_from_gva(base + 48 * MiB, n * blocks), src_t)


def test_async_copy_and_wait(mf, pool):
    import torch

    from memfabric_hybrid_b200.utils.tensors import device_tensor_from_gva

    base = pool.hbm()
    n = 8 * MiB
    src_t = device_tensor_from_gva(base, n)
    src_t.copy_(torch.from_numpy(_rand(n, 17)).cuda())
    torch.cuda.synchronize()
    for i in range(4):
        assert pool.handle.copy_data(base, base + (16 + 8 * i) * MiB, n, mf.bm.BmCopyType.G2G, 1) == 0  # ASYNC
    assert pool.handle.wait() == 0
    for i in range(4):
        assert torch.equal(device_tensor_from_gva(base + (16 + 8 * i) * MiB, n), src_t)
    # user stream variant
    s = torch.cuda.Stream()
    assert pool.handle.copy_data_on_stream(base, base + 56 * MiB, n, mf.bm.BmCopyType.G2G, s.cuda_stream, 0) == 0
    s.synchronize()
    assert torch.equal(device_tensor_from_gva(base + 56 * MiB, n), src_t)


def test_pattern_and_checksum_kernels(mf):
    import torch

    n = 1 * MiB + 5
    buf = torch.empty(n, dtype=torch.uint8, device="cuda")
    out = torch.zeros(2, dtype=torch.int64, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert mf.native.fill_pattern(buf.data_ptr(), n, 42, s) == 0
    assert mf.native.check_pattern(buf.data_ptr(), n, 42, out.data_ptr(), s) == 0
    assert mf.native.checksum(buf.data_ptr(), n, out.data_ptr() + 8, s) == 0
    torch.cuda.synchronize()
    host = buf.cpu().numpy().tobytes()
    assert host[:64] == mf.native.pattern_bytes(42, 0, 64)
    assert int(out[0]) == 0
    assert (int(out[1]) & (2**64 - 1)) == mf.native.checksum_host(host)
    buf[1000] ^= 1
    assert mf.native.check_pattern(buf.data_ptr(), n, 42, out.data_ptr(), s) == 0
    torch.cuda.synchronize()
    assert int(out[0]) == 1


def test_rank_queries(mf, pool):
    h = pool.handle
    assert h.get_rank_id_by_gva(pool.hbm() + 123) == 0
    assert h.get_rank_id_by_gva(pool.dram() + 5) == 0
    assert h.local_mem_size(mf.bm.BmMemType.DEVICE) == pool.hbm_bytes
    assert h.local_mem_size(mf.bm.BmMemType.HOST) == pool.dram_bytes
    assert h.joined_size() == 1


def _two_rank_worker(rank, port, bar, q):
    try:
        import torch

        import memfabric_hybrid_b200 as mf
        from memfabric_hybrid_b200.parallel.pool import open_pool
        from memfabric_hybrid_b200.utils.tensors import device_tensor_from_gva

        torch.cuda.set_device(0)  # both ranks share GPU 0: peer HBM is then another process's memory on the same device
        pool = open_pool(rank, 2, 0, 32 * MiB, dram_bytes=8 * MiB, store_url=f"tcp://127.0.0.1:{port}")
        bar.wait(timeout=120)
        T = mf.bm.BmCopyType
        n = 5 * MiB + 3
        peer = 1 - rank
        mine = torch.from_numpy(np.random.default_rng(100 + rank).integers(0, 256, n, dtype=np.uint8)).cuda()
        # push my data into the peer's HBM window and into the peer's DRAM window
        assert pool.handle.copy_data(mine.data_ptr(), pool.hbm(peer) + 16 * MiB + 1, n, T.L2G, 0) == 0, mf.get_last_err_msg()
        assert pool.handle.copy_data(mine.data_ptr(), pool.dram(peer) + 64, n, T.L2GH, 0) == 0, mf.get_last_err_msg()
        bar.wait(timeout=120)
        expect = np.random.default_rng(100 + peer).integers(0, 256, n, dtype=np.uint8)
        got = device_tensor_from_gva(pool.hbm(rank) + 16 * MiB + 1, n).cpu().numpy()
        assert (got == expect).all(), "peer HBM push mismatch"
        out = np.zeros(n, dtype=np.uint8)
        assert pool.handle.copy_data(pool.dram(rank) + 64, out.ctypes.data, n, T.GH2H, 0) == 0
        assert (out == expect).all(), "peer DRAM push mismatch"
        # pull from the peer (remote read) and a batch of KV-like blocks
        pulled = torch.zeros(n, dtype=torch.uint8, device="cuda")
        assert pool.handle.copy_data(pool.hbm(peer) + 16 * MiB + 1, pulled.data_ptr(), n, T.G2L, 0) == 0
        assert (pulled.cpu().numpy() == np.random.default_rng(100 + rank).integers(0, 256, n, dtype=np.uint8)).all()
        assert pool.handle.get_rank_id_by_gva(pool.hbm(peer) + 5) == peer
        bar.wait(timeout=120)
        pool.close()
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover - reported to the parent
        import traceback

        traceback.print_exc()
        q.put((rank, repr(e)))


def test_two_ranks_map_each_other(mf):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    bar = ctx.Barrier(2)
    port = free_port()
    ps = [ctx.Process(target=_two_rank_worker, args=(r, port, bar, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = sorted(q.get(timeout=240) for _ in ps)
    for p in ps:
        p.join(timeout=60)
    assert res == [(0, "ok"), (1, "ok")], res
