"""Big Memory on CPU-only ranks: two (and three) processes on one host joined through the TCP config store, each contributing
DRAM to one GVA range. LH→GH / GH→LH over sizes 4 KiB – 32 MiB, one batch of 64 discrete 16 KiB blocks at random aligned
offsets, GH→GH, auto-ranking, dynamic join/leave, a rank that dies. Verification by byte compare. Pattern: the reference's
fork-based multi-rank tests (test/ut/testcase/smem/smem_bm_test.cpp:209-416)."""
import multiprocessing as mp
import os
import time

import numpy as np
import pytest

from conftest import free_port

MiB = 1 << 20
POOL = 64 * MiB


def _open(mf, rank, world, port, auto=False, pool=POOL):
    cfg = mf.bm.BmConfig()
    cfg.auto_ranking = auto
    if not auto:
        cfg.rank_id = rank
    cfg.init_timeout = cfg.create_timeout = cfg.operation_timeout = 30
    rc = mf.bm.initialize(f"tcp://127.0.0.1:{port}", world, -1, cfg)
    assert rc == 0, (rc, mf.get_last_err_msg())
    b = mf.bm.create(0, pool, 0, mf.bm.BmDataOpType.HOST_RDMA)
    assert b.join() == 0, mf.get_last_err_msg()
    return b


def _seeded(n, seed):
    return np.random.default_rng(seed).integers(0, 256, n, dtype=np.uint8)


def _pair_worker(rank, port, bar, q):
    try:
        import memfabric_hybrid_b200 as mf

        b = _open(mf, rank, 2, port)
        T = mf.bm.BmCopyType
        H = mf.bm.BmMemType.HOST
        peer = 1 - rank
        bar.wait(60)
        assert b.joined_size() == 2
        assert b.peer_rank_ptr(H, 1) - b.peer_rank_ptr(H, 0) == POOL  # linear layout: base + rank * maxSize
        assert b.get_rank_id_by_gva(b.peer_rank_ptr(H, peer) + 5) == peer
        # sizes 4 KiB .. 32 MiB: write into the peer's window (LH→GH), peer reads its own window back (GH→LH)
        sizes = [1 << k for k in range(12, 26)]
        for i, n in enumerate(sizes):
            data = _seeded(n, 1000 * rank + i)
            assert b.copy_data(data.ctypes.data, b.peer_rank_ptr(H, peer), n, T.H2GH, 0) == 0, mf.get_last_err_msg()
            bar.wait(60)
            out = np.zeros(n, dtype=np.uint8)
            assert b.copy_data(b.peer_rank_ptr(H, rank), out.ctypes.data, n, T.GH2H, 0) == 0, mf.get_last_err_msg()
            assert (out == _seeded(n, 1000 * peer + i)).all(), f"size {n}"
            bar.wait(60)
        # one batch of 64 discrete 16 KiB blocks at random 4 KiB-aligned offsets
        rng = np.random.default_rng(77 + rank)
        slots = rng.choice(POOL // (16 << 10), size=64, replace=False)
        offs = [int(s) * (16 << 10) for s in slots]
        blocks = _seeded(64 * (16 << 10), 5 + rank)
        srcs = [blocks.ctypes.data + i * (16 << 10) for i in range(64)]
        dsts = [b.peer_rank_ptr(H, peer) + o for o in offs]
        assert b.copy_data_batch(srcs, dsts, [16 << 10] * 64, 64, T.H2GH, 0) == 0, mf.get_last_err_msg()
        bar.wait(60)
        peer_offs = [int(s) * (16 << 10) for s in np.random.default_rng(77 + peer).choice(POOL // (16 << 10), size=64, replace=False)]
        peer_blocks = _seeded(64 * (16 << 10), 5 + peer)
        mine = mf.native.host_read(b.peer_rank_ptr(H, rank), POOL)
        for i, o in enumerate(peer_offs):
            assert mine[o:o + (16 << 10)] == peer_blocks[i * (16 << 10):(i + 1) * (16 << 10)].tobytes(), f"block {i}"
        bar.wait(60)
        # one batch whose elements land on BOTH ranks' windows: every element is placed on its own and the batch is served as
        # one group per (source rank, destination rank)
        mix = _seeded(8 * 4096, 900 + rank)
        msrcs = [mix.ctypes.data + i * 4096 for i in range(8)]
        mdsts = [b.peer_rank_ptr(H, (rank + i) % 2) + 48 * MiB + (rank * 8 + i) * 4096 for i in range(8)]
        assert b.copy_data_batch(msrcs, mdsts, [4096] * 8, 8, T.H2GH, 0) == 0, mf.get_last_err_msg()
        assert mf.native.data_op_stats()["batch_groups_last"] == 2
        bar.wait(60)
        got = mf.native.host_read(b.peer_rank_ptr(H, rank) + 48 * MiB, 16 * 4096)
        for r in range(2):
            theirs = _seeded(8 * 4096, 900 + r)
            for i in range(8):
                if (r + i) % 2 == rank:
                    o = (r * 8 + i) * 4096
                    assert got[o:o + 4096] == theirs[i * 4096:(i + 1) * 4096].tobytes(), (r, i)
        # an element that leaves the pool fails the whole batch before anything is moved
        bad = list(mdsts)
        bad[5] = b.peer_rank_ptr(H, 1) + POOL - 8
        assert b.copy_data_batch(msrcs, bad, [4096] * 8, 8, T.H2GH, 0) != 0
        bar.wait(60)
        # GH → GH between the two windows, AUTO direction, and refusals
        assert b.copy_data(b.peer_rank_ptr(H, rank), b.peer_rank_ptr(H, peer) + 32 * MiB, 4096, T.G2G, 0) == 0
        assert b.copy_data(b.peer_rank_ptr(H, rank) + 8, b.peer_rank_ptr(H, rank) + 40 * MiB, 100, T.AUTO, 0) == 0
        tmp = np.zeros(16, dtype=np.uint8)
        assert b.copy_data(tmp.ctypes.data, tmp.ctypes.data, 16, T.AUTO, 0) != 0  # local → local
        assert b.copy_data(tmp.ctypes.data, b.peer_rank_ptr(H, 1) + POOL - 8, 16, T.H2GH, 0) != 0  # leaves the pool
        assert b.copy_data(0, b.peer_rank_ptr(H, 0), 16, T.H2GH, 0) != 0
        assert b.wait() == 0
        bar.wait(60)
        b.destroy()
        mf.bm.uninitialize()
        q.put((rank, "ok"))
    except Exception as ex:  # pragma: no cover
        import traceback

        traceback.print_exc()
        q.put((rank, repr(ex)))


def _spawn(target, n, extra=()):
    ctx = mp.get_context("spawn")
    q, bar, port = ctx.Queue(), ctx.Barrier(n), free_port()
    ps = [ctx.Process(target=target, args=(r, port, bar, q) + tuple(extra)) for r in range(n)]
    [p.start() for p in ps]
    return ps, q, bar  # the barrier must outlive the children's start-up


def test_two_cpu_ranks_all_sizes_and_batch():
    ps, q, _bar = _spawn(_pair_worker, 2)
    res = sorted(q.get(timeout=300) for _ in ps)
    [p.join(30) for p in ps]
    assert res == [(0, "ok"), (1, "ok")], res


def _large_copy_worker(rank, port, bar, q):
    try:
        import threading

        import memfabric_hybrid_b200 as mf

        b = _open(mf, rank, 1, port)
        T, H = mf.bm.BmCopyType, mf.bm.BmMemType.HOST
        g = b.peer_rank_ptr(H, 0)
        # sizes around the piece and threshold boundaries of the pooled copy (2 MiB threshold, 512 KiB pieces)
        for i, n in enumerate([2 * MiB - 1, 2 * MiB, 2 * MiB + 1, 5 * MiB + 123, 16 * MiB + 4097]):
            data = _seeded(n, 50 + i)
            assert b.copy_data(data.ctypes.data, g + 64, n, T.H2GH, 0) == 0, mf.get_last_err_msg()
            out = np.zeros(n, dtype=np.uint8)
            assert b.copy_data(g + 64, out.ctypes.data, n, T.GH2H, 0) == 0
            assert (out == data).all(), f"size {n}"
        # a batch that is spread over the helper threads: 12 elements of different sizes, 6 MiB in all
        sizes = [(256 + 64 * k) << 10 for k in range(12)]
        blocks = [_seeded(n, 70 + k) for k, n in enumerate(sizes)]
        offs = np.cumsum([0] + sizes[:-1]).tolist()
        assert b.copy_data_batch([x.ctypes.data for x in blocks], [g + int(o) for o in offs], sizes, len(sizes), T.H2GH, 0) == 0
        mine = mf.native.host_read(g, int(offs[-1]) + sizes[-1])
        for k, n in enumerate(sizes):
            assert bytes(mine[int(offs[k]):int(offs[k]) + n]) == blocks[k].tobytes(), f"batch element {k}"
        # two threads copy at once: one gets the helpers, the other copies on its own thread; both must be exact
        srcs = [_seeded(8 * MiB, 90 + t) for t in range(2)]
        errs = []

        def run(t):
            for _ in range(5):
                if b.copy_data(srcs[t].ctypes.data, g + t * 16 * MiB, 8 * MiB, T.H2GH, 0) != 0:
                    errs.append(t)

        ths = [threading.Thread(target=run, args=(t,)) for t in range(2)]
        [t.start() for t in ths]
        [t.join() for t in ths]
        assert not errs
        for t in range(2):
            assert bytes(mf.native.host_read(g + t * 16 * MiB, 8 * MiB)) == srcs[t].tobytes()
        q.put((rank, "ok"))
    except Exception as ex:  # pragma: no cover
        import traceback

        traceback.print_exc()
        q.put((rank, repr(ex)))


def _fork_after_pool_worker(rank, port, bar, q):
    try:
        import warnings

        import memfabric_hybrid_b200 as mf

        b = _open(mf, rank, 1, port)
        T, H = mf.bm.BmCopyType, mf.bm.BmMemType.HOST
        g = b.peer_rank_ptr(H, 0)
        src = _seeded(8 * MiB, 5)
        assert b.copy_data(src.ctypes.data, g, 8 * MiB, T.H2GH, 0) == 0  # the helper threads exist from here on
        warnings.simplefilter("ignore", DeprecationWarning)
        pid = os.fork()
        if pid == 0:  # the child has no helper threads: it must copy on its own thread, not wait for them
            out = np.zeros(8 * MiB, dtype=np.uint8)
            rc = b.copy_data(g, out.ctypes.data, 8 * MiB, T.GH2H, 0)
            os._exit(0 if rc == 0 and (out == src).all() else 3)
        deadline = time.time() + 30
        status = None
        while time.time() < deadline:
            r, st = os.waitpid(pid, os.WNOHANG)
            if r == pid:
                status = os.WEXITSTATUS(st) if os.WIFEXITED(st) else -1
                break
            time.sleep(0.05)
        if status is None:
            os.kill(pid, 9)
            os.waitpid(pid, 0)
        assert status == 0, f"forked child: {status}"
        q.put((rank, "ok"))
    except Exception as ex:  # pragma: no cover
        import traceback

        traceback.print_exc()
        q.put((rank, repr(ex)))


def test_forked_child_copies_without_the_helper_threads():
    ps, q, _bar = _spawn(_fork_after_pool_worker, 1)
    res = [q.get(timeout=120) for _ in ps]
    [p.join(30) for p in ps]
    assert res == [(0, "ok")], res


def test_large_host_copies_through_the_helper_threads():
    ps, q, _bar = _spawn(_large_copy_worker, 1)
    res = [q.get(timeout=300) for _ in ps]
    [p.join(30) for p in ps]
    assert res == [(0, "ok")], res


def _churn_worker(rank, port, bar, q):
    try:
        import memfabric_hybrid_b200 as mf

        H = mf.bm.BmMemType.HOST
        T = mf.bm.BmCopyType
        if rank == 2:
            bar.wait(60)  # ranks 0 and 1 form the pool first
        b = _open(mf, rank, 3, port, pool=8 * MiB)
        if rank != 2:
            bar.wait(60)
        # wait until all three are in
        deadline = time.time() + 30
        while b.joined_size() != 3 and time.time() < deadline:
            time.sleep(0.02)
        assert b.joined_size() == 3
        bar.wait(60)
        # everybody writes its rank into everybody's window
        word = np.full(64, rank, dtype=np.uint8)
        for r in range(3):
            assert b.copy_data(word.ctypes.data, b.peer_rank_ptr(H, r) + 64 * rank, 64, T.H2GH, 0) == 0, mf.get_last_err_msg()
        bar.wait(60)
        mine = mf.native.host_read(b.peer_rank_ptr(H, rank), 192)
        assert mine == bytes([0] * 64 + [1] * 64 + [2] * 64)
        bar.wait(60)
        if rank == 1:
            assert b.leave() == 0
            q.put((rank, "ok"))
            bar.wait(60)
            b.destroy()
            mf.bm.uninitialize()
            return
        deadline = time.time() + 30
        while b.joined_size() != 2 and time.time() < deadline:
            time.sleep(0.02)
        assert b.joined_size() == 2
        # the leaver's window is unmapped here: a copy into it is refused, the others still work
        other = 2 - rank
        assert b.copy_data(word.ctypes.data, b.peer_rank_ptr(H, other) + 512, 64, T.H2GH, 0) == 0
        q.put((rank, "ok"))
        bar.wait(60)
        time.sleep(0.2 if rank == 0 else 0)
        b.destroy()
        mf.bm.uninitialize()
    except Exception as ex:  # pragma: no cover
        import traceback

        traceback.print_exc()
        q.put((rank, repr(ex)))


def test_late_join_and_leave():
    ps, q, _bar = _spawn(_churn_worker, 3)
    res = sorted(q.get(timeout=300) for _ in ps)
    [p.join(30) for p in ps]
    assert res == [(0, "ok"), (1, "ok"), (2, "ok")], res


def _auto_worker(rank, port, bar, q):
    try:
        import memfabric_hybrid_b200 as mf

        b = _open(mf, rank, 2, port, auto=True, pool=4 * MiB)
        me = mf.bm.bm_rank_id()
        bar.wait(60)
        q.put((rank, me))
        bar.wait(60)
        time.sleep(0.3 if me == 0 else 0)
        b.destroy()
        mf.bm.uninitialize()
    except Exception as ex:  # pragma: no cover
        import traceback

        traceback.print_exc()
        q.put((rank, repr(ex)))


def test_auto_ranking_races_for_the_store():
    ps, q, _bar = _spawn(_auto_worker, 2)
    got = [q.get(timeout=120) for _ in ps]
    [p.join(30) for p in ps]
    assert sorted(r for _, r in got) == [0, 1], got


def _victim(port, ready):
    import memfabric_hybrid_b200 as mf

    b = _open(mf, 1, 2, port, pool=4 * MiB)
    ready.put("joined")
    time.sleep(60)  # killed long before


def test_peer_death_is_detected_and_unmapped(mf):
    port = free_port()
    mf.native.set_heartbeat_ms(100, 3)
    try:
        ctx = mp.get_context("spawn")
        ready = ctx.Queue()
        b = None
        p = ctx.Process(target=_victim, args=(port, ready))
        # rank 0 (this process) hosts the store, so start it first in a thread-free way: initialise, then the victim joins
        cfg = mf.bm.BmConfig()
        cfg.rank_id = 0
        cfg.operation_timeout = 20
        assert mf.bm.initialize(f"tcp://127.0.0.1:{port}", 2, -1, cfg) == 0, mf.get_last_err_msg()
        b = mf.bm.create(0, 4 * MiB, 0, mf.bm.BmDataOpType.HOST_RDMA)
        assert b.join() == 0
        p.start()
        assert ready.get(timeout=60) == "joined"
        deadline = time.time() + 10
        while b.joined_size() != 2 and time.time() < deadline:
            time.sleep(0.02)
        assert b.joined_size() == 2
        H = mf.bm.BmMemType.HOST
        word = np.arange(64, dtype=np.uint8)
        assert b.copy_data(word.ctypes.data, b.peer_rank_ptr(H, 1), 64, mf.bm.BmCopyType.H2GH, 0) == 0
        os.kill(p.pid, 9)  # the exact child we started
        p.join(10)
        deadline = time.time() + 10
        while b.joined_size() != 1 and time.time() < deadline:
            time.sleep(0.05)
        assert b.joined_size() == 1, "the survivor did not notice the dead rank"
        # its window is gone from the pool: the copy is refused cleanly instead of touching unmapped memory
        assert b.copy_data(word.ctypes.data, b.peer_rank_ptr(H, 1), 64, mf.bm.BmCopyType.H2GH, 0) != 0
        # our own window still works
        assert b.copy_data(word.ctypes.data, b.peer_rank_ptr(H, 0), 64, mf.bm.BmCopyType.H2GH, 0) == 0
        b.destroy()
    finally:
        mf.bm.uninitialize()
        mf.native.set_heartbeat_ms(2000, 3)


def test_argument_validation(mf):
    cfg = mf.bm.BmConfig()
    cfg.rank_id = 0
    assert mf.bm.initialize("nonsense", 1, -1, cfg) != 0
    assert mf.bm.initialize("tcp://127.0.0.1:1", 0, -1, cfg) != 0
    cfg.rank_id = 5
    assert mf.bm.initialize(f"tcp://127.0.0.1:{free_port()}", 2, -1, cfg) != 0  # rank beyond the world
    with pytest.raises(RuntimeError):
        mf.bm.create(0, 2 * MiB, 0)  # not initialised
    cfg.rank_id = 0
    port = free_port()
    assert mf.bm.initialize(f"tcp://127.0.0.1:{port}", 1, -1, cfg) == 0
    try:
        with pytest.raises(RuntimeError):
            mf.bm.create(0, 3 * MiB, 0)  # not a multiple of 2 MiB
        with pytest.raises(RuntimeError):
            mf.bm.create(0, 0, 2 * MiB)  # HBM on a CPU-only rank
        with pytest.raises(RuntimeError):
            mf.bm.create(64, 2 * MiB, 0)  # id out of range
        b = mf.bm.create(3, 2 * MiB, 0, mf.bm.BmDataOpType.HOST_RDMA)
        with pytest.raises(RuntimeError):
            mf.bm.create(3, 2 * MiB, 0)  # duplicate id
        assert b.join() == 0 and b.join() == 0  # idempotent
        assert b.local_mem_size(mf.bm.BmMemType.HOST) == 2 * MiB and b.local_mem_size(mf.bm.BmMemType.DEVICE) == 0
        assert b.peer_rank_ptr(mf.bm.BmMemType.DEVICE, 0) == 0 and b.peer_rank_ptr(mf.bm.BmMemType.HOST, 9) == 0
        assert "memory" in mf.get_last_err_msg() or mf.get_last_err_msg() != ""
        assert mf.get_and_clear_last_err_msg() != "" and mf.get_last_err_msg() == ""
        b.destroy()
    finally:
        mf.bm.uninitialize()
