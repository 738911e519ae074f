"""Big Memory across hosts, emulated on one machine: two CPU ranks whose host identities differ (MF_HOST_IDENTITY), so neither
can map the other's DRAM and every copy that touches the other rank's window is carried by the TCP host transport. Checks
the link table, single and batched copies in both directions, the remote-to-remote case, bounds and refusals, and that a
rank without cross-host mode fails the join with a clear error instead of mapping garbage. The reference reaches host memory
on other nodes through its RDMA host transport (src/hybm/csrc/transport/host/host_hcom_transport_manager.cpp); the contract
tested here is the same one-sided put/get."""
import multiprocessing as mp
import os

import numpy as np

from conftest import free_port

MiB = 1 << 20
POOL = 32 * MiB


def _seeded(n, seed):
    return np.random.default_rng(seed).integers(0, 256, n, dtype=np.uint8)


def _worker(rank, port, bar, q, cross):
    try:
        os.environ["MF_HOST_IDENTITY"] = f"emulated-host-{rank}"
        os.environ["MF_HOST_NIC"] = "127.0.0.1"
        if cross[rank]:
            os.environ["MF_CROSS_HOST"] = "1"
        import memfabric_hybrid_b200 as mf

        cfg = mf.bm.BmConfig()
        cfg.rank_id = rank
        cfg.init_timeout = cfg.create_timeout = cfg.operation_timeout = 30
        assert mf.bm.initialize(f"tcp://127.0.0.1:{port}", 2, -1, cfg) == 0, mf.get_last_err_msg()
        b = mf.bm.create(0, POOL, 0, mf.bm.BmDataOpType.HOST_RDMA)
        if not all(cross):
            # Rank 0 serves its memory, rank 1 does not. Rank 0 joins first (alone); rank 1's join then has to import rank 0's
            # slices, finds them on another host and has no transport to reach them: it fails with a message that says so.
            # Rank 0 never gets to use rank 1's window either.
            if rank == 0:
                assert b.join() == 0, mf.get_last_err_msg()
            bar.wait(60)
            msg = ""
            if rank == 1:
                rc = b.join()
                msg = mf.get_last_err_msg()
                bar.wait(60)
                q.put((rank, "join=%d" % (0 if rc == 0 else 1), msg[:300]))
            else:
                bar.wait(60)
                tmp = np.zeros(64, dtype=np.uint8)
                rc = b.copy_data(tmp.ctypes.data, b.peer_rank_ptr(mf.bm.BmMemType.HOST, 1), 64, mf.bm.BmCopyType.H2GH, 0)
                q.put((rank, "copy=%d" % (0 if rc == 0 else 1), ""))
            bar.wait(60)
            return
        rc = b.join()
        assert rc == 0, mf.get_last_err_msg()
        T, H = mf.bm.BmCopyType, mf.bm.BmMemType.HOST
        peer = 1 - rank
        mine, theirs = b.peer_rank_ptr(H, rank), b.peer_rank_ptr(H, peer)
        bar.wait(60)
        before = mf.native.data_op_stats()
        # put into the other host's window, sizes around the transport's 4 MiB slice
        sizes = [4096, 1 * MiB, 4 * MiB + 4096, 9 * MiB]
        off = 0
        for i, n in enumerate(sizes):
            data = _seeded(n, 100 * rank + i)
            assert b.copy_data(data.ctypes.data, theirs + off, n, T.H2GH, 0) == 0, mf.get_last_err_msg()
            off += n
        bar.wait(60)
        # what the other rank put into mine is there (read through the local mapping), and I can get it back from theirs
        off = 0
        for i, n in enumerate(sizes):
            want = _seeded(n, 100 * peer + i)
            assert mf.native.host_read(mine + off, n) == want.tobytes(), f"put of {n} bytes"
            back = np.zeros(n, dtype=np.uint8)
            assert b.copy_data(theirs + off, back.ctypes.data, n, T.GH2H, 0) == 0, mf.get_last_err_msg()
            assert (back == _seeded(n, 100 * rank + i)).all(), f"get of {n} bytes"
            off += n
        bar.wait(60)
        # batch: 32 blocks of 16 KiB, half to my own window, half to the other host's
        blocks = _seeded(32 * (16 << 10), 7 + rank)
        srcs = [blocks.ctypes.data + i * (16 << 10) for i in range(32)]
        base = 20 * MiB
        dsts = [(mine if i % 2 == 0 else theirs) + base + (rank * 32 + i) * (16 << 10) for i in range(32)]
        assert b.copy_data_batch(srcs, dsts, [16 << 10] * 32, 32, T.H2GH, 0) == 0, mf.get_last_err_msg()
        assert mf.native.data_op_stats()["batch_groups_last"] == 2
        bar.wait(60)
        pb = _seeded(32 * (16 << 10), 7 + peer)
        for i in range(32):
            src_rank, blocks_of = (rank, blocks) if i % 2 == 0 else (peer, pb)
            o = base + (src_rank * 32 + i) * (16 << 10)
            assert mf.native.host_read(mine + o, 16 << 10) == blocks_of[i * (16 << 10):(i + 1) * (16 << 10)].tobytes(), i
        # pool to pool between the hosts (GH → GH), both directions of "remote"
        assert b.copy_data(mine, theirs + 28 * MiB + rank * 8192, 8192, T.G2G, 0) == 0, mf.get_last_err_msg()
        bar.wait(60)
        got = np.zeros(8192, dtype=np.uint8)
        assert b.copy_data(theirs + 28 * MiB + rank * 8192, got.ctypes.data, 8192, T.GH2H, 0) == 0
        assert got.tobytes() == mf.native.host_read(mine, 8192)
        # refusals: leaving the remote window, and a local → local copy
        tmp = np.zeros(64, dtype=np.uint8)
        assert b.copy_data(tmp.ctypes.data, b.peer_rank_ptr(H, 1) + POOL - 8, 64, T.H2GH, 0) != 0
        after = mf.native.data_op_stats()
        assert after["remote_calls"] - before["remote_calls"] >= 2 * len(sizes) + 2
        assert after["remote_elems"] - before["remote_elems"] >= 2 * len(sizes) + 16
        bar.wait(60)
        b.destroy()
        mf.bm.uninitialize()
        q.put((rank, "ok", ""))
    except Exception as ex:  # pragma: no cover
        import traceback

        traceback.print_exc()
        q.put((rank, repr(ex), ""))


def _run(cross):
    ctx = mp.get_context("spawn")
    q, bar, port = ctx.Queue(), ctx.Barrier(2), free_port()
    ps = [ctx.Process(target=_worker, args=(r, port, bar, q, cross)) for r in range(2)]
    [p.start() for p in ps]
    res = sorted(q.get(timeout=240) for _ in ps)
    [p.join(30) for p in ps]
    return res


def test_two_hosts_dram_pool_over_tcp():
    res = _run((True, True))
    assert [(r[0], r[1]) for r in res] == [(0, "ok"), (1, "ok")], res


def test_join_refuses_a_host_that_does_not_serve_its_memory():
    res = _run((True, False))
    by_rank = {r[0]: r for r in res}
    assert by_rank[1][1] == "join=1" and ("cross-host" in by_rank[1][2] or "join callback failed" in by_rank[1][2]), res
    assert by_rank[0][1] == "copy=1", res


def _trans_receiver(port, q_addr, q_done):
    os.environ["MF_HOST_IDENTITY"] = "decode-host"
    os.environ["MF_HOST_NIC"] = "127.0.0.1"
    os.environ["MF_CROSS_HOST"] = "1"
    import memfabric_hybrid_b200 as mf

    try:
        e = mf.TransferEngine()
        assert e.initialize(f"tcp://127.0.0.1:{port}", "127.0.0.1:9102", "Decode", -1) == 0, mf.get_last_err_msg()
        size = 8 << 20
        addr = e.malloc(size)
        assert addr != 0
        mf.native.host_write(addr, bytes(size))
        assert e.register_memory(addr, size) == 0, mf.get_last_err_msg()
        q_addr.put(addr)
        assert q_done.get(timeout=60) == "written"
        exp = _seeded(5 << 20, 11)
        assert mf.native.host_read(addr + 4096, exp.size) == exp.tobytes()
        mf.native.host_write(addr + (6 << 20), b"pong" * 1024)
        q_addr.put("ready")
        assert q_done.get(timeout=60) == "read"
        e.unInitialize()
        q_addr.put("ok")
    except Exception as ex:  # pragma: no cover
        import traceback

        traceback.print_exc()
        q_addr.put(repr(ex))


def _trans_sender(port, q_addr, q_done, q_res):
    os.environ["MF_HOST_IDENTITY"] = "prefill-host"
    os.environ["MF_HOST_NIC"] = "127.0.0.1"
    os.environ["MF_CROSS_HOST"] = "1"
    import memfabric_hybrid_b200 as mf

    try:
        peer_addr = q_addr.get(timeout=60)
        assert isinstance(peer_addr, int), peer_addr
        e = mf.TransferEngine()
        assert e.initialize(f"tcp://127.0.0.1:{port}", "127.0.0.1:9101", "Prefill", -1) == 0, mf.get_last_err_msg()
        data = _seeded(5 << 20, 11)
        before = mf.native.data_op_stats()["remote_calls"]
        # 5 blocks of 1 MiB: each crosses the transport's slice size at most once
        locs = [data.ctypes.data + i * MiB for i in range(5)]
        rems = [peer_addr + 4096 + i * MiB for i in range(5)]
        assert e.batch_transfer_sync_write("127.0.0.1:9102", locs, rems, [MiB] * 5) == 0, mf.get_last_err_msg()
        assert mf.native.data_op_stats()["remote_calls"] - before == 5
        # outside what the peer registered: refused before anything is sent
        assert e.transfer_sync_write("127.0.0.1:9102", data.ctypes.data, peer_addr + (8 << 20) - 10, 4096) != 0
        q_done.put("written")
        assert q_addr.get(timeout=60) == "ready"
        back = np.zeros(4096, dtype=np.uint8)
        assert e.transfer_sync_read("127.0.0.1:9102", back.ctypes.data, peer_addr + (6 << 20), 4096) == 0, mf.get_last_err_msg()
        assert back.tobytes() == b"pong" * 1024
        q_done.put("read")
        assert q_addr.get(timeout=60) == "ok"
        e.unInitialize()
        q_res.put("ok")
    except Exception as ex:  # pragma: no cover
        import traceback

        traceback.print_exc()
        q_res.put(repr(ex))


def test_transfer_engine_between_two_emulated_hosts(mf, port):
    """Prefill on one host writes KV blocks into memory a decode process registered on another host, by the decoder's own
    addresses, and reads a reply back: the transfer engine's sender/receiver contract over the host transport."""
    assert mf.create_config_store(f"tcp://127.0.0.1:{port}") == 0
    ctx = mp.get_context("spawn")
    q_addr, q_done, q_res = ctx.Queue(), ctx.Queue(), ctx.Queue()
    pr = ctx.Process(target=_trans_receiver, args=(port, q_addr, q_done))
    ps = ctx.Process(target=_trans_sender, args=(port, q_addr, q_done, q_res))
    pr.start()
    ps.start()
    try:
        assert q_res.get(timeout=120) == "ok"
    finally:
        pr.join(30)
        ps.join(30)
        mf.destroy_config_store(f"tcp://127.0.0.1:{port}")
