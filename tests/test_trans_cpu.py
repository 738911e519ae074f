"""Transfer engine without a GPU: two processes, host memory from the engine's shareable allocator, one-sided writes and
reads by peer address, deregistration, peer death seen through the store's fault handler. Mirrors the reference's
two-process sender/receiver tests (test/ut/testcase/smem/smem_trans_test.cpp:272-1269)."""
import multiprocessing as mp
import time

import numpy as np

from conftest import free_port


def _receiver(port, q_addr, q_done, die_early):
    import memfabric_hybrid_b200 as mf

    try:
        e = mf.TransferEngine()
        assert e.initialize(f"tcp://127.0.0.1:{port}", "127.0.0.1:9002", "Decode", -1) == 0, mf.get_last_err_msg()
        size = 4 << 20
        addr = e.malloc(size)
        assert addr != 0
        buf = mf.native.host_read  # noqa: F841
        mf.native.host_write(addr, bytes(size))
        assert e.register_memory(addr, size) == 0, mf.get_last_err_msg()
        assert e.register_memory(addr, size) != 0  # duplicate
        q_addr.put(addr)
        if die_early:
            q_done.get(timeout=60)
            import os

            os._exit(0)  # no goodbye: the store must notice the broken link
        assert q_done.get(timeout=60) == "written"
        got = mf.native.host_read(addr + 4096, 1 << 20)
        exp = np.random.default_rng(5).integers(0, 256, 1 << 20, dtype=np.uint8).tobytes()
        assert got == exp
        # leave something for the sender to read back
        mf.native.host_write(addr + (2 << 20), b"pong" * 1024)
        q_addr.put("ready")
        assert q_done.get(timeout=60) == "read"
        assert e.unregister_memory(addr) == 0
        assert e.unregister_memory(addr) != 0
        q_addr.put("unregistered")
        assert q_done.get(timeout=60) == "bye"
        assert e.free(addr) == 0
        e.unInitialize()
        q_addr.put("ok")
    except Exception as ex:  # pragma: no cover
        import traceback

        traceback.print_exc()
        q_addr.put(repr(ex))


def test_two_processes_write_read_deregister(mf, port):
    url = f"tcp://127.0.0.1:{port}"
    assert mf.create_config_store(url) == 0
    ctx = mp.get_context("spawn")
    q_addr, q_done = ctx.Queue(), ctx.Queue()
    p = ctx.Process(target=_receiver, args=(port, q_addr, q_done, False))
    p.start()
    try:
        peer_addr = q_addr.get(timeout=60)
        assert isinstance(peer_addr, int), peer_addr
        e = mf.TransferEngine()
        assert e.initialize(url, "127.0.0.1:9001", "Prefill", -1) == 0, mf.get_last_err_msg()
        assert e.get_rpc_port() == 9001
        assert e.get_rank() != 0xFFFFFFFF
        data = np.random.default_rng(5).integers(0, 256, 1 << 20, dtype=np.uint8)
        # batch write of 16 blocks into the peer's registered range, by the peer's own addresses
        blk = 65536
        locs = [data.ctypes.data + i * blk for i in range(16)]
        rems = [peer_addr + 4096 + i * blk for i in range(16)]
        assert e.batch_transfer_sync_write("127.0.0.1:9002", locs, rems, [blk] * 16) == 0, mf.get_last_err_msg()
        # outside the registered range / unknown peer
        assert e.transfer_sync_write("127.0.0.1:9002", data.ctypes.data, peer_addr + (4 << 20) - 10, 4096) != 0
        q_done.put("written")
        assert q_addr.get(timeout=60) == "ready"
        back = np.zeros(4096, dtype=np.uint8)
        assert e.transfer_sync_read("127.0.0.1:9002", back.ctypes.data, peer_addr + (2 << 20), 4096) == 0, mf.get_last_err_msg()
        assert back.tobytes() == b"pong" * 1024
        q_done.put("read")
        assert q_addr.get(timeout=60) == "unregistered"
        # roles: a second receiver ("Decode") may not reach into the first one's memory; its registration is never mapped
        e_rr = mf.TransferEngine()
        assert e_rr.initialize(url, "127.0.0.1:9005", "Decode", -1) == 0
        assert e_rr.transfer_sync_read("127.0.0.1:9002", back.ctypes.data, peer_addr + (2 << 20), 4096) != 0
        assert "same role" in mf.get_last_err_msg()
        e_rr.destroy()
        # a fresh engine (empty cache) must see the deregistration
        e2 = mf.TransferEngine()
        assert e2.initialize(url, "127.0.0.1:9003", "Prefill", -1) == 0
        assert e2.transfer_sync_write("127.0.0.1:9002", data.ctypes.data, peer_addr, 4096) != 0
        e2.destroy()
        q_done.put("bye")
        assert q_addr.get(timeout=60) == "ok"
        e.unInitialize()
    finally:
        p.join(timeout=30)
        if p.is_alive():
            p.terminate()
        mf.destroy_config_store(url)


def test_peer_death_marks_records_abnormal(mf, port):
    url = f"tcp://127.0.0.1:{port}"
    assert mf.create_config_store(url) == 0
    ctx = mp.get_context("spawn")
    q_addr, q_done = ctx.Queue(), ctx.Queue()
    p = ctx.Process(target=_receiver, args=(port, q_addr, q_done, True))
    p.start()
    try:
        peer_addr = q_addr.get(timeout=60)
        assert isinstance(peer_addr, int), peer_addr
        e = mf.TransferEngine()
        assert e.initialize(url, "127.0.0.1:9001", "Prefill", -1) == 0
        data = np.arange(4096, dtype=np.uint8)
        assert e.transfer_sync_write("127.0.0.1:9002", data.ctypes.data, peer_addr, 4096) == 0, mf.get_last_err_msg()
        q_done.put("die")
        p.join(timeout=30)
        # the server saw the link break and flagged the device record; a client reading it sees the status byte 'A'
        c = mf.native.TcpStore("127.0.0.1", port, False, 0, -1)
        assert c.startup(3, 100) == 0
        deadline = time.time() + 5
        status = b""
        while time.time() < deadline:
            rc, v = c.get("/trans/dev/127.0.0.1:9002", 0)
            status = v[:1]
            if status == b"A":
                break
            time.sleep(0.05)
        assert status == b"A"
        rc, sl = c.get("/trans/slices/127.0.0.1:9002", 0)
        assert rc == 0 and sl[:1] == b"A"
        c.shutdown()
        # a new engine refuses to talk to the dead peer instead of touching unmapped memory
        e3 = mf.TransferEngine()
        assert e3.initialize(url, "127.0.0.1:9004", "Prefill", -1) == 0
        mf.native.set_retry_policy(2, 50, 1)
        assert e3.transfer_sync_write("127.0.0.1:9002", data.ctypes.data, peer_addr, 4096) != 0
        mf.native.set_retry_policy(3, 1000, 2)
        e3.destroy()
        e.unInitialize()
    finally:
        if p.is_alive():
            p.terminate()
        mf.destroy_config_store(url)


def _restartable_receiver(port, q_addr, q_cmd, generation):
    import memfabric_hybrid_b200 as mf

    try:
        e = mf.TransferEngine()
        assert e.initialize(f"tcp://127.0.0.1:{port}", "127.0.0.1:9012", "Decode", -1) == 0, mf.get_last_err_msg()
        size = 2 << 20
        addr = e.malloc(size)
        mf.native.host_write(addr, bytes([generation]) * size)
        assert e.register_memory(addr, size) == 0, mf.get_last_err_msg()
        q_addr.put(addr)
        cmd = q_cmd.get(timeout=60)
        if cmd == "die":
            import os

            os._exit(0)
        got = mf.native.host_read(addr, 4096)
        q_addr.put(got == bytes([77]) * 4096)
        assert q_cmd.get(timeout=60) == "bye"
        e.unInitialize()
    except Exception as ex:  # pragma: no cover
        import traceback

        traceback.print_exc()
        q_addr.put(repr(ex))


def test_transfer_is_retried_while_the_peer_restarts(mf, port):
    """The receiver process is killed and started again under the same id; a transfer issued in between fails at first (the peer's
    records are flagged abnormal), is retried with growing pauses after re-reading the peer's records, and lands in the NEW
    process's memory. Reference policy: three attempts, 1 s and 2 s apart, forced reconnect in between
    (host_hcom_transport_manager.cpp:865-883); the pauses are shortened here."""
    import threading

    url = f"tcp://127.0.0.1:{port}"
    assert mf.create_config_store(url) == 0
    mf.native.set_retry_policy(6, 300, 2)
    ctx = mp.get_context("spawn")
    q_addr, q_cmd = ctx.Queue(), ctx.Queue()
    p1 = ctx.Process(target=_restartable_receiver, args=(port, q_addr, q_cmd, 1))
    p1.start()
    p2 = None
    try:
        addr1 = q_addr.get(timeout=60)
        assert isinstance(addr1, int), addr1
        e = mf.TransferEngine()
        assert e.initialize(url, "127.0.0.1:9011", "Prefill", -1) == 0
        data = np.full(4096, 77, dtype=np.uint8)
        assert e.transfer_sync_write("127.0.0.1:9012", data.ctypes.data, addr1, 4096) == 0, mf.get_last_err_msg()
        q_cmd.put("die")
        p1.join(timeout=30)
        time.sleep(0.5)  # the store notices the broken link and flags the records
        before = mf.native.retry_stats()[0]
        # restart the peer a little later, from another thread, while the transfer below is in its retry pauses
        holder = {}

        def restart():
            time.sleep(0.2)
            holder["p"] = ctx.Process(target=_restartable_receiver, args=(port, q_addr, q_cmd, 2))
            holder["p"].start()
            holder["addr"] = q_addr.get(timeout=60)

        t = threading.Thread(target=restart)
        t.start()
        # the engine's host allocator hands out the same address in every process, so the address is still the right one
        rc = e.transfer_sync_write("127.0.0.1:9012", data.ctypes.data, addr1, 4096)
        t.join(60)
        p2 = holder["p"]
        assert holder["addr"] == addr1, (holder["addr"], addr1)
        assert rc == 0, mf.get_last_err_msg()
        assert mf.native.retry_stats()[0] > before  # it did not succeed at the first attempt
        q_cmd.put("check")
        assert q_addr.get(timeout=60) is True  # and the bytes are in the NEW process
        q_cmd.put("bye")
        p2.join(timeout=30)
        e.unInitialize()
    finally:
        mf.native.set_retry_policy(3, 1000, 2)
        for p in (p1, p2):
            if p is not None and p.is_alive():
                p.terminate()
        mf.destroy_config_store(url)
