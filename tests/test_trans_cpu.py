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
        assert e3.transfer_sync_write("127.0.0.1:9002", data.ctypes.data, peer_addr, 4096) != 0
        e3.destroy()
        e.unInitialize()
    finally:
        if p.is_alive():
            p.terminate()
        mf.destroy_config_store(url)
