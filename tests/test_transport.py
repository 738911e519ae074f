"""Transport layer on CPU: one-sided put/get over the host TCP transport (registration, keys, access rights, slicing,
asynchronous forms with the counting synchronise, role rule, refusal of bad tokens and ranges, retry with forced reconnect across
a restarted peer, TLS), the device-link manager driven through hooks, and the compose router. Scenarios follow the reference's
transport contract (src/hybm/csrc/transport/hybm_transport_manager.h:25-117) and its host transport's retry policy
(src/hybm/csrc/transport/host/host_hcom_transport_manager.cpp:865-883)."""
import ctypes
import multiprocessing as mp
import os
import threading
import time

import numpy as np
import pytest

BM_OK, BM_ERROR, BM_INVALID_PARAM = 0, -1, -2


def _buf(n, seed=None):
    a = np.zeros(n, dtype=np.uint8) if seed is None else np.random.default_rng(seed).integers(0, 256, n, dtype=np.uint8)
    return a, a.ctypes.data


def _pair(n, mf, roles=(0, 0), **kw):
    """Two host transports in this process, each serving one region, prepared with each other's address and keys."""
    ts, bufs = [], []
    for r in range(2):
        t = n.Transport(n.TT_HOST_TCP)
        assert t.open(r, 2, roles[r], "127.0.0.1:0", **kw) == BM_OK
        a, p = _buf(8 << 20)
        assert t.register_region(p, a.nbytes) == BM_OK
        ts.append(t)
        bufs.append((a, p))
    for r in range(2):
        o = 1 - r
        assert ts[r].prepare({o: {"nic": ts[o].nic(), "role": roles[o], "keys": [ts[o].memory_key(bufs[o][1])]}}) == BM_OK
    return ts, bufs


def test_put_get_sliced_and_async(mf):
    n = mf.native
    ts, bufs = _pair(n, mf, slice_bytes=256 << 10)
    assert ts[0].connect() == BM_OK and ts[0].linked(1)
    src, sp = _buf(3 << 20, seed=1)
    # blocking write of 3 MiB = 12 slices, then read it back
    assert ts[0].write(1, sp, bufs[1][1] + 4096, src.nbytes) == BM_OK
    assert np.array_equal(bufs[1][0][4096:4096 + src.nbytes], src)
    back, bp = _buf(src.nbytes)
    assert ts[0].read(1, bp, bufs[1][1] + 4096, src.nbytes) == BM_OK
    assert np.array_equal(back, src)
    st = ts[0].stats()
    assert st["slices"] == 24 and st["bytes_written"] == src.nbytes and st["bytes_read"] == src.nbytes
    assert ts[1].stats()["bytes_served"] == 2 * src.nbytes
    # asynchronous batch: nothing is promised before synchronize, everything is there after it
    bufs[1][0][:] = 0
    offs = [i * (300 << 10) for i in range(8)]
    assert ts[0].write_batch_async(1, [sp + o for o in offs], [bufs[1][1] + o for o in offs], [200 << 10] * 8) == BM_OK
    assert ts[0].synchronize(1) == BM_OK
    for o in offs:
        assert np.array_equal(bufs[1][0][o:o + (200 << 10)], src[o:o + (200 << 10)])
    # a rank may address its own registered memory through the same calls
    mine, mp_ = _buf(4096, seed=2)
    assert ts[0].write(0, mp_, bufs[0][1], 4096) == BM_OK and np.array_equal(bufs[0][0][:4096], mine)
    for t in ts:
        t.close()


def test_refusals_leave_memory_untouched(mf):
    n = mf.native
    ts, bufs = _pair(n, mf)
    assert ts[0].connect() == BM_OK
    src, sp = _buf(4096, seed=3)
    # outside every region the peer registered: refused locally, no request leaves
    assert ts[0].write(1, sp, bufs[1][1] + bufs[1][0].nbytes - 100, 4096) == BM_INVALID_PARAM
    # a forged token: the owner refuses, the bytes stay as they were, no retry is spent on it
    key = list(ts[1].memory_key(bufs[1][1]))
    key[0] ^= 0x5A5A
    assert ts[0].update_ranks({1: {"nic": ts[1].nic(), "role": 0, "keys": [tuple(key)]}}) == BM_OK
    before = mf.native.retry_stats()[0]
    assert ts[0].write(1, sp, bufs[1][1], 4096) == BM_INVALID_PARAM
    assert mf.native.retry_stats()[0] == before
    assert int(bufs[1][0][:4096].sum()) == 0 and ts[1].stats()["refused"] == 1
    # a read-only region refuses writes and serves reads
    ro, rp = _buf(8192, seed=4)
    assert ts[1].register_region(rp, ro.nbytes, n.MR_ACCESS_REMOTE_READ) == BM_OK
    assert ts[0].update_ranks({1: {"nic": ts[1].nic(), "role": 0, "keys": [ts[1].memory_key(bufs[1][1]), ts[1].memory_key(rp)]}}) == BM_OK
    assert ts[0].write(1, sp, rp, 4096) == BM_INVALID_PARAM
    got, gp = _buf(8192)
    assert ts[0].read(1, gp, rp, 8192) == BM_OK and np.array_equal(got, ro)
    # overlapping registration and unknown rank
    assert ts[1].register_region(rp + 100, 50) == BM_INVALID_PARAM
    assert ts[0].write(5, sp, rp, 16) == BM_INVALID_PARAM
    # unregistering takes the region away from peers
    assert ts[1].unregister_region(rp) == BM_OK
    assert ts[0].read(1, gp, rp, 8192) == BM_INVALID_PARAM and not ts[1].has_registered(rp, 1)
    for t in ts:
        t.close()


def test_role_rule(mf):
    n = mf.native
    assert n.role_permits_link(0, 0) and n.role_permits_link(1, 2) and n.role_permits_link(2, 1) and n.role_permits_link(0, 1)
    assert not n.role_permits_link(1, 1) and not n.role_permits_link(2, 2)
    # two senders: prepared with each other, yet neither opens a link nor may address the other
    ts, bufs = _pair(n, mf, roles=(1, 1))
    assert ts[0].connect() == BM_OK and not ts[0].linked(1)
    src, sp = _buf(64, seed=5)
    assert ts[0].write(1, sp, bufs[1][1], 64) == BM_INVALID_PARAM
    for t in ts:
        t.close()
    # sender and receiver link up
    ts, bufs = _pair(n, mf, roles=(1, 2))
    assert ts[0].connect() == BM_OK and ts[0].linked(1)
    assert ts[0].write(1, sp, bufs[1][1], 64) == BM_OK and np.array_equal(bufs[1][0][:64], src)
    for t in ts:
        t.close()


def _serve(port, ready, stop, token_q):
    import memfabric_hybrid_b200 as mf

    n = mf.native
    t = n.Transport(n.TT_HOST_TCP)
    assert t.open(1, 2, 0, "127.0.0.1:%d" % port) == 0
    a = np.zeros(1 << 20, dtype=np.uint8)
    # a fixed address so that the restarted server owns "the same" region under a new token
    assert t.register_region(a.ctypes.data, a.nbytes) == 0
    token_q.put((t.memory_key(a.ctypes.data), a.ctypes.data))
    ready.set()
    stop.wait(30)
    token_q.put(int(a[:4096].astype(np.uint64).sum()))
    t.close()


def test_retry_reconnects_to_a_restarted_peer(mf, port):
    """The peer dies between two writes and comes back on the same address with a new region key: the first write after
    the loss fails over the dead link, the retry policy reconnects, and once the new key is known the write lands."""
    n = mf.native
    ctx = mp.get_context("spawn")
    n.set_retry_policy(3, 150, 2)
    try:
        def start():
            ready, stop, q = ctx.Event(), ctx.Event(), ctx.Queue()
            p = ctx.Process(target=_serve, args=(port, ready, stop, q))
            p.start()
            assert ready.wait(30)
            key, addr = q.get(timeout=10)
            return p, stop, q, key, addr

        p, stop, q, key, addr = start()
        t = n.Transport(n.TT_HOST_TCP)
        assert t.open(0, 2, 0, "127.0.0.1:0", op_timeout_ms=2000) == BM_OK
        assert t.prepare({1: {"nic": "127.0.0.1:%d" % port, "role": 0, "keys": [key]}}) == BM_OK
        assert t.connect() == BM_OK
        src, sp = _buf(4096, seed=6)
        assert t.write(1, sp, addr, 4096) == BM_OK
        stop.set()
        assert q.get(timeout=10) == int(src.astype(np.uint64).sum())
        p.join(10)
        # peer gone: every attempt fails, the call gives up after the policy's attempts
        before = n.retry_stats()
        assert t.write(1, sp, addr, 4096) != BM_OK
        after = n.retry_stats()
        assert after[0] - before[0] == 2 and after[1] - before[1] == 1
        # peer back (new process, new token): a writer that starts while it is still down succeeds through the retries
        res = []
        th = threading.Thread(target=lambda: res.append(t.write(1, sp, addr2[0], 4096) if addr2 else None))
        addr2 = []
        p, stop, q, key2, a2 = start()
        addr2.append(a2)
        assert key2[0] != key[0]
        assert t.update_ranks({1: {"nic": "127.0.0.1:%d" % port, "role": 0, "keys": [key2]}}) == BM_OK
        th.start()
        th.join(20)
        assert res == [BM_OK] and t.stats()["reconnects"] >= 1
        stop.set()
        assert q.get(timeout=10) == int(src.astype(np.uint64).sum())
        p.join(10)
        t.close()
    finally:
        n.set_retry_policy(3, 1000, 2)


def test_device_links_through_hooks(mf):
    """The device transport keeps the link table and calls the owner's hooks: map on connect, copy on put/get, unmap on
    removal; a rank whose role forbids the link is never mapped."""
    n = mf.native
    calls = []
    t = n.Transport(n.TT_DEVICE_PEER)
    assert t.open(0, 4, 1) == BM_OK  # this rank is a sender
    peers = {r: _buf(1 << 16, seed=10 + r) for r in (1, 2, 3)}

    def copy(dst, src, size, is_async):
        ctypes.memmove(dst, src, size)
        calls.append(("copy", size, is_async))
        return 0

    assert t.set_device_hooks(lambda r: calls.append(("map", r)) or 0, lambda r: calls.append(("unmap", r)) or 0, copy) == 0
    prep = {r: {"role": 2 if r != 3 else 1, "keys": [(1, peers[r][1], 1 << 16, n.MR_ACCESS_ALL, n.MR_FLAG_HBM)]} for r in peers}
    assert t.prepare(prep) == BM_OK and t.connect() == BM_OK
    assert sorted(c for c in calls if c[0] == "map") == [("map", 1), ("map", 2)]  # rank 3 is a sender too
    states = {l["rank"]: l["state"] for l in t.links()}
    assert states == {1: "mapped", 2: "mapped", 3: "refused"}
    local, lp = _buf(4096, seed=20)
    assert t.write(1, lp, peers[1][1] + 128, 4096) == BM_OK and np.array_equal(peers[1][0][128:128 + 4096], local)
    got, gp = _buf(4096)
    assert t.read(2, gp, peers[2][1], 4096) == BM_OK and np.array_equal(got, peers[2][0][:4096])
    assert t.write(3, lp, peers[3][1], 64) == BM_INVALID_PARAM           # refused by role
    assert t.write(1, lp, peers[1][1] + (1 << 16) - 8, 64) == BM_INVALID_PARAM  # leaves what the rank exported
    assert t.remove_ranks([1]) == BM_OK and ("unmap", 1) in calls
    assert t.write(1, lp, peers[1][1], 64) != BM_OK
    assert {l["rank"]: l["state"] for l in t.links()}[1] == "removed"
    t.close()


def test_compose_routes_by_memory_kind(mf):
    n = mf.native
    comps, host_bufs, dev_bufs = [], [], []
    for r in range(2):
        c = n.Transport(n.TT_COMPOSE)
        assert c.open(r, 2, 0, "127.0.0.1:0") == BM_OK
        assert c.set_device_hooks(None, None, lambda d, s, sz, a: ctypes.memmove(d, s, sz) and 0) == 0
        hb, db = _buf(1 << 20), _buf(1 << 20)
        assert c.register_region(hb[1], 1 << 20, n.MR_ACCESS_ALL, n.MR_FLAG_DRAM) == BM_OK
        assert c.register_region(db[1], 1 << 20, n.MR_ACCESS_ALL, n.MR_FLAG_HBM) == BM_OK
        assert c.register_region(hb[1] + (2 << 20), 16, n.MR_ACCESS_ALL, 0) == BM_INVALID_PARAM  # a region must name its kind
        comps.append(c)
        host_bufs.append(hb)
        dev_bufs.append(db)
    for r in range(2):
        o = 1 - r
        keys = [comps[o].memory_key(host_bufs[o][1]), comps[o].memory_key(dev_bufs[o][1])]
        assert keys[0][4] == n.MR_FLAG_DRAM and keys[1][4] == n.MR_FLAG_HBM
        assert comps[r].prepare({o: {"nic": comps[o].nic(), "role": 0, "keys": keys}}) == BM_OK
    assert comps[0].connect() == BM_OK
    assert comps[0].route_of(1, host_bufs[1][1], 64) == n.TT_HOST_TCP
    assert comps[0].route_of(1, dev_bufs[1][1], 64) == n.TT_DEVICE_PEER
    assert comps[0].route_of(1, 0x1000, 64) == n.TT_COMPOSE
    src, sp = _buf(8192, seed=30)
    assert comps[0].write(1, sp, host_bufs[1][1], 8192) == BM_OK      # over the wire
    assert comps[0].write(1, sp, dev_bufs[1][1] + 64, 8192) == BM_OK  # through the copy hook
    assert np.array_equal(host_bufs[1][0][:8192], src) and np.array_equal(dev_bufs[1][0][64:64 + 8192], src)
    assert comps[0].stats()["bytes_written"] == 8192 and comps[1].stats()["bytes_served"] == 8192
    assert comps[0].write_async(1, sp, host_bufs[1][1] + 16384, 8192) == BM_OK and comps[0].synchronize(1) == BM_OK
    assert np.array_equal(host_bufs[1][0][16384:16384 + 8192], src)
    assert comps[0].write(1, sp, 0x1000, 64) == BM_INVALID_PARAM
    for c in comps:
        c.close()


def test_async_connect(mf):
    n = mf.native
    ts, _ = _pair(n, mf)
    assert ts[0].async_connect() == BM_OK
    assert ts[0].wait_connected(5_000_000_000) == BM_OK and ts[0].linked(1)
    for t in ts:
        t.close()
