"""Config store over loopback: every operation of the protocol, blocking gets, timeouts, watches, prefixes, large and binary
values, heartbeat supervision, rank-down notification, server loss and reconnect. Scenarios follow the reference's store
tests (test/ut/testcase/smem/acc_config_store_test.cpp:68-462)."""
import threading
import time

import pytest

ST_OK, ST_NOT_EXIST, ST_TIMEOUT, ST_IO_ERROR, ST_INVALID_KEY = 0, -404, -601, -602, -401


@pytest.fixture
def pair(mf, port):
    n = mf.native
    srv = n.TcpStore("127.0.0.1", port, True, 4, 0)
    assert srv.startup(5, 100) == 0
    cli = n.TcpStore("127.0.0.1", port, False, 4, 1)
    assert cli.startup(5, 100) == 0
    yield srv, cli
    cli.shutdown()
    srv.shutdown()


def test_url_parsing(mf):
    p = mf.native.parse_url
    assert p("tcp://127.0.0.1:5000") == ("127.0.0.1", 5000, False)
    assert p("tcp://[::1]:6000") == ("::1", 6000, True)
    assert p("tcp6://[fe80::1]:7") == ("fe80::1", 7, True)
    assert p("10.1.2.3:80") == ("10.1.2.3", 80, False)
    for bad in ["", "tcp://", "tcp://1.2.3.4", "tcp://1.2.3.4:0", "tcp://1.2.3.4:70000", "tcp://300.1.1.1:5", "tcp://[::1]6000", "tcp://1.2.3.4:12ab"]:
        assert p(bad) is None, bad


def test_message_codec(mf):
    n = mf.native
    buf = n.pack_message(1234, ["k1", "key2"], [b"\x00\x01binary\xff", b""])
    assert n.unpack_message(buf) == (1234, ["k1", "key2"], [b"\x00\x01binary\xff", b""])
    assert n.unpack_message(buf[:-1]) is None
    assert n.unpack_message(buf + b"x") is None
    assert n.unpack_message(b"short") is None
    assert n.unpack_message(n.pack_message(-1, ["k"] * 11, [])) is None


def test_set_get_remove(pair):
    srv, cli = pair
    assert cli.set("a", b"1") == ST_OK
    assert srv.get("a", 0) == (ST_OK, b"1")
    assert cli.set("a", b"2") == ST_OK
    assert cli.get("a", 0) == (ST_OK, b"2")
    assert cli.remove("a") == ST_OK
    assert cli.remove("a") == ST_NOT_EXIST
    assert cli.get("a", 0)[0] == ST_NOT_EXIST
    assert cli.set("", b"x") == ST_INVALID_KEY
    assert cli.set("k" * 1025, b"x") == ST_INVALID_KEY


def test_blocking_get_is_woken_by_set(pair):
    srv, cli = pair
    out = {}

    def waiter():
        out["r"] = cli.get("later", 5000)

    t = threading.Thread(target=waiter)
    t.start()
    time.sleep(0.1)
    assert srv.set("later", b"now") == ST_OK
    t.join(5)
    assert out["r"] == (ST_OK, b"now")


def test_get_timeout(pair):
    _, cli = pair
    t0 = time.time()
    rc, _ = cli.get("never", 200)
    assert rc == ST_TIMEOUT
    assert 0.15 < time.time() - t0 < 2.0


def test_add_append_cas_write(pair):
    srv, cli = pair
    assert cli.add("cnt", 5) == (ST_OK, 5)
    assert srv.add("cnt", -2) == (ST_OK, 3)
    assert cli.get("cnt", 0) == (ST_OK, b"3")
    assert cli.append("log", b"ab") == (ST_OK, 2)
    assert srv.append("log", b"cde") == (ST_OK, 5)
    assert cli.get("log", 0) == (ST_OK, b"abcde")
    # cas: expected "" matches an absent key; the previous value comes back either way
    assert cli.cas("lock", b"", b"A") == (ST_OK, b"")
    assert srv.cas("lock", b"", b"B") == (ST_OK, b"A")
    assert srv.cas("lock", b"A", b"C") == (ST_OK, b"A")
    assert cli.get("lock", 0) == (ST_OK, b"C")
    # write at an offset zero-fills the gap
    assert cli.write("slots", b"XY", 4) == ST_OK
    assert cli.get("slots", 0) == (ST_OK, b"\x00\x00\x00\x00XY")
    assert cli.write("slots", b"Q", 0) == ST_OK
    assert cli.get("slots", 0) == (ST_OK, b"Q\x00\x00\x00XY")


def test_add_and_append_wake_waiters(pair):
    srv, cli = pair
    got = []
    t = threading.Thread(target=lambda: got.append(cli.get("c2", 3000)))
    t.start()
    time.sleep(0.05)
    srv.add("c2", 7)
    t.join(3)
    assert got == [(ST_OK, b"7")]


def test_large_and_binary_values(pair):
    _, cli = pair
    blob = bytes(range(256)) * 4096 * 8  # 8 MiB
    assert cli.set("big", blob) == ST_OK
    assert cli.get("big", 0) == (ST_OK, blob)


def test_prefix_and_nested_prefix(mf, pair):
    srv, cli = pair
    p1 = mf.native.prefix_store(cli, "A_")
    p2 = mf.native.prefix_store(p1, "(3)_")
    assert p2.common_prefix() == "A_(3)_"
    assert p2.set("k", b"v") == ST_OK
    assert srv.get("A_(3)_k", 0) == (ST_OK, b"v")
    assert p1.get("(3)_k", 0) == (ST_OK, b"v")
    assert p2.get("k", 0) == (ST_OK, b"v")
    assert p1.get("k", 0)[0] == ST_NOT_EXIST


def test_arrive_is_one_request_rendezvous(mf, port):
    """Three clients arrive at a barrier key: nobody returns before the last one, the completing request drops the listed
    keys of an older round, a late duplicate is answered at once, and an arrival that nobody completes times out."""
    n = mf.native
    srv = n.StoreServer()
    assert srv.start("127.0.0.1", port) == 0
    clients = [n.TcpStore("127.0.0.1", port, False, 0, i) for i in range(3)]
    for c in clients:
        assert c.startup(5, 100) == 0
    assert clients[0].set("old_BA", b"3") == ST_OK and clients[0].set("old_BW", b"ok") == ST_OK
    done = []

    def arrive(i):
        rc = clients[i].arrive("r1_BA", "r1_BW", 3, 5000, ["old_BA", "old_BW"])
        done.append((i, rc, time.monotonic()))

    threads = [threading.Thread(target=arrive, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    time.sleep(0.3)
    assert done == []  # parked on the server
    assert clients[0].get("old_BA", 0)[0] == ST_OK  # nothing collected before the round completes
    t_last = time.monotonic()
    assert clients[2].arrive("r1_BA", "r1_BW", 3, 5000, ["old_BA", "old_BW"]) == ST_OK
    for t in threads:
        t.join(5)
    assert sorted(d[0] for d in done) == [0, 1] and all(d[1] == ST_OK and d[2] >= t_last for d in done)
    assert clients[0].get("r1_BW", 0) == (ST_OK, b"ok")
    assert clients[0].get("old_BA", 0)[0] == ST_NOT_EXIST and clients[0].get("old_BW", 0)[0] == ST_NOT_EXIST
    assert clients[1].arrive("r1_BA", "r1_BW", 3, 5000) == ST_OK  # the wake key already exists
    t0 = time.monotonic()
    assert clients[1].arrive("r2_BA", "r2_BW", 3, 200) == ST_TIMEOUT
    assert 0.15 <= time.monotonic() - t0 < 3
    assert clients[1].arrive("r3_BA", "r3_BW", 0, 200) != ST_OK  # a rendezvous of nobody is refused
    for c in clients:
        c.shutdown()
    srv.stop()


def test_gather_returns_every_record_once_full(mf, pair):
    srv, cli = pair
    pre = mf.native.prefix_store(cli, "G_")
    out = []
    t = threading.Thread(target=lambda: out.append(pre.gather("d", "w", b"AAAA", 8, 5000)))
    t.start()
    time.sleep(0.2)
    assert out == []
    assert srv.gather("G_d", "G_w", b"BBBB", 8, 5000) == (ST_OK, b"AAAABBBB")
    t.join(5)
    assert out == [(ST_OK, b"AAAABBBB")]
    assert srv.gather("G_d", "G_w", b"CCCC", 8, 1000)[0] != ST_OK  # the value would outgrow its full size
    assert srv.gather("x", "xw", b"AAAA", 12, 150)[0] == ST_TIMEOUT


def test_arrive_and_gather_base_composition(mf, pair):
    """An HA store wrapper has no request of its own for the rendezvous; a store without one composes it from the basic
    operations. Both routes end in the same state."""
    srv, cli = pair
    ha = mf.native.ha_store(cli) if hasattr(mf.native, "ha_store") else cli
    assert ha.arrive("b_BA", "b_BW", 1, 1000) == ST_OK
    assert srv.get("b_BW", 0) == (ST_OK, b"ok")
    assert ha.gather("g", "gw", b"zz", 2, 1000) == (ST_OK, b"zz")


def test_watch_and_unwatch(pair):
    srv, cli = pair
    seen = []
    rc, wid = cli.watch("w1", lambda r, k, v: seen.append((r, k, v)))
    assert rc == ST_OK
    rc2, wid2 = cli.watch("w2", lambda r, k, v: seen.append("w2"))
    assert cli.unwatch(wid2) == ST_OK
    srv.set("w1", b"hello")
    srv.set("w2", b"ignored")
    deadline = time.time() + 3
    while not seen and time.time() < deadline:
        time.sleep(0.01)
    time.sleep(0.1)
    assert seen == [(ST_OK, "w1", b"hello")]
    assert cli.unwatch(wid) == ST_NOT_EXIST  # one-shot: already consumed


def test_auto_ranking_hands_out_lowest_free(mf, port):
    n = mf.native
    srv = n.StoreServer()
    assert srv.start("127.0.0.1", port) == 0
    clients = [n.TcpStore("127.0.0.1", port, False, 0, -1) for _ in range(3)]
    for c in clients:
        assert c.startup(5, 100) == 0
    ranks = [int(c.get("AutoRanking#job", 1000)[1]) for c in clients]
    assert sorted(ranks) == [0, 1, 2]
    assert int(clients[1].get("AutoRanking#job", 1000)[1]) == ranks[1]  # stable per link
    clients[0].shutdown()
    time.sleep(0.3)
    late = n.TcpStore("127.0.0.1", port, False, 0, -1)
    assert late.startup(5, 100) == 0
    assert int(late.get("AutoRanking#job", 1000)[1]) == ranks[0]  # the freed id is reused
    for c in clients[1:] + [late]:
        c.shutdown()
    srv.stop()


def test_rank_down_notification_on_close(mf, port):
    n = mf.native
    srv = n.StoreServer()
    assert srv.start("127.0.0.1", port) == 0
    a = n.TcpStore("127.0.0.1", port, False, 2, 0)
    b = n.TcpStore("127.0.0.1", port, False, 2, 1)
    assert a.startup(5, 100) == 0 and b.startup(5, 100) == 0
    down = []
    assert a.watch_rank_down(lambda r: down.append(r))[0] == ST_OK
    time.sleep(0.1)
    b.shutdown()
    deadline = time.time() + 3
    while not down and time.time() < deadline:
        time.sleep(0.01)
    assert down == [1]
    a.shutdown()
    srv.stop()


def test_heartbeat_loss_marks_rank_down(mf, port):
    n = mf.native
    n.set_heartbeat_ms(50, 3)
    try:
        srv = n.StoreServer()
        assert srv.start("127.0.0.1", port) == 0
        a = n.TcpStore("127.0.0.1", port, False, 2, 0)
        b = n.TcpStore("127.0.0.1", port, False, 2, 1)
        assert a.startup(5, 100) == 0 and b.startup(5, 100) == 0
        down = []
        a.watch_rank_down(lambda r: down.append(r))
        time.sleep(0.3)
        assert down == [] and srv.alive_links() == 2  # heartbeats keep both alive
        b.set_drop_heartbeat(True)  # the process is alive, its socket is open, but it went silent
        deadline = time.time() + 5
        while not down and time.time() < deadline:
            time.sleep(0.02)
        assert down == [1]
        a.shutdown()
        b.shutdown()
        srv.stop()
    finally:
        n.set_heartbeat_ms(2000, 3)


def _server_process(port, conn):
    import memfabric_hybrid_b200 as mf

    n = mf.native
    n.set_heartbeat_ms(100, 3)
    srv = n.StoreServer()
    conn.send(srv.start("127.0.0.1", port))
    conn.recv()  # lives until the parent says so
    conn.send(srv.alive_links())
    srv.stop()


@pytest.mark.timeout(90)
def test_a_held_server_does_not_blame_its_clients(mf, port):
    """The server's process is stopped for much longer than the heartbeat deadline (as the kernel does to a process that pins
    gigabytes of host memory). When it runs again the silence was its own: no link is declared dead, nobody is told that a
    rank went down, the store keeps working."""
    import multiprocessing as mp
    import os
    import signal

    n = mf.native
    ctx = mp.get_context("spawn")
    parent, child = ctx.Pipe()
    proc = ctx.Process(target=_server_process, args=(port, child))
    proc.start()
    n.set_heartbeat_ms(100, 3)
    try:
        assert parent.recv() == 0
        a = n.TcpStore("127.0.0.1", port, False, 2, 0)
        b = n.TcpStore("127.0.0.1", port, False, 2, 1)
        assert a.startup(5, 100) == 0 and b.startup(5, 100) == 0
        down = []
        a.watch_rank_down(lambda r: down.append(r))
        assert a.set("k", b"v1") == ST_OK
        time.sleep(0.3)
        os.kill(proc.pid, signal.SIGSTOP)
        time.sleep(3.0)  # deadline for a silent link: 4 x 100 ms
        os.kill(proc.pid, signal.SIGCONT)
        time.sleep(1.0)  # several supervision passes after the hold
        assert down == []
        assert b.get("k", 1000) == (ST_OK, b"v1")
        parent.send("stop")
        assert parent.recv() == 2  # both links survived
        a.shutdown()
        b.shutdown()
    finally:
        n.set_heartbeat_ms(2000, 3)
        if proc.is_alive():
            os.kill(proc.pid, signal.SIGCONT)
        proc.join(timeout=10)


def test_store_cleared_when_last_client_leaves(mf, port):
    n = mf.native
    srv = n.StoreServer()
    assert srv.start("127.0.0.1", port) == 0
    a = n.TcpStore("127.0.0.1", port, False, 1, 0)
    assert a.startup(5, 100) == 0
    a.set("k", b"v")
    assert srv.size() == 1
    a.shutdown()
    deadline = time.time() + 3
    while srv.size() != 0 and time.time() < deadline:
        time.sleep(0.02)
    assert srv.size() == 0
    srv.stop()


def test_get_when_server_exits_then_reconnect(mf, port):
    n = mf.native
    srv = n.StoreServer()
    assert srv.start("127.0.0.1", port) == 0
    c = n.TcpStore("127.0.0.1", port, False, 1, 0)
    assert c.startup(5, 100) == 0
    broken, again = [], []
    c.set_broken_handler(lambda: broken.append(1))
    c.set_reconnect_handler(lambda: again.append(1))
    res = []
    t = threading.Thread(target=lambda: res.append(c.get("never", -1)))
    t.start()
    time.sleep(0.1)
    srv.stop()
    t.join(5)
    assert res and res[0][0] == ST_IO_ERROR  # the blocked get fails instead of hanging
    deadline = time.time() + 3
    while not broken and time.time() < deadline:
        time.sleep(0.01)
    assert broken
    assert c.set("x", b"1") == ST_IO_ERROR
    srv2 = n.StoreServer()
    assert srv2.start("127.0.0.1", port) == 0
    assert c.reconnect(5) == ST_OK
    assert again
    assert c.set("x", b"1") == ST_OK
    c.shutdown()
    srv2.stop()


def test_second_server_on_same_port_reports_in_use(mf, port):
    n = mf.native
    s1, s2 = n.StoreServer(), n.StoreServer()
    assert s1.start("127.0.0.1", port) == 0
    assert s2.start("127.0.0.1", port) == -98  # EADDRINUSE
    s1.stop()


def test_ipv6_loopback(mf, port):
    n = mf.native
    srv = n.StoreServer()
    if srv.start("::1", port) != 0:
        pytest.skip("no IPv6 loopback here")
    c = n.TcpStore("::1", port, False, 1, 0)
    assert c.startup(3, 100) == 0
    assert c.set("v6", b"ok") == ST_OK and c.get("v6", 0) == (ST_OK, b"ok")
    c.shutdown()
    srv.stop()


def test_ha_store_delegates(mf, pair):
    srv, cli = pair
    ha = mf.native.ha_store(cli)
    assert ha.set("h", b"1") == ST_OK and srv.get("h", 0) == (ST_OK, b"1")


def test_create_config_store_api(mf, port):
    url = f"tcp://127.0.0.1:{port}"
    assert mf.create_config_store(url) == 0
    assert mf.create_config_store("tcp://nonsense") != 0
    c = mf.native.TcpStore("127.0.0.1", port, False, 1, 0)
    assert c.startup(3, 100) == 0
    assert c.add("n", 1) == (ST_OK, 1)
    c.shutdown()
    mf.destroy_config_store(url)
