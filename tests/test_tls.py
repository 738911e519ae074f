"""TLS 1.3 on the config-store links: mutual authentication with generated certificates, encrypted private key with a pass
phrase (plain and through a decrypt callback), rejection of plain-text clients and of certificates from a foreign CA, the
certificate validity check and its environment knobs. Scenario source: the reference's acc_links TLS tests with generated
certificates (test/ut/testcase/acc_links/acc_links_test.cpp, test/certs/generate_*.py)."""
import os
import shutil
import subprocess

import pytest

ST_OK = 0
OPENSSL = shutil.which("openssl")
pytestmark = pytest.mark.skipif(OPENSSL is None, reason="the openssl command line tool is needed to generate test certificates")


def _run(*args, cwd):
    subprocess.run([OPENSSL, *args], cwd=cwd, check=True, capture_output=True)


def _make_ca(d, name):
    _run("req", "-x509", "-newkey", "rsa:2048", "-nodes", "-keyout", f"{name}.key", "-out", f"{name}.pem", "-days", "365", "-subj", f"/CN={name}", cwd=d)


def _make_cert(d, ca, name, days=365, passphrase=None):
    _run("req", "-newkey", "rsa:2048", "-nodes", "-keyout", f"{name}.plain.key", "-out", f"{name}.csr", "-subj", f"/CN={name}", cwd=d)
    _run("x509", "-req", "-in", f"{name}.csr", "-CA", f"{ca}.pem", "-CAkey", f"{ca}.key", "-CAcreateserial", "-out", f"{name}.crt", "-days", str(days), cwd=d)
    if passphrase is not None:
        _run("pkey", "-in", f"{name}.plain.key", "-aes256", "-passout", f"pass:{passphrase}", "-out", f"{name}.key", cwd=d)
    else:
        shutil.copy(os.path.join(d, f"{name}.plain.key"), os.path.join(d, f"{name}.key"))


@pytest.fixture(scope="module")
def certs(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("tls"))
    _make_ca(d, "ca")
    _make_ca(d, "otherca")
    _make_cert(d, "ca", "node", passphrase="s3cret-pass")
    _make_cert(d, "otherca", "stranger")
    _make_cert(d, "ca", "shortlived", days=3)
    return d


def _info(d, cert, ca="ca.pem"):
    return f"tlsCaPath: {d}/; tlsCaFile: {ca}; tlsCert: {d}/{cert};"


@pytest.fixture
def tls_off(mf):
    yield
    mf.set_conf_store_tls(False, "")


def test_store_over_tls_and_rejections(mf, port, certs, tls_off):
    n = mf.native
    n.set_server_linger_ms(0)
    assert mf.set_conf_store_tls_key(f"{certs}/node.key", "s3cret-pass") == 0
    assert mf.set_conf_store_tls(True, _info(certs, "node.crt")) == 0, mf.get_last_err_msg()
    srv = n.TcpStore("127.0.0.1", port, True, 4, 0)
    assert srv.startup(5, 100) == 0, mf.get_last_err_msg()
    try:
        cli = n.TcpStore("127.0.0.1", port, False, 4, 1)
        assert cli.startup(5, 100) == 0, mf.get_last_err_msg()
        big = os.urandom(3 << 20)  # several TLS records in both directions
        assert cli.set("k", big) == ST_OK
        assert srv.get("k", 0) == (ST_OK, big)
        assert cli.get("k", 1000) == (ST_OK, big)
        assert cli.add("n", 5) == (ST_OK, 5)
        cli.shutdown()
        # a client that speaks plain TCP is turned away
        assert mf.set_conf_store_tls(False, "") == 0
        plain = n.TcpStore("127.0.0.1", port, False, 4, 2)
        assert plain.startup(1, 50) != 0
        plain.shutdown()
        # so is one whose certificate comes from a CA the server does not know (and which does not know the server's)
        assert mf.set_conf_store_tls_key(f"{certs}/stranger.key", "") == 0
        assert mf.set_conf_store_tls(True, _info(certs, "stranger.crt", ca="otherca.pem")) == 0
        stranger = n.TcpStore("127.0.0.1", port, False, 4, 3)
        assert stranger.startup(1, 50) != 0
        stranger.shutdown()
        # the right credentials still work afterwards
        assert mf.set_conf_store_tls_key(f"{certs}/node.key", "s3cret-pass") == 0
        assert mf.set_conf_store_tls(True, _info(certs, "node.crt")) == 0
        again = n.TcpStore("127.0.0.1", port, False, 4, 1)
        assert again.startup(5, 100) == 0
        assert again.get("n", 0) == (ST_OK, b"5")
        again.shutdown()
    finally:
        srv.shutdown()
        n.set_server_linger_ms(1500)


def test_wrong_pass_phrase_and_decrypt_callback(mf, port, certs, tls_off):
    n = mf.native
    n.set_server_linger_ms(0)
    assert mf.set_conf_store_tls(True, _info(certs, "node.crt")) == 0
    assert mf.set_conf_store_tls_key(f"{certs}/node.key", "wrong") == 0
    bad = n.TcpStore("127.0.0.1", port, True, 2, 0)
    assert bad.startup(1, 50) != 0  # the server cannot load its key
    bad.shutdown()
    # the pass phrase is stored reversed; the callback (the reference ships the same toy decrypter as its plug-in example) restores it
    seen = []

    def decrypt(cipher: bytes):
        seen.append(cipher)
        return cipher[::-1]

    assert mf.set_conf_store_tls_key(open(f"{certs}/node.key").read(), "s3cret-pass"[::-1], decrypt) == 0  # PEM text instead of a path
    srv = n.TcpStore("127.0.0.1", port, True, 2, 0)
    assert srv.startup(5, 100) == 0, mf.get_last_err_msg()
    cli = n.TcpStore("127.0.0.1", port, False, 2, 1)
    assert cli.startup(5, 100) == 0
    assert cli.set("x", b"y") == ST_OK and srv.get("x", 0) == (ST_OK, b"y")
    assert seen and seen[0] == b"s3cret-pass"[::-1]
    cli.shutdown()
    srv.shutdown()
    mf.set_conf_store_tls_key("unused", "", None)
    n.set_server_linger_ms(1500)


def test_certificate_validity_check(mf, certs, monkeypatch):
    n = mf.native
    rc, detail = n.tls_check_certificates(_info(certs, "node.crt"), f"{certs}/node.key", "s3cret-pass", 30)
    assert rc == 0, detail
    rc, detail = n.tls_check_certificates(_info(certs, "shortlived.crt"), f"{certs}/shortlived.key", "", 30)
    assert rc == 1 and "shortlived" in detail  # valid now, expires within the warning horizon
    rc, detail = n.tls_check_certificates(_info(certs, "shortlived.crt"), f"{certs}/shortlived.key", "", 1)
    assert rc == 0
    rc, detail = n.tls_check_certificates(_info(certs, "node.crt"), f"{certs}/stranger.key", "", 30)
    assert rc == -1  # key and certificate do not belong together
    rc, detail = n.tls_check_certificates("tlsCaPath: /nonexistent/; tlsCaFile: ca.pem; tlsCert: /nonexistent/x.crt", "k", "", 30)
    assert rc == -1
    assert n.tls_check_certificates("tlsBogus: 1", "k", "", 30)[0] == -2
    # environment knobs with the reference's ranges and defaults
    monkeypatch.delenv("ACCLINK_CHECK_PERIOD_HOURS", raising=False)
    monkeypatch.delenv("ACCLINK_CERT_CHECK_AHEAD_DAYS", raising=False)
    assert n.tls_cert_check_params() == (168, 30)
    monkeypatch.setenv("ACCLINK_CHECK_PERIOD_HOURS", "48")
    monkeypatch.setenv("ACCLINK_CERT_CHECK_AHEAD_DAYS", "14")
    assert n.tls_cert_check_params() == (48, 14)
    monkeypatch.setenv("ACCLINK_CHECK_PERIOD_HOURS", "5")       # below 24: default
    monkeypatch.setenv("ACCLINK_CERT_CHECK_AHEAD_DAYS", "400")  # above 180: default
    assert n.tls_cert_check_params() == (168, 30)


def test_enabling_tls_needs_options(mf, tls_off):
    assert mf.set_conf_store_tls(True, "") != 0
    assert mf.set_conf_store_tls(True, "tlsCaPath: /x/") != 0  # certificate and CA file missing
    assert mf.set_conf_store_tls(False, "") == 0


def test_host_transport_over_tls(mf, certs):
    """The one-sided host transport speaks TLS 1.3 with mutual authentication on its links when its options say so; a rank
    whose certificate chains to another CA cannot link."""
    import numpy as np

    n = mf.native
    n.set_retry_policy(2, 50, 2)
    try:
        ts, bufs = [], []
        for r, (crt, ca) in enumerate((("node.crt", "ca.pem"), ("node.crt", "ca.pem"), ("stranger.crt", "otherca.pem"))):
            t = n.Transport(n.TT_HOST_TCP)
            key = f"{certs}/{crt.split('.')[0]}.plain.key"
            assert t.open(r, 3, 0, "127.0.0.1:0", tls_info=_info(certs, crt, ca), tls_pk=key, op_timeout_ms=3000) == 0, mf.get_last_err_msg()
            a = np.zeros(1 << 16, dtype=np.uint8)
            assert t.register_region(a.ctypes.data, a.nbytes) == 0
            ts.append(t)
            bufs.append(a)
        recs = {r: {"nic": ts[r].nic(), "role": 0, "keys": [ts[r].memory_key(bufs[r].ctypes.data)]} for r in range(3)}
        assert ts[0].prepare({1: recs[1]}) == 0 and ts[0].connect() == 0
        src = np.random.default_rng(0).integers(0, 256, 4096, dtype=np.uint8)
        assert ts[0].write(1, src.ctypes.data, bufs[1].ctypes.data, 4096) == 0
        assert np.array_equal(bufs[1][:4096], src)
        # the stranger trusts only its own CA and presents a certificate ours does not trust: no link, no bytes
        assert ts[2].prepare({1: recs[1]}) == 0
        assert ts[2].connect() != 0 and not ts[2].linked(1)
        assert ts[2].write(1, src.ctypes.data, bufs[1].ctypes.data + 8192, 4096) != 0
        assert int(bufs[1][8192:8192 + 4096].sum()) == 0
        for t in ts:
            t.close()
    finally:
        n.set_retry_policy(3, 1000, 2)
