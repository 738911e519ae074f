"""The SHM example programs as tests: each is started as one process per GPU on two GPUs and must exit 0. The shift-put example
checks the message it received; the put/signal micro-benchmark prints a table (latency of put + signal, put and get bandwidth
per message size) whose rows must be complete and positive."""
import os
import subprocess

import pytest

from conftest import free_port, has_gpu

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _two_gpus():
    if not has_gpu():
        return False
    import torch

    return torch.cuda.device_count() >= 2


def _run_pair(binary):
    url = f"tcp://127.0.0.1:{free_port()}"
    ps = [subprocess.Popen([binary, str(r), "2", url], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for p in ps:
        try:
            out, _ = p.communicate(timeout=180)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    return [p.returncode for p in ps], outs


@pytest.mark.skipif(not _two_gpus(), reason="needs two GPUs")
def test_shift_put_example():
    subprocess.run(["make", "-C", "examples", "shm_shift_put/shift_put"], cwd=ROOT, check=True, capture_output=True)
    codes, outs = _run_pair(os.path.join(ROOT, "examples", "shm_shift_put", "shift_put"))
    assert codes == [0, 0], outs


@pytest.mark.skipif(not _two_gpus(), reason="needs two GPUs")
def test_put_signal_bench_example():
    subprocess.run(["make", "-C", "examples", "shm_put_signal_bench/put_signal_bench"], cwd=ROOT, check=True, capture_output=True)
    codes, outs = _run_pair(os.path.join(ROOT, "examples", "shm_put_signal_bench", "put_signal_bench"))
    assert codes == [0, 0], outs
    rows = [ln.split() for ln in outs[0].splitlines() if ln.strip() and ln.split()[0].isdigit()]
    assert [int(r[0]) for r in rows] == [16 * 4 ** k for k in range(10)], outs[0]
    for r in rows:
        lat, put, get = float(r[1]), float(r[2]), float(r[3])
        assert 0.5 < lat < 5000 and put > 0 and get > 0, r
    # a 4 MiB put+signal is bandwidth-bound, a 16-byte one latency-bound
    assert float(rows[-1][1]) > float(rows[0][1])
