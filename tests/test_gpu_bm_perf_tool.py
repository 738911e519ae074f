"""The C++ bandwidth tool doubles as the multi-process direction matrix: one forked process per GPU, all ten directions of the
reference's bm_perf_benchmark (local/remote x host/device on either side, remote-host directions included), every transfer
byte-checked by the rank that received it. Model: test/python/hybm/data_op_all_path_test.py:32-110 of the reference (2 processes,
2 devices, 64 MiB per path, hash compare) and example/bm/BmBenchmark/band_width_calculator.cpp:423-600."""
import os
import subprocess

import pytest

from conftest import free_port

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOOL = os.path.join(ROOT, "examples", "bm_perf", "bm_perf")


def _build():
    subprocess.run(["make", "examples/bm_perf/bm_perf"], cwd=ROOT, check=True, capture_output=True)


@pytest.mark.parametrize("block,batch", [(1 << 20, 8), (64 << 20, 1), (4096 + 24, 5)])
def test_all_directions_verified(block, batch):
    import torch

    _build()
    ranks = min(torch.cuda.device_count(), 2)
    r = subprocess.run([TOOL, "-bw", "-t", "all", "-s", str(block), "-bs", str(batch), "-cc", "3", "-ws", str(ranks), "-lrs", str(ranks), "-ip",
                        f"tcp://127.0.0.1:{free_port()}"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "all directions verified" in r.stdout
    for name in ("h2d", "d2h", "h2rd", "h2rh", "d2rd", "d2rh", "rh2d", "rh2h", "rd2d", "rd2h"):
        assert r.stdout.count(f"  {name} ") == ranks and "FAILED" not in r.stdout, r.stdout[-3000:]


def test_pinned_local_host_buffers():
    import torch

    _build()
    ranks = min(torch.cuda.device_count(), 2)
    r = subprocess.run([TOOL, "-bw", "-t", "h2rd", "-pin", "-s", str(2 << 20), "-bs", "4", "-cc", "3", "-ws", str(ranks), "-lrs", str(ranks), "-ip",
                        f"tcp://127.0.0.1:{free_port()}"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "all directions verified" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
