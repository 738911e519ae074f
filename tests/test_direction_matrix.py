"""Every legal (source, destination) placement of a copy, driven through the scripted multi-rank harness: two ranks, sources and
destinations drawn from {local host, local device, pooled host, pooled device} x {this rank, the other rank}, 64 MiB per copy on
GPUs (4 MiB on CPU ranks), verified by comparing checksums computed where the bytes live. A copy is legal when at least one
side is pooled memory. Mirrors the reference's all-path test (test/python/hybm/data_op_all_path_test.py:32-110: 2 processes x 2
devices, every (src, dst) pair, hash compare)."""
import itertools

import pytest

from conftest import free_port, has_gpu
from memfabric_hybrid_b200.testing import RankHarness

MiB = 1 << 20


def _device_count():
    if not has_gpu():
        return 0
    import torch

    return torch.cuda.device_count()


def _matrix(h, kinds, nbytes, pool_span):
    """Runs every legal pair from rank 0's point of view ("local" buffers live on rank 0) and returns how many it ran."""
    # local buffers of rank 0
    locs = {}
    if "LH" in kinds:
        locs["LH"] = h.call(0, "alloc", "host_pinned", nbytes, "lh")
        locs["LHp"] = h.call(0, "alloc", "host_pageable", nbytes, "lhp")
    if "LD" in kinds:
        locs["LD"] = h.call(0, "alloc", "device", nbytes, "ld")
    pool = {}
    for kind, tag in (("dram", "GH"), ("hbm", "GD")):
        if tag in kinds:
            pool[tag + "0"] = (kind, 0, 0)          # this rank's window
            pool[tag + "1"] = (kind, 1, 0)          # the other rank's window
    places = dict(locs)
    places.update(pool)
    ran, seed = 0, 100
    for s, d in itertools.product(places, places):
        s_pool, d_pool = s in pool, d in pool
        if not (s_pool or d_pool) or s == d:
            continue
        seed += 1
        src = places[s]
        dst = places[d]
        if d_pool:
            dst = (dst[0], dst[1], pool_span // 2)  # second half of the window, so a pool source is never overwritten
        # the bytes are written and summed where they live: by the owner of a pool window, by rank 0 for its locals
        filler = src[1] if s_pool else 0
        h.call(filler, "fill", src, nbytes, seed)
        want = h.call(filler, "checksum", src, nbytes)
        assert h.call(0, "copy", src, dst, nbytes) == 0, (s, d)
        owner = dst[1] if d_pool else 0
        got = h.call(owner, "checksum", dst, nbytes)
        assert got == want, f"{s} -> {d}: checksum differs"
        ran += 1
    return ran


def test_cpu_ranks_host_directions():
    """CPU ranks: local host (pinned and pageable) and pooled host memory of both ranks."""
    port = free_port()
    with RankHarness(2) as h:
        assert [r["rank"] for r in h.all("ping")] == [0, 1]
        h.all("bm_init", f"tcp://127.0.0.1:{port}", 2)
        h.all("bm_create", 0, 32 * MiB)
        assert h.all("bm_join")[-1] >= 1
        while min(h.all("joined_size")) < 2:
            pass
        ran = _matrix(h, {"LH", "GH"}, 4 * MiB, 32 * MiB)
        # LH, LHp, GH0, GH1: 16 ordered pairs - 4 equal - 4 with no pooled side + ... = every pair with a pooled side
        assert ran == 10
        with pytest.raises(Exception, match="copy_data"):
            h.call(0, "copy", "lh", "lhp", 4096)  # local to local is not a pool operation
        assert h.call(0, "copy", "lh", ("dram", 1, 32 * MiB - 8), 4096, None, 0, False) != 0  # leaves the pool


def test_cpu_ranks_on_two_emulated_hosts():
    """The same host-side matrix when the two ranks cannot map each other's memory: every remote placement goes over the wire."""
    port = free_port()
    env = [{"MF_HOST_IDENTITY": f"host-{r}", "MF_CROSS_HOST": "1", "MF_HOST_NIC": "127.0.0.1"} for r in range(2)]
    with RankHarness(2, env=env) as h:
        h.all("bm_init", f"tcp://127.0.0.1:{port}", 2)
        h.all("bm_create", 0, 32 * MiB)
        h.all("bm_join")
        while min(h.all("joined_size")) < 2:
            pass
        before = h.call(0, "stats")["remote_calls"]
        assert _matrix(h, {"LH", "GH"}, 4 * MiB, 32 * MiB) == 10
        assert h.call(0, "stats")["remote_calls"] - before >= 5  # LH→GH1, LHp→GH1, GH0→GH1, GH1→LH, GH1→LHp, GH1→GH0


@pytest.mark.gpu
@pytest.mark.skipif(_device_count() < 2, reason="needs two GPUs")
def test_two_gpu_ranks_all_directions():
    """2 processes x 2 GPUs, {LH, LD, GH, GD} x {local, remote}, 64 MiB per copy, checksum compare."""
    port = free_port()
    with RankHarness(2, gpus=[0, 1]) as h:
        h.all("bm_init", f"tcp://127.0.0.1:{port}", 2)
        h.all("bm_create", 256 * MiB, 256 * MiB)
        h.all("bm_join")
        while min(h.all("joined_size")) < 2:
            pass
        ran = _matrix(h, {"LH", "LD", "GH", "GD"}, 64 * MiB, 256 * MiB)
        # places: LH, LHp, LD, GH0, GH1, GD0, GD1 = 49 ordered pairs - 7 equal - 6 local-to-local
        assert ran == 36
        st = h.call(0, "stats")
        assert st["kernel_calls"] > 0 and st["copy_engine_calls"] > 0


@pytest.mark.gpu
@pytest.mark.skipif(_device_count() < 2, reason="needs two GPUs")
def test_two_gpu_ranks_on_two_emulated_hosts():
    """Two GPU ranks that believe they sit on different hosts: pooled HBM and DRAM of the other rank are reached over the host
    transport (device memory staged by the owner), locals on the device are staged through the pinned bounce buffer."""
    port = free_port()
    env = [{"MF_HOST_IDENTITY": f"host-{r}", "MF_CROSS_HOST": "1", "MF_HOST_NIC": "127.0.0.1"} for r in range(2)]
    with RankHarness(2, gpus=[0, 1], env=env) as h:
        h.all("bm_init", f"tcp://127.0.0.1:{port}", 2)
        h.all("bm_create", 64 * MiB, 64 * MiB)
        h.all("bm_join")
        while min(h.all("joined_size")) < 2:
            pass
        before = h.call(0, "stats")["remote_calls"]
        assert _matrix(h, {"LH", "LD", "GH", "GD"}, 16 * MiB, 64 * MiB) == 36
        assert h.call(0, "stats")["remote_calls"] - before >= 20
