"""Share Memory (symmetric heap) API on a GPU: creation with address negotiation, peer visibility, control collectives,
extra context, atomic values. Two ranks share GPU 0 here (no kernel of one rank waits on the other), mirroring the
reference's fork-based two-rank tests (test/ut/testcase/smem/smem_bm_test.cpp:209-416) and its ShiftPutGet example
(example/shm/ShiftPutGet/shm_all_shift.cpp:86-141)."""
import multiprocessing as mp

import pytest

from conftest import free_port

pytestmark = pytest.mark.gpu


def _worker(rank, port, q):
    try:
        import torch

        import memfabric_hybrid_b200 as mf
        from memfabric_hybrid_b200.parallel.heap import SymmetricHeap

        torch.cuda.set_device(0)
        heap = SymmetricHeap(rank, 2, 0, 16 << 20, store_url=f"tcp://127.0.0.1:{port}")
        h = heap.handle
        assert h.local_rank == rank and h.rank_size == 2
        assert heap.gva != 0 and h.device_meta != 0 and h.signal_base != 0
        assert h.local_ptr() == heap.gva + rank * heap.size
        # every rank got the same window address
        gathered = h.all_gather(heap.gva.to_bytes(8, "little"))
        assert gathered[:8] == gathered[8:16]
        # shift put: write my rank into the next rank's heap, read what the previous rank left in mine
        off, mine = heap.empty((1024,), torch.int32)
        mine.fill_(-1)
        torch.cuda.synchronize()
        heap.barrier()
        heap.tensor(off, (1024,), torch.int32, rank=1 - rank).fill_(100 + rank)
        torch.cuda.synchronize()
        heap.barrier()
        assert int(mine[0]) == 100 + (1 - rank) and int(mine[-1]) == 100 + (1 - rank)
        # control plane
        assert h.subgroup_barrier("pair", 2, rank) == 0
        assert h.subgroup_all_gather("pair", 2, rank, bytes([rank])) == b"\x00\x01"
        rc, v = h.atomic_alloc_value(8)
        assert rc == 0
        vals = h.all_gather(bytes([v]))
        assert sorted(vals) == [0, 1]
        assert h.atomic_release_value(v) == 0
        assert h.set_context(b"ctx-%d" % rank) == 0
        assert h.set_context(b"") != 0 and h.set_context(b"x" * 65537) != 0
        rc, reach = h.topology_can_reach(1 - rank)
        assert rc == 0 and reach & int(mf.shm.ShmDataOpType.MTE)
        assert h.topology_can_reach(5)[0] != 0
        # device meta mirrors the host view
        import struct

        from memfabric_hybrid_b200.utils.tensors import device_tensor_from_gva

        meta = bytes(device_tensor_from_gva(h.device_meta, 128).cpu().numpy())
        _, mrank, mcount, ctxlen, sym, base = struct.unpack_from("<4I2Q", meta)
        assert (mrank, mcount, sym, base) == (rank, 2, heap.size, heap.gva) and ctxlen == len(b"ctx-%d" % rank)
        heap.barrier()
        heap.close()
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        import traceback

        traceback.print_exc()
        q.put((rank, repr(e)))


def test_two_ranks_symmetric_heap():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    ps = [ctx.Process(target=_worker, args=(r, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = sorted(q.get(timeout=240) for _ in ps)
    for p in ps:
        p.join(timeout=60)
    assert res == [(0, "ok"), (1, "ok")], res


def test_invalid_create_arguments(mf):
    cfg = mf.shm.ShmConfig()
    assert mf.shm.initialize("tcp://nonsense", 1, 0, 0, cfg) != 0
    assert mf.shm.initialize(f"tcp://127.0.0.1:{free_port()}", 1, 3, 0, cfg) != 0  # rank >= world
    port = free_port()
    assert mf.shm.initialize(f"tcp://127.0.0.1:{port}", 1, 0, 0, cfg) == 0
    try:
        with pytest.raises(RuntimeError):
            mf.shm.create(0, 1, 0, 3 << 20)  # not a multiple of 2 MiB
        with pytest.raises(RuntimeError):
            mf.shm.create(64, 1, 0, 2 << 20)  # id out of range
        s = mf.shm.create(1, 1, 0, 2 << 20)
        with pytest.raises(RuntimeError):
            mf.shm.create(1, 1, 0, 2 << 20)  # duplicate id
        assert s.barrier() == 0
        s.destroy()
    finally:
        mf.shm.uninitialize()
