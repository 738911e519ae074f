"""Fused all-reduce + residual + RMSNorm kernel against a plain PyTorch fp32 oracle.

One GPU: the R ranks are emulated as slices of one cooperative launch over a fake heap (separate launches that wait on
each other are never run on one GPU). Two or more GPUs: real ranks, one process per GPU, over the real symmetric heap.
The bounded-wait path is exercised by leaving a rank out of the launch: its flags never arrive, the waits run out after
a short limit and the kernel reports the timeout in its status word while the context stays usable."""
import multiprocessing as mp

import pytest

from conftest import free_port

pytestmark = pytest.mark.gpu


def _make_inputs(world, T, H, seed):
    import torch

    g = torch.Generator(device="cuda").manual_seed(seed)
    xs = [torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
    res = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn(H, generator=g, device="cuda")).to(torch.bfloat16)
    return xs, res, w


@pytest.mark.parametrize("algo", ["oneshot", "twoshot"])
@pytest.mark.parametrize("world,T,H", [(2, 1, 512), (2, 5, 8192), (4, 33, 4096), (8, 16, 8192), (8, 257, 8192), (3, 7, 16384), (8, 3, 1024)])
def test_emulated_ranks_match_oracle(algo, world, T, H):
    import torch

    from memfabric_hybrid_b200.ops.allreduce import emulated_allreduce, reference
    from memfabric_hybrid_b200.parallel.heap import EmulatedHeap

    eps = 1e-6
    xs, res, w = _make_inputs(world, T, H, 1000 * world + T)
    heap = EmulatedHeap(world, 2 * T * H * 2 + 8192)
    x_off, r_off = heap.alloc(T * H * 2), heap.alloc(T * H * 2)
    for r in range(world):
        heap.tensor(r, x_off, (T, H), torch.bfloat16).copy_(xs[r])
    outs, status = emulated_allreduce(heap, x_off, r_off, [res] * world, w, T, H, eps, algo)
    assert status == [0] * world
    ref_out, ref_h = reference(xs, res, w, eps)
    for r in range(world):
        h = heap.tensor(r, r_off, (T, H), torch.bfloat16)
        assert torch.equal(h.float(), ref_h), f"rank {r}: new residual differs"
        torch.testing.assert_close(outs[r].float(), ref_out, atol=2e-2, rtol=2e-2)
        assert torch.equal(outs[r], outs[0]), "ranks must agree bit for bit"


def test_emulated_oneshot_without_closing_barrier_on_alternating_buffers():
    """The one-shot variant that skips its closing barrier, driven the way it must be: inputs alternate between two buffers."""
    import torch

    from memfabric_hybrid_b200.ops.allreduce import emulated_allreduce, reference

    from memfabric_hybrid_b200.parallel.heap import EmulatedHeap

    world, T, H = 4, 6, 4096
    heap = EmulatedHeap(world, 3 * T * H * 2 + 8192)
    x_offs = [heap.alloc(T * H * 2), heap.alloc(T * H * 2)]
    r_off = heap.alloc(T * H * 2)
    for it in range(5):
        xs, res, w = _make_inputs(world, T, H, 77 + it)
        off = x_offs[it % 2]
        for r in range(world):
            heap.tensor(r, off, (T, H), torch.bfloat16).copy_(xs[r])
        outs, status = emulated_allreduce(heap, off, r_off, [res] * world, w, T, H, 1e-6, "oneshot_notail")
        assert status == [0] * world
        ref_out, ref_h = reference(xs, res, w, 1e-6)
        for r in range(world):
            assert torch.equal(heap.tensor(r, r_off, (T, H), torch.bfloat16).float(), ref_h)
            torch.testing.assert_close(outs[r].float(), ref_out, atol=2e-2, rtol=2e-2)


def test_emulated_second_call_reuses_signal_words():
    """Epochs only grow: repeated calls on one heap need no flag reset."""
    import torch

    from memfabric_hybrid_b200.ops.allreduce import emulated_allreduce, reference
    from memfabric_hybrid_b200.parallel.heap import EmulatedHeap

    world, T, H = 4, 9, 2048
    heap = EmulatedHeap(world, 2 * T * H * 2 + 8192)
    x_off, r_off = heap.alloc(T * H * 2), heap.alloc(T * H * 2)
    for it in range(3):
        xs, res, w = _make_inputs(world, T, H, 77 + it)
        for r in range(world):
            heap.tensor(r, x_off, (T, H), torch.bfloat16).copy_(xs[r])
        outs, status = emulated_allreduce(heap, x_off, r_off, [res] * world, w, T, H, 1e-6, "twoshot" if it % 2 else "oneshot")
        assert status == [0] * world
        ref_out, _ = reference(xs, res, w, 1e-6)
        torch.testing.assert_close(outs[0].float(), ref_out, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("algo", ["oneshot", "twoshot"])
def test_missing_rank_times_out_with_status(algo):
    """A rank that never joins: the others give up after the limit and say who was missing; nothing hangs."""
    import torch

    from memfabric_hybrid_b200.ops.allreduce import emulated_allreduce
    from memfabric_hybrid_b200.parallel.heap import EmulatedHeap

    world, T, H = 4, 4, 1024
    xs, res, w = _make_inputs(world, T, H, 5)
    heap = EmulatedHeap(world, 2 * T * H * 2 + 8192)
    x_off, r_off = heap.alloc(T * H * 2), heap.alloc(T * H * 2)
    outs, status = emulated_allreduce(heap, x_off, r_off, [res] * world, w, T, H, 1e-6, algo, timeout_ns=50_000_000, participating=3)
    for r in range(3):
        assert status[r] & 0xFF == 1, status          # MF_DEV_ERR_TIMEOUT
        assert status[r] >> 8 == 3, status            # the peer that never arrived
    # the context is still usable
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0


def _real_rank(rank, world, port, q):
    try:
        import torch

        from memfabric_hybrid_b200.ops.allreduce import AllReduceRMSNorm, reference
        from memfabric_hybrid_b200.parallel.heap import SymmetricHeap

        torch.cuda.set_device(rank)
        heap = SymmetricHeap(rank, world, rank, 64 << 20, store_url=f"tcp://127.0.0.1:{port}")
        T, H = 300, 8192
        ar = AllReduceRMSNorm(heap, T, H)
        for algo, t in (("oneshot", 7), ("oneshot", 9), ("auto", 5), ("twoshot", 300), ("auto", 64), ("auto", 3)):
            xs, res, w = _make_inputs(world, t, H, 4242 + t)  # same seed everywhere: every rank can build the oracle
            ar.x[:t].copy_(xs[rank])
            torch.cuda.synchronize()
            heap.barrier()
            out, h = ar(t, res, w, algo=algo)
            torch.cuda.synchronize()
            assert ar.check_status() == 0
            ref_out, ref_h = reference(xs, res, w, 1e-6)
            assert torch.equal(h.float(), ref_h), f"{algo}: residual differs"
            torch.testing.assert_close(out.float(), ref_out, atol=2e-2, rtol=2e-2)
            heap.barrier()
        heap.close()
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        import traceback

        traceback.print_exc()
        q.put((rank, repr(e)))


def test_real_ranks_one_per_gpu():
    import torch

    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    ps = [ctx.Process(target=_real_rank, args=(r, world, port, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = sorted(q.get(timeout=300) for _ in ps)
    for p in ps:
        p.join(timeout=60)
    assert res == [(r, "ok") for r in range(world)], res


@pytest.mark.parametrize("algo", ["oneshot", "twoshot"])
def test_emulated_ranks_replayed_from_a_cuda_graph(algo):
    """Device-resident epochs: the launch is captured once and replayed with new inputs; the flags must order every replay
    (a frozen epoch would let a replay run through on the flags of the previous one and read half-written inputs)."""
    import torch

    from memfabric_hybrid_b200.ops.allreduce import EmulatedAllReduce, reference
    from memfabric_hybrid_b200.parallel.heap import EmulatedHeap

    world, T, H, eps = 4, 24, 4096, 1e-6
    xs, res, w = _make_inputs(world, T, H, 77)
    heap = EmulatedHeap(world, 2 * T * H * 2 + 8192)
    x_off, r_off = heap.alloc(T * H * 2), heap.alloc(T * H * 2)
    op = EmulatedAllReduce(heap, x_off, r_off, [res] * world, w, T, H, eps, algo)
    for r in range(world):
        heap.tensor(r, x_off, (T, H), torch.bfloat16).copy_(xs[r])
    op.launch()  # plain launch first (also warms the function up before capture)
    torch.cuda.synchronize()
    ref_out, _ = reference(xs, res, w, eps)
    torch.testing.assert_close(op.outs[0].float(), ref_out, atol=2e-2, rtol=2e-2)
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            op.launch(stream=side)
            op.launch(stream=side)
    torch.cuda.synchronize()
    first = int(op.epoch_state[0, 0])
    for it in range(3):
        xs2, _, _ = _make_inputs(world, T, H, 500 + it)
        for r in range(world):
            heap.tensor(r, x_off, (T, H), torch.bfloat16).copy_(xs2[r])
        graph.replay()
        torch.cuda.synchronize()
        assert op.status.cpu().tolist() == [0] * world
        ref_out, _ = reference(xs2, res, w, eps)
        for r in range(world):
            torch.testing.assert_close(op.outs[r].float(), ref_out, atol=2e-2, rtol=2e-2)
    # every rank counted every call: one plain launch, then three replays of two
    assert op.epoch_state[:, 0].cpu().tolist() == [first + 6] * world and op.epoch_state[:, 1].cpu().tolist() == [0] * world


def _graph_rank(rank, world, port, q):
    try:
        import torch

        from memfabric_hybrid_b200.ops.allreduce import AllReduceRMSNorm, reference
        from memfabric_hybrid_b200.parallel.heap import SymmetricHeap

        torch.cuda.set_device(rank)
        heap = SymmetricHeap(rank, world, rank, 64 << 20, store_url=f"tcp://127.0.0.1:{port}")
        T, H = 8, 8192
        ar = AllReduceRMSNorm(heap, T, H, device_epochs=True)
        xs, res, w = _make_inputs(world, T, H, 99)
        bufs = [ar.x]
        ar.x.copy_(xs[rank])
        torch.cuda.synchronize()
        heap.barrier()
        ar(T, res, w)  # warm-up calls outside the graph: argument blocks are uploaded, both input buffers seen
        bufs.append(ar.x)
        ar.x.copy_(xs[rank])
        torch.cuda.synchronize()
        heap.barrier()
        ar(T, res, w)
        torch.cuda.synchronize()
        heap.barrier()
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        outs = []
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for _ in range(2):
                    o, _h = ar(T, res, w, stream=side)
                    outs.append(o.clone())
        for it in range(3):
            xs2, _, _ = _make_inputs(world, T, H, 1000 + it)
            for b in bufs:
                b.copy_(xs2[rank])
            torch.cuda.synchronize()
            heap.barrier()
            graph.replay()
            torch.cuda.synchronize()
            assert ar.check_status() == 0
            ref_out, _ = reference(xs2, res, w, 1e-6)
            for o in outs:
                torch.testing.assert_close(o.float(), ref_out, atol=2e-2, rtol=2e-2)
            heap.barrier()
        heap.close()
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        import traceback

        traceback.print_exc()
        q.put((rank, repr(e)))


def test_real_ranks_replay_a_captured_graph():
    import torch

    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    ps = [ctx.Process(target=_graph_rank, args=(r, world, port, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = sorted(q.get(timeout=300) for _ in ps)
    for p in ps:
        p.join(timeout=60)
    assert res == [(r, "ok") for r in range(world)], res
