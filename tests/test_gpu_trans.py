"""Transfer engine on a GPU: a "prefill" process writes tensors into a "decode" process's registered torch tensors by their
addresses in that process (CUDA IPC mapping under the hood), batch and stream-ordered variants, read-back. Mirrors the
reference's demo (example/trans/demo/test_transfer_engine.py) with a byte-exact check."""
import multiprocessing as mp

import pytest

from conftest import free_port

pytestmark = pytest.mark.gpu


def _decode(port, q_addr, q_done):
    try:
        import torch

        import memfabric_hybrid_b200 as mf

        torch.cuda.set_device(0)
        e = mf.TransferEngine()
        assert e.initialize(f"tcp://127.0.0.1:{port}", "127.0.0.1:7002", "Decode", 0) == 0, mf.get_last_err_msg()
        kv = torch.zeros(10, 1 << 20, dtype=torch.float16, device="cuda")  # ten "layers"
        torch.cuda.synchronize()
        assert e.register_memory(kv.data_ptr(), kv.numel() * 2) == 0, mf.get_last_err_msg()
        q_addr.put((kv.data_ptr(), kv.numel() * 2))
        assert q_done.get(timeout=120) == "written"
        torch.cuda.synchronize()
        for i in range(10):
            g = torch.Generator(device="cuda").manual_seed(100 + i)
            exp = torch.randn(1 << 20, generator=g, device="cuda").to(torch.float16)
            assert torch.equal(kv[i], exp), f"layer {i} differs"
        kv.mul_(2)
        torch.cuda.synchronize()
        q_addr.put("doubled")
        assert q_done.get(timeout=120) == "bye"
        assert e.unregister_memory(kv.data_ptr()) == 0
        e.unInitialize()
        q_addr.put("ok")
    except Exception as ex:  # pragma: no cover
        import traceback

        traceback.print_exc()
        q_addr.put(repr(ex))


def test_prefill_writes_decode_tensors(mf):
    import torch

    port = free_port()
    url = f"tcp://127.0.0.1:{port}"
    assert mf.create_config_store(url) == 0
    ctx = mp.get_context("spawn")
    q_addr, q_done = ctx.Queue(), ctx.Queue()
    p = ctx.Process(target=_decode, args=(port, q_addr, q_done))
    p.start()
    try:
        got = q_addr.get(timeout=120)
        assert isinstance(got, tuple), got
        peer, nbytes = got
        torch.cuda.set_device(0)
        e = mf.TransferEngine()
        assert e.initialize(url, "127.0.0.1:7001", "Prefill", 0) == 0, mf.get_last_err_msg()
        layers = []
        for i in range(10):
            g = torch.Generator(device="cuda").manual_seed(100 + i)
            layers.append(torch.randn(1 << 20, generator=g, device="cuda").to(torch.float16))
        torch.cuda.synchronize()
        per = (1 << 20) * 2
        # layers 0-4 one by one, 5-8 as one batch, 9 on a stream
        for i in range(5):
            assert e.transfer_sync_write("127.0.0.1:7002", layers[i].data_ptr(), peer + i * per, per) == 0, mf.get_last_err_msg()
        assert e.batch_transfer_sync_write("127.0.0.1:7002", [layers[i].data_ptr() for i in range(5, 9)], [peer + i * per for i in range(5, 9)],
                                           [per] * 4) == 0, mf.get_last_err_msg()
        s = torch.cuda.Stream()
        assert e.transfer_async_write_submit("127.0.0.1:7002", layers[9].data_ptr(), peer + 9 * per, per, s.cuda_stream) == 0
        s.synchronize()
        q_done.put("written")
        assert q_addr.get(timeout=120) == "doubled"
        back = torch.empty(1 << 20, dtype=torch.float16, device="cuda")
        assert e.transfer_sync_read("127.0.0.1:7002", back.data_ptr(), peer + 3 * per, per) == 0, mf.get_last_err_msg()
        assert torch.equal(back, layers[3] * 2)
        assert e.transfer_sync_write("127.0.0.1:7002", back.data_ptr(), peer + nbytes - 16, 4096) != 0  # leaves the registration
        q_done.put("bye")
        assert q_addr.get(timeout=120) == "ok"
        e.unInitialize()
    finally:
        p.join(timeout=60)
        if p.is_alive():
            p.terminate()
        mf.destroy_config_store(url)
