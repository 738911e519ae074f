"""Prefill → Decode tensor transfer with the TransferEngine (counterpart of the reference's
example/trans/demo/test_transfer_engine.py). Start a store, then the two roles in two shells (or GPUs):

    python -m memfabric_hybrid_b200.launch_store tcp://127.0.0.1:7766 &
    python examples/python/transfer_engine_demo.py decode  tcp://127.0.0.1:7766 0 /tmp/mf_demo_addr
    python examples/python/transfer_engine_demo.py prefill tcp://127.0.0.1:7766 0 /tmp/mf_demo_addr
"""
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import memfabric_hybrid_b200 as mf  # noqa: E402

role, url, dev, addr_file = sys.argv[1], sys.argv[2], int(sys.argv[3]), sys.argv[4]
torch.cuda.set_device(dev)
e = mf.TransferEngine()
if role == "decode":
    assert e.initialize(url, "127.0.0.1:9102", "Decode", dev) == 0, mf.get_last_err_msg()
    kv = torch.zeros(10, 1 << 20, dtype=torch.float16, device="cuda")
    assert e.register_memory(kv.data_ptr(), kv.numel() * 2) == 0
    with open(addr_file, "w") as f:
        f.write(str(kv.data_ptr()))
    while float(kv[9, -1]) == 0.0:
        time.sleep(0.05)
    print("decode received:", [float(kv[i, 0]) for i in range(10)])
else:
    assert e.initialize(url, "127.0.0.1:9101", "Prefill", dev) == 0, mf.get_last_err_msg()
    while not os.path.exists(addr_file):
        time.sleep(0.05)
    time.sleep(0.2)
    peer = int(open(addr_file).read())
    tensors = [torch.full((1 << 20,), float(i + 1), dtype=torch.float16, device="cuda") for i in range(10)]
    torch.cuda.synchronize()
    per = (1 << 20) * 2
    rc = e.batch_transfer_sync_write("127.0.0.1:9102", [t.data_ptr() for t in tensors], [peer + i * per for i in range(10)], [per] * 10)
    print("prefill wrote 10 tensors, rc =", rc)
e.unInitialize()
