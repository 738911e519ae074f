"""Big Memory from Python, one process per GPU (torchrun sets RANK/WORLD_SIZE/LOCAL_RANK):

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/python/bm_example.py

Each rank writes a tensor into its pooled HBM, copies it to the next rank's pooled HBM and DRAM through the GVA, and reads
back what the previous rank left (counterpart of the reference's example/bm/BmPython/smem_bm_example.py)."""
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import memfabric_hybrid_b200 as mf  # noqa: E402
from memfabric_hybrid_b200.parallel.pool import env_rank_world, open_pool  # noqa: E402
from memfabric_hybrid_b200.utils.tensors import device_tensor_from_gva, host_array_from_gva  # noqa: E402

rank, local, world = env_rank_world()
torch.cuda.set_device(local)
pool = open_pool(rank, world, local, hbm_bytes=64 << 20, dram_bytes=64 << 20)
while pool.handle.joined_size() != world:
    time.sleep(0.01)
nxt, prv = (rank + 1) % world, (rank - 1) % world
n = 4 << 20
mine = device_tensor_from_gva(pool.hbm(), n, torch.float32)          # a torch view of my pooled HBM
mine.fill_(float(rank))
torch.cuda.synchronize()
T = mf.bm.BmCopyType
assert pool.handle.copy_data(pool.hbm(), pool.hbm(nxt) + n, n, T.G2G, 0) == 0, mf.get_last_err_msg()   # HBM → peer HBM
assert pool.handle.copy_data(pool.hbm(), pool.dram(nxt), n, T.G2G, 0) == 0, mf.get_last_err_msg()      # HBM → peer DRAM
time.sleep(1.0)
got_hbm = device_tensor_from_gva(pool.hbm() + n, n, torch.float32)
got_dram = host_array_from_gva(pool.dram(), n).view("float32")
print(f"rank {rank}: HBM holds {got_hbm[0].item()} and DRAM holds {got_dram[0]} from rank {prv}")
assert got_hbm[0].item() == float(prv) and got_dram[-1] == float(prv)
time.sleep(0.5)
pool.close()
