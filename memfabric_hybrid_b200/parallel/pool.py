"""One-call bring-up of a Big Memory pool for a torchrun-style job (one process per GPU)."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

from .. import _loader  # noqa: F401  (loads the native module)
from .. import bm, get_last_err_msg

MiB = 1 << 20
GRANULE = 2 * MiB


def env_rank_world():
    """(rank, local_rank, world) from torchrun's environment, defaulting to a single process."""
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    return rank, local, world


def default_store_url(offset: int = 37) -> str:
    """tcp://MASTER_ADDR:(MASTER_PORT + offset): a port next to torch.distributed's own rendezvous."""
    host = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MF_STORE_PORT", int(os.environ.get("MASTER_PORT", "29500")) + offset))
    return f"tcp://{host}:{port}"


@dataclass
class Pool:
    handle: "bm.BigMemory"
    rank: int
    world: int
    hbm_bytes: int
    dram_bytes: int

    def hbm(self, rank: Optional[int] = None) -> int:
        """GVA of `rank`'s HBM window (this rank by default)."""
        return self.handle.peer_rank_ptr(bm.BmMemType.DEVICE, self.rank if rank is None else rank)

    def dram(self, rank: Optional[int] = None) -> int:
        return self.handle.peer_rank_ptr(bm.BmMemType.HOST, self.rank if rank is None else rank)

    def close(self) -> None:
        self.handle.destroy()
        bm.uninitialize()


def open_pool(rank: int, world: int, device: int, hbm_bytes: int, dram_bytes: int = 0, store_url: Optional[str] = None,
              pool_id: int = 0, timeout_s: int = 120) -> Pool:
    """bm.initialize → bm.create → join. `device` < 0 opens a CPU-only (DRAM) rank. Sizes are rounded up to 2 MiB."""
    hbm_bytes = (hbm_bytes + GRANULE - 1) // GRANULE * GRANULE
    dram_bytes = (dram_bytes + GRANULE - 1) // GRANULE * GRANULE
    cfg = bm.BmConfig()
    cfg.rank_id = rank
    cfg.start_store = True
    cfg.init_timeout = timeout_s
    cfg.create_timeout = timeout_s
    cfg.operation_timeout = timeout_s
    rc = bm.initialize(store_url or default_store_url(), world, device, cfg)
    if rc != 0:
        raise RuntimeError(f"bm.initialize failed ({rc}): {get_last_err_msg()}")
    op = bm.BmDataOpType.SDMA if device >= 0 else bm.BmDataOpType.HOST_RDMA
    # DRAM slices of GPU ranks are placed on the GPU's own NUMA node (flag bits 0-6 = 0x7F): host legs then stay local.
    flags = 0x7F if device >= 0 and dram_bytes > 0 else 0
    handle = bm.create(pool_id, dram_bytes, hbm_bytes if device >= 0 else 0, op, flags, dram_bytes, hbm_bytes)
    rc = handle.join()
    if rc != 0:
        raise RuntimeError(f"bm.join failed ({rc}): {get_last_err_msg()}")
    return Pool(handle, rank, world, hbm_bytes, dram_bytes)
