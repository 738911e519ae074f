"""Symmetric heap for torch programs.

``SymmetricHeap`` brings up a Share Memory object (``shm.initialize`` + ``shm.create``) for a one-process-per-GPU job and
hands out tensors that sit at the same heap offset on every rank, which is what the fused kernels in
``memfabric_hybrid_b200.ops`` need: a rank reads or writes a peer's copy of a tensor with plain loads/stores over NVLink.

``EmulatedHeap`` lays out R "ranks" inside one GPU's memory with the same meta records and signal areas. Kernels are then
run for all R ranks as slices of ONE cooperative launch, which is how the multi-rank logic is tested on a single GPU.
"""
from __future__ import annotations

import struct
from typing import List, Optional

from .. import _loader  # noqa: F401
from .. import get_last_err_msg, shm
from .pool import default_store_url

MiB = 1 << 20
GRANULE = 2 * MiB
SIGNAL_BYTES = 2 * MiB
META_BYTES = 128


def _round_up(v: int, a: int) -> int:
    return (v + a - 1) // a * a


class _Bump:
    def __init__(self, size: int):
        self.size = size
        self.used = 0

    def alloc(self, nbytes: int, align: int = 256) -> int:
        off = _round_up(self.used, align)
        if off + nbytes > self.size:
            raise MemoryError(f"symmetric heap exhausted: need {nbytes} at {off}, size {self.size}")
        self.used = off + nbytes
        return off


class SymmetricHeap:
    """One rank's view of a symmetric heap shared by `world` ranks (collective constructor)."""

    def __init__(self, rank: int, world: int, device: int, size_bytes: int, store_url: Optional[str] = None, heap_id: int = 0,
                 nvls: bool = False, timeout_s: int = 120):
        import torch

        self.rank, self.world, self.device = rank, world, device
        self.size = _round_up(size_bytes, GRANULE)
        cfg = shm.ShmConfig()
        cfg.init_timeout = cfg.create_timeout = cfg.operation_timeout = timeout_s
        rc = shm.initialize(store_url or default_store_url(41), world, rank, device, cfg)
        if rc != 0:
            raise RuntimeError(f"shm.initialize failed ({rc}): {get_last_err_msg()}")
        op = int(shm.ShmDataOpType.MTE) | int(shm.ShmDataOpType.SDMA) | (int(shm.ShmDataOpType.RDMA) if nvls else 0)
        self.handle = shm.create(heap_id, world, rank, self.size, op, 0)
        self.gva = self.handle.gva
        self.meta_ptr = self.handle.device_meta
        self.multicast_ptr = self.handle.multicast_ptr
        self._bump = _Bump(self.size)
        self._torch = torch

    # ---- allocation (call in the same order on every rank)
    def alloc(self, nbytes: int, align: int = 256) -> int:
        return self._bump.alloc(nbytes, align)

    def addr(self, offset: int, rank: Optional[int] = None) -> int:
        return self.gva + (self.rank if rank is None else rank) * self.size + offset

    def tensor(self, offset: int, shape, dtype, rank: Optional[int] = None):
        """Tensor view of heap offset `offset` on `rank` (default: this rank). Peer views work over NVLink for torch ops too."""
        from ..utils.tensors import device_tensor_from_gva

        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * self._torch.empty(0, dtype=dtype).element_size()
        return device_tensor_from_gva(self.addr(offset, rank), nbytes, dtype).view(*shape)

    def empty(self, shape, dtype):
        """(offset, tensor) of a new symmetric allocation."""
        numel = 1
        for s in shape:
            numel *= s
        off = self.alloc(numel * self._torch.empty(0, dtype=dtype).element_size())
        return off, self.tensor(off, shape, dtype)

    def next_epoch(self, channel: int = 0) -> int:
        return self.handle.next_epoch(channel)

    def set_check_bounds(self, on: bool = True) -> None:
        """Kernels validate their heap arguments before touching a peer (debug aid; also MF_CHECK_BOUNDS=1 in the environment)."""
        rc = self.handle.set_debug_flags(1 if on else 0)
        if rc != 0:
            raise RuntimeError(f"set_debug_flags failed ({rc}): {get_last_err_msg()}")

    def barrier(self) -> None:
        rc = self.handle.barrier()
        if rc != 0:
            raise RuntimeError(f"shm barrier failed ({rc}): {get_last_err_msg()}")

    def close(self) -> None:
        self.handle.destroy()
        shm.uninitialize()


class _EmulatedRank:
    def __init__(self, parent: "EmulatedHeap", rank: int):
        self.parent, self.rank, self.world = parent, rank, parent.world
        self.size = parent.size
        self.gva = parent.gva
        self.meta_ptr = parent.meta_base + rank * META_BYTES
        self.multicast_ptr = 0

    def addr(self, offset: int, rank: Optional[int] = None) -> int:
        return self.gva + (self.rank if rank is None else rank) * self.size + offset

    def tensor(self, offset: int, shape, dtype, rank: Optional[int] = None):
        return self.parent.tensor(self.rank if rank is None else rank, offset, shape, dtype)


class EmulatedHeap:
    """R ranks' heaps, signal areas and meta records inside one GPU (tests and single-GPU development only)."""

    def __init__(self, world: int, size_bytes: int, device: int = 0, check_bounds: bool = False):
        """check_bounds sets the debug bit in every emulated rank's meta record: kernels then validate their heap arguments
        before they touch a peer and report an error code instead of reaching outside the heap."""
        import torch

        self.world = world
        self.size = _round_up(size_bytes, 4096)
        self._heap = torch.zeros(world * self.size, dtype=torch.uint8, device=f"cuda:{device}")
        self._signal = torch.zeros(world * SIGNAL_BYTES, dtype=torch.uint8, device=f"cuda:{device}")
        self.gva = self._heap.data_ptr()
        metas = b""
        for r in range(world):
            metas += struct.pack("<4I7Q7Q", 0, r, world, 0, self.size, self.gva, 0, 0, self._signal.data_ptr(), 0, 0, 1 if check_bounds else 0,
                                 *([0] * 6))
        assert len(metas) == world * META_BYTES
        self._meta = torch.frombuffer(bytearray(metas), dtype=torch.uint8).to(f"cuda:{device}")
        self.meta_base = self._meta.data_ptr()
        self._bump = _Bump(self.size)
        self._epochs = {}
        self.ranks: List[_EmulatedRank] = [_EmulatedRank(self, r) for r in range(world)]
        self._torch = torch

    def alloc(self, nbytes: int, align: int = 256) -> int:
        return self._bump.alloc(nbytes, align)

    def tensor(self, rank: int, offset: int, shape, dtype):
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * self._torch.empty(0, dtype=dtype).element_size()
        lo = rank * self.size + offset
        return self._heap[lo:lo + nbytes].view(dtype).view(*shape)

    def next_epoch(self, channel: int = 0) -> int:
        self._epochs[channel] = self._epochs.get(channel, 0) + 1
        return self._epochs[channel]
