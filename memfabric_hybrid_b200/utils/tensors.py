"""Zero-copy torch views over global virtual addresses (pooled HBM of any rank, pooled pinned DRAM)."""
from __future__ import annotations

import ctypes

import numpy as np


class _CudaBlob:
    """Minimal __cuda_array_interface__ provider for a raw device-visible address."""

    def __init__(self, addr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,),
            "typestr": "|u1",
            "data": (addr, False),
            "version": 3,
            "strides": None,
        }


def device_tensor_from_gva(addr: int, nbytes: int, dtype=None, device=None):
    """uint8 (or `dtype`) CUDA tensor aliasing [addr, addr+nbytes). The memory is owned by the pool, not by torch."""
    import torch

    t = torch.as_tensor(_CudaBlob(addr, nbytes), device=device if device is not None else torch.device("cuda", torch.cuda.current_device()))
    if dtype is not None and dtype != torch.uint8:
        t = t.view(dtype)
    return t


def host_array_from_gva(addr: int, nbytes: int) -> np.ndarray:
    """uint8 numpy array aliasing pooled host DRAM (valid on CPU-only ranks too)."""
    buf = (ctypes.c_uint8 * nbytes).from_address(addr)
    return np.frombuffer(buf, dtype=np.uint8)
