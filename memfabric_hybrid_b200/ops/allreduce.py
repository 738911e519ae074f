"""Fused all-reduce + residual add + RMSNorm (tensor-parallel epilogue) on the symmetric heap.

    ar = AllReduceRMSNorm(heap, max_tokens, hidden)
    ar.x[:T].copy_(partial)                      # or have the producing GEMM write straight into ar.x
    out, new_residual = ar(T, residual, weight)  # every rank calls with the same T

`out = RMSNorm(residual + sum_r x_r) * weight`, `new_residual = residual + sum_r x_r`, both bf16 [T, hidden]. The kernel
(csrc/kernels/mf_allreduce.cu) picks one-shot / two-shot / NVLS by size unless `algo` is given.
"""
from __future__ import annotations

from typing import Optional

from .. import _loader  # noqa: F401
from .._loader import _pymf

_ops = _pymf.ops
ALGOS = {"auto": _ops.AR_AUTO, "oneshot": _ops.AR_ONESHOT, "twoshot": _ops.AR_TWOSHOT, "nvls": _ops.AR_NVLS}


def reference(xs, residual, weight, eps: float):
    """Plain PyTorch fp32 oracle. xs: list of per-rank [T, H] tensors."""
    import torch

    h = sum(x.float() for x in xs)
    if residual is not None:
        h = h + residual.float()
    h = h.to(torch.bfloat16).float()
    out = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return out, h


class AllReduceRMSNorm:
    def __init__(self, heap, max_tokens: int, hidden: int, eps: float = 1e-6, channel: int = 0, timeout_ns: int = 0):
        import torch

        if hidden % 8 != 0 or hidden > 16384:
            raise ValueError("hidden must be a multiple of 8 and at most 16384")
        self.heap, self.max_tokens, self.hidden, self.eps = heap, max_tokens, hidden, eps
        self.channel, self.timeout_ns = channel, timeout_ns
        nbytes = max_tokens * hidden * 2
        self.x_off = heap.alloc(nbytes)
        self.res_off = heap.alloc(nbytes)
        self.x = heap.tensor(self.x_off, (max_tokens, hidden), torch.bfloat16)
        self.residual_out = heap.tensor(self.res_off, (max_tokens, hidden), torch.bfloat16)
        self.out = torch.empty(max_tokens, hidden, dtype=torch.bfloat16, device=self.x.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.x.device)
        self._args = torch.empty(_ops.ALLREDUCE_ARGS_BYTES, dtype=torch.uint8, device=self.x.device)
        self._args_key = None
        self.launches = 0

    def _pack(self, residual, weight):
        import torch

        key = (residual.data_ptr() if residual is not None else 0, weight.data_ptr())
        if key != self._args_key:
            blob = _ops.pack_allreduce_args(self.heap.meta_ptr, self.x.data_ptr(), key[0], key[1], self.residual_out.data_ptr(),
                                            self.out.data_ptr(), self.status.data_ptr())
            self._args.copy_(torch.frombuffer(bytearray(blob), dtype=torch.uint8), non_blocking=False)
            self._args_key = key
        return self._args.data_ptr()

    def __call__(self, tokens: int, residual, weight, algo: str = "auto", ctas: int = 0, stream=None):
        import torch

        if tokens > self.max_tokens:
            raise ValueError("tokens exceeds max_tokens")
        a = ALGOS[algo]
        if a == _ops.AR_AUTO and self.heap.multicast_ptr and tokens * self.hidden * 2 > (512 << 10):
            a = _ops.AR_NVLS
        if a == _ops.AR_NVLS and not self.heap.multicast_ptr:
            raise RuntimeError("the NVLS algorithm needs a heap created with nvls=True on a platform with multicast")
        args = self._pack(residual, weight)
        s = stream or torch.cuda.current_stream()
        epoch = self.heap.next_epoch(self.channel)
        rc = _ops.allreduce_rmsnorm(args, 1, self.heap.world, tokens, self.hidden, self.eps, a, self.channel, epoch, self.timeout_ns, ctas, s.cuda_stream)
        if rc != 0:
            raise RuntimeError(f"allreduce_rmsnorm launch failed ({rc})")
        self.launches += 1
        return self.out[:tokens], self.residual_out[:tokens]

    def check_status(self) -> int:
        """Synchronises and returns the device status word (0 = fine, else MF_DEV_ERR_* | peer << 8)."""
        return int(self.status.item())


def emulated_allreduce(eheap, xs_off: int, res_out_off: int, residuals, weight, tokens: int, hidden: int, eps: float, algo: str,
                       timeout_ns: int = 0, ctas: int = 0, participating: Optional[int] = None):
    """Runs all ranks of an EmulatedHeap in one cooperative launch. Returns (outs, status) with one output per rank.
    `participating` < world launches only the first ranks, which makes the others' flags never arrive: the waits run out
    and the status word reports the timeout (used to test the bounded-wait path without hanging anything)."""
    import torch

    world = eheap.world
    n = world if participating is None else participating
    outs = [torch.zeros(tokens, hidden, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    status = torch.zeros(world, dtype=torch.int32, device="cuda")
    blob = b""
    for r in range(n):
        rk = eheap.ranks[r]
        blob += _ops.pack_allreduce_args(rk.meta_ptr, rk.addr(xs_off), residuals[r].data_ptr() if residuals is not None else 0, weight.data_ptr(),
                                         rk.addr(res_out_off), outs[r].data_ptr(), status.data_ptr() + 4 * r)
    args = torch.frombuffer(bytearray(blob), dtype=torch.uint8).cuda()
    epoch = eheap.next_epoch(0)
    rc = _ops.allreduce_rmsnorm(args.data_ptr(), n, world, tokens, hidden, eps, ALGOS[algo], 0, epoch, timeout_ns, ctas,
                                torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise RuntimeError(f"allreduce_rmsnorm launch failed ({rc})")
    torch.cuda.synchronize()
    return outs, status.cpu().tolist()
