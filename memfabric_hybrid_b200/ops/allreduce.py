"""Fused all-reduce + residual add + RMSNorm (tensor-parallel epilogue) on the symmetric heap.

    ar = AllReduceRMSNorm(heap, max_tokens, hidden)
    ar.x[:T].copy_(partial)                      # or have the producing GEMM write straight into ar.x
    out, new_residual = ar(T, residual, weight)  # every rank calls with the same T

`ar.x` is the input buffer of the NEXT call: by default there are two, used alternately (`double_buffer=True`), which lets the
small-input (one-shot) algorithm drop its closing cross-rank barrier — a rank rewrites a buffer two calls later at the earliest,
when every peer has long passed the opening barrier of the call in between. Fetch `ar.x` anew before every call. With
`double_buffer=False` there is one buffer (half the heap space) and the one-shot algorithm keeps its closing barrier.

`out = RMSNorm(residual + sum_r x_r) * weight`, `new_residual = residual + sum_r x_r`, both bf16 [T, hidden]. The kernel
(csrc/kernels/mf_allreduce.cu) picks one-shot / two-shot / NVLS by size unless `algo` is given.

CUDA graphs: with `device_epochs=True` the epoch that orders the cross-rank flags lives in device memory and is advanced by the
kernel itself, so calls may be captured into a graph and replayed (a decode step is typically one graph). Every rank must
use the same setting, the op then owns its signal channel, and with two input buffers a captured sequence must contain an
even number of calls (the buffers alternate per call, a replay must start on the buffer the capture started on).
"""
from __future__ import annotations

from typing import Optional

from .. import _loader  # noqa: F401
from .._loader import _pymf

_ops = _pymf.ops
ALGOS = {"auto": _ops.AR_AUTO, "oneshot": _ops.AR_ONESHOT, "twoshot": _ops.AR_TWOSHOT, "nvls": _ops.AR_NVLS,
         "oneshot_notail": _ops.AR_ONESHOT_NOTAIL}
ONESHOT_MAX_BYTES = 512 << 10


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
    def __init__(self, heap, max_tokens: int, hidden: int, eps: float = 1e-6, channel: int = 0, timeout_ns: int = 0, double_buffer: bool = True,
                 device_epochs: bool = False):
        import torch

        if hidden % 8 != 0 or hidden > 16384:
            raise ValueError("hidden must be a multiple of 8 and at most 16384")
        self.heap, self.max_tokens, self.hidden, self.eps = heap, max_tokens, hidden, eps
        self.channel, self.timeout_ns = channel, timeout_ns
        nbytes = max_tokens * hidden * 2
        self.double_buffer = double_buffer
        self._x_offs = [heap.alloc(nbytes) for _ in range(2 if double_buffer else 1)]
        self.res_off = heap.alloc(nbytes)
        self._xs = [heap.tensor(off, (max_tokens, hidden), torch.bfloat16) for off in self._x_offs]
        self._cur = 0
        self.x_off = self._x_offs[0]
        self.residual_out = heap.tensor(self.res_off, (max_tokens, hidden), torch.bfloat16)
        dev = self._xs[0].device
        self.out = torch.empty(max_tokens, hidden, dtype=torch.bfloat16, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self._args = [torch.empty(_ops.ALLREDUCE_ARGS_BYTES, dtype=torch.uint8, device=dev) for _ in range(2)]
        self._args_key = [None, None]
        self.launches = 0
        self.device_epochs = device_epochs
        self._epoch_state = None
        if device_epochs:
            # [0] = epoch of the last finished call, [1] = CTAs of the running call that have retired. Starts at the channel's
            # current host-side epoch (the same number on every rank), so that flags left by earlier host-epoch calls are stale.
            self._epoch_state = torch.tensor([heap.next_epoch(channel), 0], dtype=torch.int64, device=dev)

    @property
    def x(self):
        """Input buffer of the next call (bf16 [max_tokens, hidden])."""
        return self._xs[self._cur]

    def _pack(self, residual, weight):
        import torch

        c = self._cur
        key = (residual.data_ptr() if residual is not None else 0, weight.data_ptr())
        if key != self._args_key[c]:
            blob = _ops.pack_allreduce_args(self.heap.meta_ptr, self._xs[c].data_ptr(), key[0], key[1], self.residual_out.data_ptr(),
                                            self.out.data_ptr(), self.status.data_ptr(),
                                            self._epoch_state.data_ptr() if self._epoch_state is not None else 0)
            self._args[c].copy_(torch.frombuffer(bytearray(blob), dtype=torch.uint8), non_blocking=False)
            self._args_key[c] = key
        return self._args[c].data_ptr()

    def __call__(self, tokens: int, residual, weight, algo: str = "auto", ctas: int = 0, stream=None):
        import torch

        if tokens > self.max_tokens:
            raise ValueError("tokens exceeds max_tokens")
        a = ALGOS[algo]
        nbytes = tokens * self.hidden * 2
        if a == _ops.AR_AUTO:
            if nbytes <= ONESHOT_MAX_BYTES:
                a = _ops.AR_ONESHOT_NOTAIL if self.double_buffer else _ops.AR_ONESHOT
            elif self.heap.multicast_ptr and self.heap.world > 2:
                a = _ops.AR_NVLS  # in-switch reduction pays from three ranks on (measured: with two, plain peer loads are faster)
            else:
                a = _ops.AR_TWOSHOT
        elif a == _ops.AR_ONESHOT and self.double_buffer:
            a = _ops.AR_ONESHOT_NOTAIL  # inputs alternate between two buffers (see the module docstring): the closing barrier is not needed
        elif a == _ops.AR_ONESHOT_NOTAIL and not self.double_buffer:
            raise ValueError("oneshot_notail needs double_buffer=True")
        if a == _ops.AR_NVLS and not self.heap.multicast_ptr:
            raise RuntimeError("the NVLS algorithm needs a heap created with nvls=True on a platform with multicast")
        args = self._pack(residual, weight)
        s = stream or torch.cuda.current_stream()
        epoch = 0 if self.device_epochs else self.heap.next_epoch(self.channel)
        rc = _ops.allreduce_rmsnorm(args, 1, self.heap.world, tokens, self.hidden, self.eps, a, self.channel, epoch, self.timeout_ns, ctas, s.cuda_stream)
        if rc != 0:
            raise RuntimeError(f"allreduce_rmsnorm launch failed ({rc})")
        self.launches += 1
        if self.double_buffer:
            self._cur = 1 - self._cur
        return self.out[:tokens], self.residual_out[:tokens]

    def check_status(self) -> int:
        """Synchronises and returns the device status word (0 = fine, else MF_DEV_ERR_* | peer << 8)."""
        return int(self.status.item())


class EmulatedAllReduce:
    """All ranks of an EmulatedHeap as ONE cooperative launch with device-resident epochs: `launch()` may be called any number
    of times and captured into a CUDA graph (the epochs advance on the device). Inputs are read from the heap at `xs_off` of
    every rank, outputs land in `outs[r]`."""

    def __init__(self, eheap, xs_off: int, res_out_off: int, residuals, weight, tokens: int, hidden: int, eps: float, algo: str, channel: int = 1):
        import torch

        self.eheap, self.tokens, self.hidden, self.eps, self.algo, self.channel = eheap, tokens, hidden, eps, ALGOS[algo], channel
        world = eheap.world
        self.outs = [torch.zeros(tokens, hidden, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        self.status = torch.zeros(world, dtype=torch.int32, device="cuda")
        self.epoch_state = torch.zeros(world, 2, dtype=torch.int64, device="cuda")
        self.epoch_state[:, 0] = eheap.next_epoch(channel)
        blob = b""
        for r in range(world):
            rk = eheap.ranks[r]
            blob += _ops.pack_allreduce_args(rk.meta_ptr, rk.addr(xs_off), residuals[r].data_ptr() if residuals is not None else 0, weight.data_ptr(),
                                             rk.addr(res_out_off), self.outs[r].data_ptr(), self.status.data_ptr() + 4 * r,
                                             self.epoch_state.data_ptr() + 16 * r)
        self.args = torch.frombuffer(bytearray(blob), dtype=torch.uint8).cuda()
        self._keep = (residuals, weight)

    def launch(self, stream=None):
        import torch

        s = stream or torch.cuda.current_stream()
        rc = _ops.allreduce_rmsnorm(self.args.data_ptr(), self.eheap.world, self.eheap.world, self.tokens, self.hidden, self.eps, self.algo,
                                    self.channel, 0, 0, 0, s.cuda_stream)
        if rc != 0:
            raise RuntimeError(f"allreduce_rmsnorm launch failed ({rc})")


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
