"""Expert-parallel MoE layer over the symmetric heap: dispatch (fp8 quantisation with 1x128 power-of-two scales fused) →
grouped block-scaled FP8 expert FFN on tcgen05 tensor cores (scales applied by the tensor core; SwiGLU and the 1x32
re-quantisation of the intermediate fused into the first GEMM's epilogue) → combine (owner-side reduction of a token's
experts that share an owner, then the weighted top-k sum at the source).

    layer = FusedMoE(heap, max_tokens, hidden, n_experts, topk, inter, w13_q, w13_s, w2_q, w2_s)
    out = layer(x, topk_idx, topk_w)        # every rank calls; x [T, hidden] bf16, idx int32 [T, topk], w fp32 [T, topk]

`w13` holds this rank's experts' gate/up projections in the interleaved layout of ops.fp8_gemm.interleave_gate_up,
`w2` the down projections; both e4m3 with 128x128 power-of-two block scales (ops.fp8_gemm.quant_weight_mx_torch). `route()` turns router logits into (idx, renormalised w).

With ``overlap=True`` dispatch ends without its closing barrier: every row that lands is counted in a per-tile arrival counter
on the owner and the first GEMM starts each 128-row tile when its counter is complete, so an owner computes on what has arrived
while slower senders are still pushing (every pair then carries its payload over the link; without it a token crosses once per
owner and the owner replicates it).

CUDA graphs: with ``device_epochs=True`` the epochs that order the cross-rank flags of dispatch and combine live in device
memory and are advanced by the kernels themselves, so a call of the layer may be captured into a graph and replayed (call it once
eagerly with the same tensors first: the argument blocks are uploaded on first use). Every rank must use the same setting.

``EmulatedMoE`` drives the same kernels for all ranks of an ``EmulatedHeap`` on one GPU (dispatch and combine each as one
cooperative launch over all ranks; the per-rank GEMMs in between are ordinary launches) — this is how the multi-rank logic
is tested without several GPUs.
"""
from __future__ import annotations

from typing import List, Optional

from .. import _loader  # noqa: F401
from .._loader import _pymf
from . import fp8_gemm as F

_ops = _pymf.ops
CH_DISPATCH, CH_COMBINE = 2, 3


def route(logits, topk: int):
    """softmax → top-k → renormalise. Returns (idx int32 [T, k], w fp32 [T, k])."""
    import torch

    p = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(p, topk, dim=-1)
    w = w / w.sum(-1, keepdim=True)
    return idx.to(torch.int32).contiguous(), w.contiguous()


def capacity_rows(tokens: int, topk: int, ranks: int, experts_local: int, factor: float) -> int:
    """Rows of the receive buffer: `factor` times the balanced load plus the 128-row alignment slack of every expert."""
    rows = int(tokens * topk * factor) + experts_local * 128
    rows = min(rows, tokens * topk * ranks + experts_local * 128)
    return (rows + 127) // 128 * 128


class _RankState:
    """Buffers of one rank (real or emulated)."""

    def __init__(self, heap, alloc, max_tokens, hidden, n_experts, topk, inter, cap, device):
        import torch

        R = heap.world
        self.heap = heap
        self.cap = cap
        nblk = hidden // 128
        self.cnt_off = alloc(2 * R * n_experts * 4)  # two halves: calls in arrival mode alternate between them
        self.recv_x_off = alloc(cap * hidden, 1024)
        self.recv_s_off = alloc(cap * nblk * 4)
        self.recv_m_off = alloc(cap * 16)
        self.recv_sib_off = alloc(cap * _ops.MOE_MAX_SIBLINGS * 8)
        self.ret_y_off = alloc(max_tokens * topk * hidden * 2)
        self.arrive_off = alloc(cap // 128 * 4)
        self.arrive = heap.tensor(self.arrive_off, (cap // 128,), torch.int32)
        self.arrive.zero_()
        self.cnt = heap.tensor(self.cnt_off, (2, R, n_experts), torch.int32)
        self.recv_x = heap.tensor(self.recv_x_off, (cap, hidden), torch.uint8).view(torch.float8_e4m3fn)
        self.recv_s = heap.tensor(self.recv_s_off, (cap, nblk), torch.int32)  # four UE8M0 bytes per 128-column block
        self.recv_m = heap.tensor(self.recv_m_off, (cap, 4), torch.int32)
        self.recv_sib = heap.tensor(self.recv_sib_off, (cap, _ops.MOE_MAX_SIBLINGS, 2), torch.int32)
        self.ret_y = heap.tensor(self.ret_y_off, (max_tokens * topk, hidden), torch.bfloat16)
        self.cnt.zero_()
        el = n_experts // R
        self.local_cnt = torch.zeros(n_experts, dtype=torch.int32, device=device)
        self.cursor = torch.zeros(n_experts, dtype=torch.int32, device=device)
        self.expert_offset = torch.zeros(el + 1, dtype=torch.int32, device=device)
        self.expert_count = torch.zeros(el, dtype=torch.int32, device=device)
        self.send_slot = torch.zeros(max_tokens * topk, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.max_rows_ret = max_tokens * topk
        self.h1_q = torch.empty(cap, inter, dtype=torch.float8_e4m3fn, device=device)
        self.h1_sf = torch.empty(cap, inter // 32, dtype=torch.uint8, device=device)
        self.y = torch.empty(cap, hidden, dtype=torch.bfloat16, device=device)
        self.out = torch.empty(max_tokens, hidden, dtype=torch.bfloat16, device=device)


class _MoEBase:
    def __init__(self, hidden, n_experts, topk, inter, world):
        if hidden % 128 or inter % 128 or n_experts % world:
            raise ValueError("hidden and inter must be multiples of 128 and n_experts a multiple of the rank count")
        self.hidden, self.n_experts, self.topk, self.inter, self.world = hidden, n_experts, topk, inter, world
        self.el = n_experts // world
        self.launches = 0
        self.overlap = False
        self.wait_ns = 0
        # Pairs per rank from which a token crosses the link once per owner and is replicated there (0 = the kernel's threshold).
        self.dedup_min_pairs = 0

    def _experts(self, st: _RankState, w13_q, w13_s, w2_q, w2_s, stream=None):
        """The expert FFN of one rank on what dispatch delivered: GEMM1 (+SwiGLU, + 1x32 quantisation) → GEMM2."""
        rows = st.cap
        F.grouped_gemm_mx(st.recv_x, st.recv_s, w13_q, w13_s, st.expert_offset, st.expert_count, mode="swiglu_fp8", out=st.h1_q, out_sf=st.h1_sf,
                          status=st.status, stream=stream, arrive=st.arrive if self.overlap else None, wait_ns=self.wait_ns)
        F.grouped_gemm_mx(st.h1_q, st.h1_sf, w2_q, w2_s, st.expert_offset, st.expert_count, mode="bf16", out=st.y, status=st.status, stream=stream)
        self.launches += 2
        return rows


class FusedMoE(_MoEBase):
    """One rank of an expert-parallel MoE layer on a real SymmetricHeap."""

    def __init__(self, heap, max_tokens: int, hidden: int, n_experts: int, topk: int, inter: int, w13_q, w13_s, w2_q, w2_s,
                 capacity_factor: float = 2.0, timeout_ns: int = 0, overlap: bool = False, device_epochs: bool = False):
        import torch

        super().__init__(hidden, n_experts, topk, inter, heap.world)
        self.heap, self.max_tokens, self.timeout_ns = heap, max_tokens, timeout_ns
        self.overlap, self.wait_ns = overlap, min(timeout_ns, 1_500_000_000)
        self.w13_q, self.w13_s, self.w2_q, self.w2_s = w13_q, w13_s, w2_q, w2_s
        cap = capacity_rows(max_tokens, topk, heap.world, self.el, capacity_factor)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.st = _RankState(heap, heap.alloc, max_tokens, hidden, n_experts, topk, inter, cap, dev)
        self._dargs = torch.empty(_ops.MOE_DISPATCH_ARGS_BYTES, dtype=torch.uint8, device=dev)
        self._cargs = torch.empty(_ops.MOE_COMBINE_ARGS_BYTES, dtype=torch.uint8, device=dev)
        self._key = None
        self.device_epochs = device_epochs
        self._epoch_d = self._epoch_c = None
        if device_epochs:
            # {epoch of the last finished call, CTAs of the running call that have retired}, starting from the channels' host-side
            # epochs (the same numbers on every rank) so that flags left by earlier calls are stale
            self._epoch_d = torch.tensor([heap.next_epoch(CH_DISPATCH), 0], dtype=torch.int64, device=dev)
            self._epoch_c = torch.tensor([heap.next_epoch(CH_COMBINE), 0], dtype=torch.int64, device=dev)
        torch.cuda.synchronize()
        heap.barrier()  # everybody's count matrix is zeroed before the first dispatch touches it

    def _pack(self, x, idx, w, T):
        import torch

        key = (x.data_ptr(), idx.data_ptr(), w.data_ptr(), T, self.overlap, self.dedup_min_pairs)
        if key == self._key:
            return
        st, h = self.st, self.heap
        d = _ops.pack_moe_dispatch_args(h.meta_ptr, x.data_ptr(), idx.data_ptr(), w.data_ptr(), st.cnt.data_ptr(), st.recv_x.data_ptr(), st.recv_s.data_ptr(),
                                        st.recv_m.data_ptr(), st.recv_sib.data_ptr(), st.local_cnt.data_ptr(), st.cursor.data_ptr(), st.expert_offset.data_ptr(),
                                        st.expert_count.data_ptr(), st.send_slot.data_ptr(), st.status.data_ptr(), T, st.cap,
                                        st.arrive.data_ptr() if self.overlap else 0, self.dedup_min_pairs,
                                        self._epoch_d.data_ptr() if self.device_epochs else 0)
        c = _ops.pack_moe_combine_args(h.meta_ptr, st.y.data_ptr(), st.recv_m.data_ptr(), st.recv_sib.data_ptr(), st.expert_offset.data_ptr(),
                                       st.expert_count.data_ptr(), st.ret_y.data_ptr(), idx.data_ptr(), st.out.data_ptr(), st.status.data_ptr(), T,
                                       st.cap, st.max_rows_ret, self._epoch_c.data_ptr() if self.device_epochs else 0)
        self._dargs.copy_(torch.frombuffer(bytearray(d), dtype=torch.uint8))
        self._cargs.copy_(torch.frombuffer(bytearray(c), dtype=torch.uint8))
        self._key = key

    def dispatch(self, x, idx, w, stream=None):
        import torch

        T = x.shape[0]
        self._pack(x, idx, w, T)
        s = stream or torch.cuda.current_stream()
        # One warp per token: small batches get a small grid (its grid-wide barriers are cheaper), large ones every SM.
        ctas = max(1, min(1 << 16, (T + 7) // 8))
        rc = _ops.moe_dispatch(self._dargs.data_ptr(), 1, self.world, self.hidden, self.topk, self.n_experts, CH_DISPATCH,
                               0 if self.device_epochs else self.heap.next_epoch(CH_DISPATCH), self.timeout_ns, ctas, s.cuda_stream)
        if rc != 0:
            raise RuntimeError(f"moe_dispatch launch failed ({rc})")
        self.launches += 1

    def experts(self, stream=None):
        return self._experts(self.st, self.w13_q, self.w13_s, self.w2_q, self.w2_s, stream)

    def combine(self, T, stream=None):
        import torch

        s = stream or torch.cuda.current_stream()
        ctas = max(1, min(1 << 16, (T * self.topk * ((self.hidden // 8 + 127) // 128) + 7) // 8))  # one warp per 2 KiB piece of a returned row
        rc = _ops.moe_combine(self._cargs.data_ptr(), 1, self.world, self.hidden, self.topk, self.el, CH_COMBINE,
                              0 if self.device_epochs else self.heap.next_epoch(CH_COMBINE), self.timeout_ns, ctas, s.cuda_stream)
        if rc != 0:
            raise RuntimeError(f"moe_combine launch failed ({rc})")
        self.launches += 1
        return self.st.out[:T]

    def __call__(self, x, idx, w, stream=None):
        self.dispatch(x, idx, w, stream)
        self.experts(stream)
        return self.combine(x.shape[0], stream)

    def check_status(self) -> int:
        return int(self.st.status.item())


class EmulatedMoE(_MoEBase):
    """All ranks of an EmulatedHeap on one GPU. weights: per-rank lists of (w13_q, w13_s, w2_q, w2_s)."""

    def __init__(self, eheap, max_tokens, hidden, n_experts, topk, inter, weights: List[tuple], capacity_factor: float = 8.0,
                 overlap: bool = False):
        import torch

        super().__init__(hidden, n_experts, topk, inter, eheap.world)
        self.eheap, self.max_tokens, self.weights = eheap, max_tokens, weights
        self.overlap = overlap
        cap = capacity_rows(max_tokens, topk, eheap.world, self.el, capacity_factor)
        # one set of symmetric offsets, shared by every emulated rank
        offs = {}

        def alloc_once(name_holder=[0]):
            def alloc(nbytes, align=256):
                i = name_holder[0]
                name_holder[0] += 1
                if i not in offs:
                    offs[i] = eheap.alloc(nbytes, align)
                return offs[i]
            return alloc

        self.states = []
        for r in range(eheap.world):
            self.states.append(_RankState(eheap.ranks[r], alloc_once([0]), max_tokens, hidden, n_experts, topk, inter, cap, torch.device("cuda")))

    def __call__(self, xs, idxs, ws, timeout_ns: int = 0, participating: Optional[int] = None):
        import torch

        R = self.world
        n = R if participating is None else participating
        T = xs[0].shape[0]
        d, c = b"", b""
        for r in range(n):
            st, rk = self.states[r], self.eheap.ranks[r]
            d += _ops.pack_moe_dispatch_args(rk.meta_ptr, xs[r].data_ptr(), idxs[r].data_ptr(), ws[r].data_ptr(), st.cnt.data_ptr(), st.recv_x.data_ptr(),
                                             st.recv_s.data_ptr(), st.recv_m.data_ptr(), st.recv_sib.data_ptr(), st.local_cnt.data_ptr(), st.cursor.data_ptr(),
                                             st.expert_offset.data_ptr(), st.expert_count.data_ptr(), st.send_slot.data_ptr(), st.status.data_ptr(), T, st.cap,
                                             st.arrive.data_ptr() if self.overlap else 0, self.dedup_min_pairs)
            c += _ops.pack_moe_combine_args(rk.meta_ptr, st.y.data_ptr(), st.recv_m.data_ptr(), st.recv_sib.data_ptr(), st.expert_offset.data_ptr(),
                                            st.expert_count.data_ptr(), st.ret_y.data_ptr(), idxs[r].data_ptr(), st.out.data_ptr(), st.status.data_ptr(),
                                            T, st.cap, st.max_rows_ret)
        dargs = torch.frombuffer(bytearray(d), dtype=torch.uint8).cuda()
        cargs = torch.frombuffer(bytearray(c), dtype=torch.uint8).cuda()
        s = torch.cuda.current_stream().cuda_stream
        rc = _ops.moe_dispatch(dargs.data_ptr(), n, R, self.hidden, self.topk, self.n_experts, CH_DISPATCH, self.eheap.next_epoch(CH_DISPATCH), timeout_ns, 0, s)
        if rc != 0:
            raise RuntimeError(f"moe_dispatch launch failed ({rc})")
        torch.cuda.synchronize()
        status = [int(st.status.item()) for st in self.states]
        if any(status):
            return None, status
        for r in range(n):
            self._experts(self.states[r], *self.weights[r])
        rc = _ops.moe_combine(cargs.data_ptr(), n, R, self.hidden, self.topk, self.el, CH_COMBINE, self.eheap.next_epoch(CH_COMBINE), timeout_ns, 0, s)
        if rc != 0:
            raise RuntimeError(f"moe_combine launch failed ({rc})")
        torch.cuda.synchronize()
        return [self.states[r].out[:T] for r in range(n)], [int(st.status.item()) for st in self.states]


def moe_reference(xs, idxs, ws, weights, n_experts: int, inter: int):
    """fp32 PyTorch oracle of the whole layer with the same quantisation points: tokens → e4m3 (1x128 power-of-two scales), FFN1 +
    SwiGLU in fp32 on dequantised operands → e4m3 (1x32 power-of-two scales), FFN2 in fp32, bf16 rounding, weighted sum over k in fp32.
    xs/idxs/ws: per-rank inputs; weights: per-rank (w13_q, w13_s, w2_q, w2_s). Returns per-rank outputs (fp32)."""
    import torch

    R = len(xs)
    el = n_experts // R
    w13 = [F.dequant_weight(w[0], w[1]) for w in weights]
    w2 = [F.dequant_weight(w[2], w[3]) for w in weights]
    outs = []
    for r in range(R):
        x = xs[r]
        T, H = x.shape
        xq, xsf = F.quant_act_mx_torch(x)
        xd = F.dequant_act_mx(xq, xsf)
        out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
        for k in range(idxs[r].shape[1]):
            e_all = idxs[r][:, k].long()
            yk = torch.zeros(T, H, dtype=torch.float32, device=x.device)
            for e in e_all.unique().tolist():
                sel = (e_all == e).nonzero().squeeze(-1)
                owner, le = e // el, e % el
                h = xd[sel] @ w13[owner][le].T
                h = h.view(len(sel), -1, 2, 32)
                h = (torch.nn.functional.silu(h[:, :, 0]) * h[:, :, 1]).reshape(len(sel), inter)
                hq, hsf = F.quant_act_mx_torch(h, block=32)
                y = (F.dequant_act_mx(hq, hsf) @ w2[owner][le].T).to(torch.bfloat16).float()
                yk[sel] = y
            out += ws[r][:, k:k + 1].float() * yk
        outs.append(out)
    return outs
