"""Weight reshard for RL: FSDP flat shards (training) → tensor-parallel inference layout, optional fp8 cast, one kernel.

    plan = ReshardPlan(specs, world, tp_rank, tp_size, fp8=True)      # pure Python, no GPU needed
    rs = Resharder(heap, plan)                                        # collective: allocates the shard in the heap
    rs.shard.copy_(my_flat_shard)                                     # training side writes its FSDP shard
    weights = rs()                                                    # dict name -> tensor (bf16, or (fp8, scales))

The flat vector is every parameter in `specs` order, each padded to a multiple of 8 elements, cut into `world` equal shards
(the last one zero-padded). `reference_reshard` is the PyTorch oracle (all-gather + slice + cast).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

from .. import _loader  # noqa: F401
from .._loader import _pymf
from ..models.llama import ParamSpec, tp_block

_ops = _pymf.ops
CH_RESHARD = 4


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


@dataclass
class PlanEntry:
    spec: ParamSpec
    src_off: int      # element offset in the flat vector
    r0: int
    c0: int
    nrows: int
    ncols: int
    cols_full: int
    dst_off: int      # byte offset in the destination buffer
    scale_off: int    # float offset in the scale buffer
    quant: bool
    tile_start: int


class ReshardPlan:
    def __init__(self, specs: List[ParamSpec], world: int, tp_rank: int, tp_size: int, fp8: bool = False):
        self.specs, self.world, self.tp_rank, self.tp_size, self.fp8 = specs, world, tp_rank, tp_size, fp8
        off = 0
        self.flat_offsets: Dict[str, int] = {}
        for s in specs:
            self.flat_offsets[s.name] = off
            off += _pad8(s.numel)
        self.total_elems = off
        self.shard_elems = _pad8((off + world - 1) // world)
        self.entries: List[PlanEntry] = []
        dst, sc, tiles = 0, 0, 0
        for s in specs:
            r0, c0, nr, nc, cf = tp_block(s, tp_rank, tp_size)
            if cf % 8 or c0 % 8 or nc % 8:
                raise ValueError(f"{s.name}: column extents must be multiples of 8 elements")
            q = bool(fp8 and s.quantizable and nr % 128 == 0 and nc % 128 == 0)
            self.entries.append(PlanEntry(s, self.flat_offsets[s.name], r0, c0, nr, nc, cf, dst, sc, q, tiles))
            dst += _pad8(nr * nc) * (1 if q else 2)
            dst = (dst + 255) // 256 * 256
            if q:
                sc += (nr // 128) * (nc // 128)
            tiles += ((nr + 127) // 128) * ((nc + 255) // 256)  # kernel tiles: 128 rows x 256 columns
        self.dst_bytes, self.scale_floats, self.total_tiles = dst, sc, tiles

    def table_bytes(self) -> bytes:
        return b"".join(_ops.pack_reshard_desc(e.src_off, e.dst_off, e.scale_off, e.cols_full, e.r0, e.c0, e.nrows, e.ncols, e.tile_start, int(e.quant))
                        for e in self.entries)

    def bytes_pulled(self) -> int:
        """Source bytes this destination reads (bf16)."""
        return sum(e.nrows * e.ncols * 2 for e in self.entries)


class Resharder:
    def __init__(self, heap, plan: ReshardPlan, timeout_ns: int = 0, shard=None):
        """`shard` = (offset, tensor) of another Resharder over the same source layout: both then read the same heap buffer
        (e.g. a bf16 and an fp8 destination of one training shard)."""
        import torch

        self.heap, self.plan, self.timeout_ns = heap, plan, timeout_ns
        dev = torch.device("cuda", torch.cuda.current_device())
        self.shard_off, self.shard = shard if shard is not None else heap.empty((plan.shard_elems,), torch.bfloat16)
        if self.shard.numel() != plan.shard_elems:
            raise ValueError("the shared shard does not match this plan's shard size")
        self.dst = torch.empty(plan.dst_bytes, dtype=torch.uint8, device=dev)
        self.scales = torch.empty(max(plan.scale_floats, 1), dtype=torch.float32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.table = torch.frombuffer(bytearray(plan.table_bytes()), dtype=torch.uint8).to(dev)
        blob = _ops.pack_reshard_args(heap.meta_ptr, self.shard.data_ptr(), self.dst.data_ptr(), self.scales.data_ptr(), self.table.data_ptr(),
                                      self.status.data_ptr(), plan.shard_elems, len(plan.entries), plan.total_tiles)
        self.args = torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(dev)
        self.launches = 0

    def launch(self, stream=None, ctas: int = 0):
        import torch

        s = stream or torch.cuda.current_stream()
        rc = _ops.reshard(self.args.data_ptr(), 1, self.heap.world, CH_RESHARD, self.heap.next_epoch(CH_RESHARD), self.timeout_ns, ctas, s.cuda_stream)
        if rc != 0:
            raise RuntimeError(f"reshard launch failed ({rc})")
        self.launches += 1

    def views(self):
        """name -> bf16 tensor, or (float8_e4m3fn tensor, fp32 scales [rows/128, cols/128]) for quantised parameters."""
        import torch

        out = {}
        for e in self.plan.entries:
            shape = (e.ncols,) if len(e.spec.shape) == 1 else (e.nrows, e.ncols)
            n = e.nrows * e.ncols
            if e.quant:
                w = self.dst[e.dst_off:e.dst_off + n].view(torch.float8_e4m3fn).view(*shape)
                sc = self.scales[e.scale_off:e.scale_off + (e.nrows // 128) * (e.ncols // 128)].view(e.nrows // 128, e.ncols // 128)
                out[e.spec.name] = (w, sc)
            else:
                out[e.spec.name] = self.dst[e.dst_off:e.dst_off + 2 * n].view(torch.bfloat16).view(*shape)
        return out

    def __call__(self, stream=None):
        self.launch(stream)
        return self.views()

    def check_status(self) -> int:
        return int(self.status.item())


def reference_reshard(flat, plan: ReshardPlan):
    """Oracle: slice the full flat vector (as an all-gather would produce it) and cast with PyTorch."""
    from .fp8_gemm import quant_weight_torch

    out = {}
    for e in plan.entries:
        full = flat[e.src_off:e.src_off + e.spec.numel]
        if len(e.spec.shape) == 1:
            out[e.spec.name] = full.clone()
            continue
        blk = full.view(*e.spec.shape)[e.r0:e.r0 + e.nrows, e.c0:e.c0 + e.ncols].contiguous()
        out[e.spec.name] = quant_weight_torch(blk) if e.quant else blk
    return out


def emulated_reshard(eheap, plans: List[ReshardPlan], shard_off: int, timeout_ns: int = 0, participating: Optional[int] = None):
    """All destination ranks of an EmulatedHeap in one cooperative launch. Returns per-rank (dst, scales, status)."""
    import torch

    world = eheap.world
    n = world if participating is None else participating
    keep, blob = [], b""
    for r in range(n):
        p, rk = plans[r], eheap.ranks[r]
        dst = torch.empty(p.dst_bytes, dtype=torch.uint8, device="cuda")
        sc = torch.empty(max(p.scale_floats, 1), dtype=torch.float32, device="cuda")
        st = torch.zeros(1, dtype=torch.int32, device="cuda")
        tb = torch.frombuffer(bytearray(p.table_bytes()), dtype=torch.uint8).cuda()
        keep.append((dst, sc, st, tb))
        blob += _ops.pack_reshard_args(rk.meta_ptr, rk.addr(shard_off), dst.data_ptr(), sc.data_ptr(), tb.data_ptr(), st.data_ptr(), p.shard_elems,
                                       len(p.entries), p.total_tiles)
    args = torch.frombuffer(bytearray(blob), dtype=torch.uint8).cuda()
    rc = _ops.reshard(args.data_ptr(), n, world, CH_RESHARD, eheap.next_epoch(CH_RESHARD), timeout_ns, 0, torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise RuntimeError(f"reshard launch failed ({rc})")
    torch.cuda.synchronize()
    return [(k[0], k[1], int(k[2].item())) for k in keep]
