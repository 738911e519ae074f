"""Block-scaled FP8 helpers and the grouped expert GEMMs.

Two kernels share the interface:

* ``grouped_gemm_mx`` (csrc/kernels/mf_moe_gemm_mx_sm100.cu) — the product path. All scales are powers of two (UE8M0
  exponent bytes) and are applied by the tensor core itself (tcgen05.mma.kind::mxf8f6f4.block_scale): activations e4m3 with
  one scale per (row, 128 columns) on dispatch and per (row, 32 columns) for the SwiGLU output, weights e4m3 with one scale
  per 128 x 128 block; scale = 2^ceil(log2(amax / 448)).
* ``grouped_gemm`` (csrc/kernels/mf_moe_gemm_sm100.cu) — arbitrary fp32 scales (scale = amax / 448), applied per 128-wide
  K block in registers. Slower; kept for operands that were quantised elsewhere with free-form scales.
"""
from __future__ import annotations

from .. import _loader  # noqa: F401
from .._loader import _pymf

_ops = _pymf.ops
FP8_MAX = 448.0


def quant_act_torch(x):
    """Reference 1 x 128 quantisation in PyTorch. x: [M, K] (K % 128 == 0). Returns (q float8_e4m3fn [M, K], scale fp32 [M, K/128])."""
    import torch

    M, K = x.shape
    xb = x.float().view(M, K // 128, 128)
    amax = xb.abs().amax(-1).clamp_min(1e-10)
    scale = amax / FP8_MAX
    q = (xb / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(M, K)
    return q, scale.contiguous()


def quant_weight_torch(w):
    """128 x 128 block quantisation. w: [..., N, K]. Returns (q float8_e4m3fn same shape, scale fp32 [..., N/128, K/128])."""
    import torch

    *lead, N, K = w.shape
    wb = w.float().view(*lead, N // 128, 128, K // 128, 128)
    amax = wb.abs().amax(dim=(-3, -1)).clamp_min(1e-10)
    scale = amax / FP8_MAX
    q = (wb / scale.unsqueeze(-2).unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(*lead, N, K)
    return q, scale.contiguous()


def dequant_act(q, scale):
    M, K = q.shape
    return (q.float().view(M, K // 128, 128) * scale.unsqueeze(-1)).view(M, K)


def dequant_weight(q, scale):
    *lead, N, K = q.shape
    return (q.float().view(*lead, N // 128, 128, K // 128, 128) * scale.unsqueeze(-2).unsqueeze(-1)).view(*lead, N, K)


def quant_rows_fp8(x, q=None, scale=None, row_limit=None, stream=None):
    """CUDA kernel version of quant_act_torch (bf16 input). Optional preallocated outputs; row_limit: device int32 tensor."""
    import torch

    M, K = x.shape
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and K % 128 == 0
    q = q if q is not None else torch.empty(M, K, dtype=torch.float8_e4m3fn, device=x.device)
    scale = scale if scale is not None else torch.empty(M, K // 128, dtype=torch.float32, device=x.device)
    s = stream or torch.cuda.current_stream()
    rc = _ops.quant_rows_fp8(x.data_ptr(), q.data_ptr(), scale.data_ptr(), M, K, row_limit.data_ptr() if row_limit is not None else 0, s.cuda_stream)
    if rc != 0:
        raise RuntimeError(f"quant_rows_fp8 failed ({rc})")
    return q, scale


def interleave_gate_up(w_gate, w_up):
    """[..., I, K] gate and up projections → [..., 2I, K] in chunks of 64 rows = 32 gate rows followed by the 32 matching up
    rows, which is the layout the SwiGLU epilogue expects (each epilogue thread owns 64 consecutive columns of a tile)."""
    import torch

    *lead, I, K = w_gate.shape
    g = w_gate.view(*lead, I // 32, 32, K)
    u = w_up.view(*lead, I // 32, 32, K)
    return torch.cat([g, u], dim=-2).reshape(*lead, 2 * I, K).contiguous()


def grouped_gemm(a_q, a_scale, b_q, b_scale, group_offset, group_count, mode: str = "bf16", out=None, status=None, ctas: int = 0, stream=None,
                 ):
    """out[rows of group g] = dequant(a)[rows] @ dequant(b[g]).T  (bf16), optionally with the SwiGLU epilogue.

    a_q [R, K] e4m3, a_scale [R, K/128], b_q [G, N, K] e4m3, b_scale [G, N/128, K/128], group_offset int32 [G+1] (starts are
    multiples of 128), group_count int32 [G] — both on the device."""
    import torch

    R, K = a_q.shape
    G, N, K2 = b_q.shape
    assert K == K2 and a_q.is_contiguous() and b_q.is_contiguous() and a_scale.is_contiguous() and b_scale.is_contiguous()
    epi = _ops.GEMM_EPI_SWIGLU if mode == "swiglu" else _ops.GEMM_EPI_BF16
    n_out = N // 2 if mode == "swiglu" else N
    out = out if out is not None else torch.empty(R, n_out, dtype=torch.bfloat16, device=a_q.device)
    s = stream or torch.cuda.current_stream()
    rc = _ops.moe_grouped_gemm(a_q.data_ptr(), a_scale.data_ptr(), b_q.data_ptr(), b_scale.data_ptr(), out.data_ptr(), group_offset.data_ptr(),
                               group_count.data_ptr(), G, R, N, K, epi, status.data_ptr() if status is not None else 0, ctas,
                               s.cuda_stream)
    if rc != 0:
        raise RuntimeError(f"moe_grouped_gemm launch failed ({rc})")
    return out


def grouped_gemm_reference(a_q, a_scale, b_q, b_scale, group_offset, group_count, mode: str = "bf16"):
    """fp32 PyTorch oracle of grouped_gemm on the dequantised operands."""
    import torch

    a = dequant_act(a_q, a_scale)
    b = dequant_weight(b_q, b_scale)
    G, N, _ = b.shape
    n_out = N // 2 if mode == "swiglu" else N
    out = torch.zeros(a.shape[0], n_out, dtype=torch.float32, device=a.device)
    offs, cnts = group_offset.tolist(), group_count.tolist()
    for g in range(G):
        lo, n = offs[g], cnts[g]
        if n == 0:
            continue
        y = a[lo:lo + n] @ b[g].T
        if mode == "swiglu":
            y = y.view(n, N // 64, 2, 32)
            y = (torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]).reshape(n, N // 2)
        out[lo:lo + n] = y
    return out


# ---------------------------------------------------------------------------------------------- power-of-two (UE8M0) scales


def _ue8m0_ceil(t):
    """Biased exponent byte of the smallest power of two >= t (fp32 tensor, t >= 0), clamped to [1, 253] — bit for bit the rule
    of the kernels (exponent field, plus one when any mantissa bit is set)."""
    import torch

    bits = t.contiguous().view(torch.int32)
    e = ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    return e.clamp(1, 253)


def _pow2(e):
    """2^(e - 127) as fp32 for an int32 tensor of biased exponents in [1, 254]."""
    import torch

    return (e.to(torch.int32) << 23).view(torch.float32)


def quant_act_mx_torch(x, block: int = 128):
    """Reference quantisation with power-of-two scales. x: [M, K] float; one scale per (row, `block` columns), block 128 or 32.
    Returns (q float8_e4m3fn [M, K], sf uint8 [M, K/32]): the scale-factor layout of the kernels — one UE8M0 byte per 32
    columns, so a 1x128 scale appears four times (viewed as int32 [M, K/128] it is the `a_sf` operand of grouped_gemm_mx)."""
    import torch

    M, K = x.shape
    xb = x.float().view(M, K // block, block)
    amax = xb.abs().amax(-1)
    e = _ue8m0_ceil(amax * torch.tensor(1.0 / 448.0, dtype=torch.float32, device=x.device))
    inv = _pow2(254 - e)
    q = (xb * inv.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(M, K)
    sf = e.to(torch.uint8).repeat_interleave(block // 32, dim=1).contiguous()
    return q, sf


def dequant_act_mx(q, sf):
    import torch

    M, K = q.shape
    return (q.float().view(M, K // 32, 32) * _pow2(sf.to(torch.int32)).unsqueeze(-1)).view(M, K)


def quant_weight_mx_torch(w):
    """128 x 128 block quantisation with power-of-two scales. w: [..., N, K]. Returns (q float8_e4m3fn, scale fp32 [..., N/128, K/128])."""
    import torch

    *lead, N, K = w.shape
    wb = w.float().view(*lead, N // 128, 128, K // 128, 128)
    amax = wb.abs().amax(dim=(-3, -1))
    e = _ue8m0_ceil(amax * torch.tensor(1.0 / 448.0, dtype=torch.float32, device=w.device))
    scale = _pow2(e)
    q = (wb * _pow2(254 - e).unsqueeze(-2).unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(*lead, N, K)
    return q, scale.contiguous()


def pack_weight_mx(w_q):
    """Re-orders quantised weights [G, N, K] (e4m3) for streaming: [G, N/32, K/128, 32, 128], i.e. blocks of 32 rows x 128
    K-bytes stored contiguously (4 KiB). grouped_gemm_mx takes either layout (it tells them apart by the number of dimensions)
    and gives the same result; with the packed one a weight tile is read from DRAM in 4 KiB pieces instead of 128-byte
    pieces K bytes apart, which is what counts when few rows per expert make the GEMM a weight stream (decode)."""
    import torch

    G, N, K = w_q.shape
    assert N % 32 == 0 and K % 128 == 0 and w_q.is_contiguous()
    return w_q.view(torch.uint8).view(G, N // 32, 32, K // 128, 128).permute(0, 1, 3, 2, 4).contiguous().view(w_q.dtype)


def unpack_weight_mx(w_p):
    """Inverse of pack_weight_mx: [G, N/32, K/128, 32, 128] → [G, N, K]."""
    import torch

    G, nb, kb, _, _ = w_p.shape
    return w_p.view(torch.uint8).permute(0, 1, 3, 2, 4).contiguous().view(G, nb * 32, kb * 128).view(w_p.dtype)


def grouped_gemm_mx(a_q, a_sf, b_q, b_scale, group_offset, group_count, mode: str = "bf16", out=None, out_sf=None, status=None, tile_n: int = 0,
                    ctas: int = 0, stream=None, arrive=None, wait_ns: int = 0):
    """out[rows of group g] = dequant(a)[rows] @ dequant(b[g]).T on the block-scaled tensor-core path.

    a_q [R, K] e4m3; a_sf uint8 [R, K/32] (or int32 [R, K/128]); b_q [G, N, K] e4m3; b_scale fp32 powers of two [G, N/128, K/128];
    group_offset int32 [G+1] (starts are multiples of 128), group_count int32 [G], both on the device.
    mode "bf16": out bf16 [R, N]. "swiglu": out bf16 [R, N/2]. "swiglu_fp8": returns (out e4m3 [R, N/2], out_sf uint8 [R, N/64]),
    quantised per (row, 32 columns) — the a_q / a_sf of the next GEMM.
    arrive (int32 [R / 128], optional): rows of `a_q` are still being stored by other GPUs; a tile starts when the counter of
    its 128 rows has reached the tile's valid rows (each wait bounded by wait_ns, at most 1.5 s; on expiry `status` becomes
    GEMM_ARRIVAL_EXPIRED)."""
    import torch

    R, K = a_q.shape
    packed = b_q.dim() == 5  # pack_weight_mx layout
    if packed:
        G, N, K2 = b_q.shape[0], b_q.shape[1] * 32, b_q.shape[2] * 128
        assert tuple(b_q.shape[3:]) == (32, 128)
    else:
        G, N, K2 = b_q.shape
    assert K == K2 and K % 128 == 0 and a_q.is_contiguous() and b_q.is_contiguous() and a_sf.is_contiguous() and b_scale.is_contiguous()
    assert a_sf.numel() * a_sf.element_size() == R * (K // 32)
    epi = {"bf16": _ops.GEMM_EPI_BF16, "swiglu": _ops.GEMM_EPI_SWIGLU, "swiglu_fp8": _ops.GEMM_EPI_SWIGLU_FP8}[mode]
    if packed:
        epi |= _ops.GEMM_B_PACKED
    dev = a_q.device
    if mode == "bf16":
        out = out if out is not None else torch.empty(R, N, dtype=torch.bfloat16, device=dev)
    elif mode == "swiglu":
        out = out if out is not None else torch.empty(R, N // 2, dtype=torch.bfloat16, device=dev)
    else:
        out = out if out is not None else torch.empty(R, N // 2, dtype=torch.float8_e4m3fn, device=dev)
        out_sf = out_sf if out_sf is not None else torch.empty(R, N // 64, dtype=torch.uint8, device=dev)
    s = stream or torch.cuda.current_stream()
    rc = _ops.moe_grouped_gemm_mx(a_q.data_ptr(), a_sf.data_ptr(), b_q.data_ptr(), b_scale.data_ptr(), out.data_ptr(),
                                  out_sf.data_ptr() if out_sf is not None else 0, group_offset.data_ptr(), group_count.data_ptr(), G, R, N, K, epi,
                                  tile_n, status.data_ptr() if status is not None else 0, ctas, s.cuda_stream,
                                  arrive.data_ptr() if arrive is not None else 0, wait_ns)
    if rc != 0:
        raise RuntimeError(f"moe_grouped_gemm_mx launch failed ({rc})")
    return (out, out_sf) if mode == "swiglu_fp8" else out


def grouped_gemm_mx_reference(a_q, a_sf, b_q, b_scale, group_offset, group_count, mode: str = "bf16"):
    """fp32 PyTorch oracle of grouped_gemm_mx on the dequantised operands. For "swiglu_fp8" the result is quantised by the same
    rule and returned dequantised (fp32 [R, N/2]) together with the scale bytes."""
    import torch

    a = dequant_act_mx(a_q, a_sf.view(torch.uint8).view(a_q.shape[0], -1))
    b = dequant_weight(b_q, b_scale)
    G, N, _ = b.shape
    n_out = N if mode == "bf16" else N // 2
    out = torch.zeros(a.shape[0], n_out, dtype=torch.float32, device=a.device)
    offs, cnts = group_offset.tolist(), group_count.tolist()
    for g in range(G):
        lo, n = offs[g], cnts[g]
        if n == 0:
            continue
        y = a[lo:lo + n] @ b[g].T
        if mode != "bf16":
            y = y.view(n, N // 64, 2, 32)
            y = (torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]).reshape(n, N // 2)
        out[lo:lo + n] = y
    if mode == "swiglu_fp8":
        q, sf = quant_act_mx_torch(out, block=32)
        return dequant_act_mx(q, sf), sf
    return out
