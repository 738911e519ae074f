"""Block-scaled FP8 helpers and the grouped expert GEMM (tcgen05 kernel in csrc/kernels/mf_moe_gemm_sm100.cu).

Quantisation follows the DeepSeek-V3 recipe: activations e4m3 with one fp32 scale per (row, 128 columns); weights e4m3 with
one fp32 scale per 128 x 128 block; scale = amax / 448.
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
                 two_sm: bool = False):
    """out[rows of group g] = dequant(a)[rows] @ dequant(b[g]).T  (bf16), optionally with the SwiGLU epilogue.

    a_q [R, K] e4m3, a_scale [R, K/128], b_q [G, N, K] e4m3, b_scale [G, N/128, K/128], group_offset int32 [G+1] (starts are
    multiples of 128), group_count int32 [G] — both on the device. two_sm=True runs the CTA-pair (cta_group::2) variant, which
    needs N % 256 == 0."""
    import torch

    R, K = a_q.shape
    G, N, K2 = b_q.shape
    assert K == K2 and a_q.is_contiguous() and b_q.is_contiguous() and a_scale.is_contiguous() and b_scale.is_contiguous()
    epi = _ops.GEMM_EPI_SWIGLU if mode == "swiglu" else _ops.GEMM_EPI_BF16
    n_out = N // 2 if mode == "swiglu" else N
    out = out if out is not None else torch.empty(R, n_out, dtype=torch.bfloat16, device=a_q.device)
    s = stream or torch.cuda.current_stream()
    rc = _ops.moe_grouped_gemm(a_q.data_ptr(), a_scale.data_ptr(), b_q.data_ptr(), b_scale.data_ptr(), out.data_ptr(), group_offset.data_ptr(),
                               group_count.data_ptr(), G, R, N, K, epi, status.data_ptr() if status is not None else 0, -2 if two_sm else ctas,
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
