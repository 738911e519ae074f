"""tcgen05 grouped block-scaled FP8 GEMM and the row quantiser against plain PyTorch fp32 references."""
import pytest

pytestmark = pytest.mark.gpu


def _groups(counts, device):
    import torch

    offs, cur = [], 0
    for c in counts:
        offs.append(cur)
        cur += (c + 127) // 128 * 128
    offs.append(cur)
    return torch.tensor(offs, dtype=torch.int32, device=device), torch.tensor(counts, dtype=torch.int32, device=device), cur


def test_quant_rows_matches_torch():
    import torch

    from memfabric_hybrid_b200.ops import fp8_gemm as F

    g = torch.Generator(device="cuda").manual_seed(1)
    x = (torch.randn(300, 7168, generator=g, device="cuda") * 3).to(torch.bfloat16)
    x[5, 128:256] = 0  # an all-zero block must not divide by zero
    q, s = F.quant_rows_fp8(x)
    q_ref, s_ref = F.quant_act_torch(x)
    torch.cuda.synchronize()
    torch.testing.assert_close(s, s_ref, rtol=1e-6, atol=0)
    # one fp8 step of slack where the division rounds differently
    diff = (F.dequant_act(q, s) - F.dequant_act(q_ref, s_ref)).abs()
    assert float(diff.max()) <= float(s.max()) * 32 + 1e-6
    assert float((q.float() != q_ref.float()).float().mean()) < 1e-3


@pytest.mark.parametrize("counts,N,K", [([128], 128, 128), ([128], 128, 256), ([128], 256, 512), ([1], 128, 128), ([200, 0, 37, 128], 256, 1024),
                                        ([5, 17, 300, 64, 1, 129, 0, 255], 512, 2048),
                                        # large row counts take the two-SM (cta_group::2) kernel: 256-wide tiles over CTA pairs
                                        ([512], 256, 256), ([256], 256, 128), ([700, 256, 1], 512, 1024), ([1000, 130, 257, 640], 768, 2048)])
def test_grouped_gemm_matches_reference(counts, N, K):
    import torch

    from memfabric_hybrid_b200.ops import fp8_gemm as F

    dev = "cuda"
    offs, cnts, rows = _groups(counts, dev)
    g = torch.Generator(device=dev).manual_seed(sum(counts) + N + K)
    a = torch.randn(rows, K, generator=g, device=dev)
    w = torch.randn(len(counts), N, K, generator=g, device=dev) * 0.05
    a_q, a_s = F.quant_act_torch(a)
    w_q, w_s = F.quant_weight_torch(w)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.full((rows, N), float("nan"), dtype=torch.bfloat16, device=dev)
    two_sm = N % 256 == 0 and rows >= 192 * len(counts)  # the CTA-pair kernel is exercised on the large cases
    F.grouped_gemm(a_q, a_s, w_q, w_s, offs, cnts, out=out, status=status, two_sm=two_sm)
    torch.cuda.synchronize()
    assert int(status) == 0
    ref = F.grouped_gemm_reference(a_q, a_s, w_q, w_s, offs, cnts)
    o, c = offs.tolist(), cnts.tolist()
    for gi in range(len(counts)):
        got = out[o[gi]:o[gi] + c[gi]].float()
        exp = ref[o[gi]:o[gi] + c[gi]]
        if c[gi] > 0:
            torch.testing.assert_close(got, exp, rtol=2e-2, atol=2e-2 * float(exp.abs().max() + 1e-6))
        # padding rows are never written
        pad = out[o[gi] + c[gi]:o[gi + 1]]
        assert bool(torch.isnan(pad.float()).all()) or pad.numel() == 0


@pytest.mark.parametrize("big_counts", [None, [600, 257, 300]])
def test_grouped_gemm_swiglu_epilogue(big_counts):
    import torch

    from memfabric_hybrid_b200.ops import fp8_gemm as F

    dev = "cuda"
    counts, I, K = big_counts or [70, 130, 3], 256, 512
    offs, cnts, rows = _groups(counts, dev)
    g = torch.Generator(device=dev).manual_seed(9)
    a = torch.randn(rows, K, generator=g, device=dev)
    wg = torch.randn(len(counts), I, K, generator=g, device=dev) * 0.05
    wu = torch.randn(len(counts), I, K, generator=g, device=dev) * 0.05
    w = F.interleave_gate_up(wg, wu)
    a_q, a_s = F.quant_act_torch(a)
    w_q, w_s = F.quant_weight_torch(w)
    out = F.grouped_gemm(a_q, a_s, w_q, w_s, offs, cnts, mode="swiglu", two_sm=big_counts is not None)
    torch.cuda.synchronize()
    ref = F.grouped_gemm_reference(a_q, a_s, w_q, w_s, offs, cnts, mode="swiglu")
    # cross-check the interleaved layout against the textbook formula on the dequantised, de-interleaved weights
    wd = F.dequant_weight(w_q, w_s).view(len(counts), I // 32, 2, 32, K)
    ad = F.dequant_act(a_q, a_s)
    o, c = offs.tolist(), cnts.tolist()
    for gi in range(len(counts)):
        rows_a = ad[o[gi]:o[gi] + c[gi]]
        gate = rows_a @ wd[gi, :, 0].reshape(I, K).T
        up = rows_a @ wd[gi, :, 1].reshape(I, K).T
        textbook = torch.nn.functional.silu(gate) * up
        torch.testing.assert_close(ref[o[gi]:o[gi] + c[gi]], textbook, rtol=1e-4, atol=1e-4)
        got = out[o[gi]:o[gi] + c[gi]].float()
        torch.testing.assert_close(got, textbook, rtol=2e-2, atol=2e-2 * float(textbook.abs().max() + 1e-6))
