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
    F.grouped_gemm(a_q, a_s, w_q, w_s, offs, cnts, out=out, status=status)
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
    out = F.grouped_gemm(a_q, a_s, w_q, w_s, offs, cnts, mode="swiglu")
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


# ---------------------------------------------------------------------------------------------- block-scaled tensor-core path (UE8M0 scales)


def _mx_cases():
    base = [([128], 256, 128), ([128], 256, 512), ([1], 256, 384), ([200, 0, 37, 128], 256, 1024), ([5, 17, 300, 64, 1, 129, 0, 255], 512, 2048),
            ([700, 256, 1], 512, 1024), ([1000, 130, 257, 640], 768, 2048)]
    cases = [(c, n, k, t) for (c, n, k) in base for t in (128, 256)]
    # 224-column tiles (two accumulators, a tile spans up to three 128-column weight blocks): N must be a multiple of 896
    cases += [([128], 896, 128, 224), ([1, 300, 0, 129], 896, 1024, 224), ([700, 256, 1, 64], 1792, 2048, 224)]
    # the two-SM kernel (tile_n 512 = 256 x 256 tiles by CTA pairs): row counts around the 128- and 256-row boundaries
    cases += [([256], 256, 128, 512), ([128], 256, 512, 512), ([1], 256, 384, 512), ([200, 0, 37, 128, 257], 512, 1024, 512),
              ([1000, 130, 257, 640], 768, 2048, 512)]
    return cases


@pytest.mark.parametrize("counts,N,K,tile_n", _mx_cases())
def test_grouped_gemm_mx_matches_reference(counts, N, K, tile_n):
    import torch

    from memfabric_hybrid_b200.ops import fp8_gemm as F

    dev = "cuda"
    offs, cnts, rows = _groups(counts, dev)
    g = torch.Generator(device=dev).manual_seed(sum(counts) + N + K)
    # rows of very different magnitude, so that a misplaced scale factor (wrong row, wrong K block) cannot hide
    a = torch.randn(rows, K, generator=g, device=dev) * torch.exp2(torch.randint(-6, 7, (rows, 1), generator=g, device=dev).float())
    a = a * torch.exp2(torch.randint(-3, 4, (1, K // 128), generator=g, device=dev).float()).repeat_interleave(128, dim=1)
    w = torch.randn(len(counts), N, K, generator=g, device=dev) * 0.05
    w = w * torch.exp2(torch.randint(-4, 5, (len(counts), N // 128, 1, K // 128, 1), generator=g, device=dev).float()).expand(
        -1, -1, 128, -1, 128).reshape(len(counts), N, K)
    a_q, a_sf = F.quant_act_mx_torch(a)
    w_q, w_s = F.quant_weight_mx_torch(w)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.full((rows, N), float("nan"), dtype=torch.bfloat16, device=dev)
    F.grouped_gemm_mx(a_q, a_sf, w_q, w_s, offs, cnts, out=out, status=status, tile_n=tile_n)
    torch.cuda.synchronize()
    assert int(status) == 0
    ref = F.grouped_gemm_mx_reference(a_q, a_sf, w_q, w_s, offs, cnts)
    o, c = offs.tolist(), cnts.tolist()
    for gi in range(len(counts)):
        got = out[o[gi]:o[gi] + c[gi]].float()
        exp = ref[o[gi]:o[gi] + c[gi]]
        if c[gi] > 0:
            # per row: rows differ by orders of magnitude
            tol = 2e-2 * exp.abs().amax(dim=1, keepdim=True) + 1e-6
            assert bool(((got - exp).abs() <= tol).all()), f"group {gi}: {float(((got - exp).abs() / tol).max())}"
        pad = out[o[gi] + c[gi]:o[gi + 1]]
        assert bool(torch.isnan(pad.float()).all()) or pad.numel() == 0  # padding rows are never written


@pytest.mark.parametrize("tile_n", [128, 256])
@pytest.mark.parametrize("counts", [[70, 130, 3], [600, 257, 300]])
def test_grouped_gemm_mx_swiglu_and_fused_quant(counts, tile_n):
    import torch

    from memfabric_hybrid_b200.ops import fp8_gemm as F

    dev = "cuda"
    I, K = 256, 512
    offs, cnts, rows = _groups(counts, dev)
    g = torch.Generator(device=dev).manual_seed(9)
    a = torch.randn(rows, K, generator=g, device=dev)
    wg = torch.randn(len(counts), I, K, generator=g, device=dev) * 0.05
    wu = torch.randn(len(counts), I, K, generator=g, device=dev) * 0.05
    a_q, a_sf = F.quant_act_mx_torch(a)
    w_q, w_s = F.quant_weight_mx_torch(F.interleave_gate_up(wg, wu))
    out = F.grouped_gemm_mx(a_q, a_sf, w_q, w_s, offs, cnts, mode="swiglu", tile_n=tile_n)
    hq, hsf = F.grouped_gemm_mx(a_q, a_sf, w_q, w_s, offs, cnts, mode="swiglu_fp8", tile_n=tile_n)
    torch.cuda.synchronize()
    ref = F.grouped_gemm_mx_reference(a_q, a_sf, w_q, w_s, offs, cnts, mode="swiglu")
    ref_q, ref_sf = F.grouped_gemm_mx_reference(a_q, a_sf, w_q, w_s, offs, cnts, mode="swiglu_fp8")
    o, c = offs.tolist(), cnts.tolist()
    for gi in range(len(counts)):
        sl = slice(o[gi], o[gi] + c[gi])
        exp = ref[sl]
        torch.testing.assert_close(out[sl].float(), exp, rtol=2e-2, atol=2e-2 * float(exp.abs().max() + 1e-6))
        # fused quantisation: scale bytes agree except where fp32 summation order moves an amax across a power of two, and the
        # dequantised values agree to an e4m3 step
        same = (hsf[sl] == ref_sf[sl]).float().mean()
        assert float(same) > 0.99, float(same)
        assert int((hsf[sl].int() - ref_sf[sl].int()).abs().max()) <= 1
        got = F.dequant_act_mx(hq[sl], hsf[sl])
        err = (got - ref_q[sl]).abs()
        assert float(err.max()) <= 0.13 * float(exp.abs().max()) + 1e-6
        assert float(err.mean()) <= 5e-3 * float(exp.abs().max())


def _arrival_counters(offs, cnts, rows, device):
    import torch

    arrive = torch.zeros(rows // 128, dtype=torch.int32, device=device)
    for off, n in zip(offs.tolist(), cnts.tolist()):
        for mt in range((n + 127) // 128):
            arrive[off // 128 + mt] = min(128, n - 128 * mt)
    return arrive


@pytest.mark.parametrize("tile_n", [128, 256])
def test_gated_gemm_runs_on_complete_counters_and_gives_up_on_a_missing_tile(tile_n):
    """The GEMM whose tiles wait for arrival counters: complete counters → the ordinary result; one tile whose counter stays
    short → every wait is bounded, the status word names the arrival wait and the context stays usable."""
    import torch

    from memfabric_hybrid_b200.ops import fp8_gemm as F
    from memfabric_hybrid_b200._loader import _pymf

    dev = "cuda"
    counts, N, K = [300, 0, 129, 64], 512, 1024
    offs, cnts, rows = _groups(counts, dev)
    g = torch.Generator(device=dev).manual_seed(77)
    a_q, a_sf = F.quant_act_mx_torch(torch.randn(rows, K, generator=g, device=dev))
    w_q, w_s = F.quant_weight_mx_torch(torch.randn(len(counts), N, K, generator=g, device=dev) * 0.05)
    arrive = _arrival_counters(offs, cnts, rows, dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = F.grouped_gemm_mx(a_q, a_sf, w_q, w_s, offs, cnts, status=status, tile_n=tile_n, arrive=arrive, wait_ns=200_000_000)
    torch.cuda.synchronize()
    assert int(status) == 0
    ref = F.grouped_gemm_mx_reference(a_q, a_sf, w_q, w_s, offs, cnts)
    for off, n in zip(offs.tolist(), cnts.tolist()):
        if n:
            exp = ref[off:off + n]
            assert bool(((out[off:off + n].float() - exp).abs() <= 2e-2 * exp.abs().amax(dim=1, keepdim=True) + 1e-6).all())
    # nothing ever completes the second tile of the first group
    arrive[1] -= 1
    F.grouped_gemm_mx(a_q, a_sf, w_q, w_s, offs, cnts, status=status, tile_n=tile_n, arrive=arrive, wait_ns=20_000_000)
    torch.cuda.synchronize()
    assert int(status) == _pymf.ops.GEMM_ARRIVAL_EXPIRED
    assert float((torch.ones(4, device=dev) + 1).sum()) == 8.0  # the context is alive
    # a status that is already set (a failed dispatch) turns the waits off: the call returns at once
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    F.grouped_gemm_mx(a_q, a_sf, w_q, w_s, offs, cnts, status=status, tile_n=tile_n, arrive=arrive, wait_ns=1_000_000_000)
    t1.record()
    torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 100.0


@pytest.mark.parametrize("tile_n,N", [(128, 512), (256, 512), (224, 896), (0, 7168)])
def test_packed_weights_give_the_same_result(tile_n, N):
    """Weights re-ordered into 4 KiB blocks (pack_weight_mx) are the same operand: the outputs match bit for bit."""
    import torch

    from memfabric_hybrid_b200.ops import fp8_gemm as F

    dev = "cuda"
    counts, K = [200, 0, 37, 129], 1024
    offs, cnts, rows = _groups(counts, dev)
    g = torch.Generator(device=dev).manual_seed(5 + N)
    a_q, a_sf = F.quant_act_mx_torch(torch.randn(rows, K, generator=g, device=dev))
    w_q, w_s = F.quant_weight_mx_torch(torch.randn(len(counts), N, K, generator=g, device=dev) * 0.05)
    w_p = F.pack_weight_mx(w_q)
    assert w_p.shape == (len(counts), N // 32, K // 128, 32, 128) and torch.equal(F.unpack_weight_mx(w_p).view(torch.uint8), w_q.view(torch.uint8))
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    modes = ["bf16"] if tile_n == 224 else ["bf16", "swiglu_fp8"]
    for mode in modes:
        ref = F.grouped_gemm_mx(a_q, a_sf, w_q, w_s, offs, cnts, mode=mode, status=status, tile_n=tile_n)
        got = F.grouped_gemm_mx(a_q, a_sf, w_p, w_s, offs, cnts, mode=mode, status=status, tile_n=tile_n)
        torch.cuda.synchronize()
        assert int(status) == 0
        pairs = zip(ref, got) if mode == "swiglu_fp8" else [(ref, got)]
        for r, o in pairs:
            for off, n in zip(offs.tolist(), cnts.tolist()):
                assert torch.equal(r[off:off + n].view(torch.uint8), o[off:off + n].view(torch.uint8))
