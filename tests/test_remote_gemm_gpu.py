"""K2 remote GEMM (tcgen05) against a plain PyTorch fp32 matmul."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 256), (1024, 1024, 1024), (384, 768, 4096)])
@pytest.mark.parametrize("pull", [False, True, "warps"])
def test_gemm_matches_fp32(cuda_device, m, n, k, pull):
    """One CTA per 128 x 256 tile; X in place, copied by CTAs that compute afterwards, or by two warps of every CTA."""
    from execution_ucx_b200.ops.remote_gemm import RemoteGemm
    torch.manual_seed(m + n + k)
    x = torch.randn(m, k, device=cuda_device).to(torch.bfloat16)
    w = (torch.randn(k, n, device=cuda_device) * 0.02).to(torch.bfloat16)
    g = RemoteGemm(w, m)
    y = torch.zeros(m, n, dtype=torch.bfloat16, device=cuda_device)
    done = torch.zeros(1, dtype=torch.int64, device=cuda_device)
    for rnd in range(2):  # scratch (panel flags, counters) must come back clean
        y.zero_()
        g(x.data_ptr(), m, y.data_ptr(), x_is_local=not pull, done_flag_ptr=done.data_ptr(), done_value=rnd + 1,
          copy_ctas=3 if pull else 0, copy_warps=pull == "warps", cta_pairs=False)
        torch.cuda.synchronize()
        g.check_status()
        assert int(done.item()) == rnd + 1
        ref = x.float() @ w.float()
        torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
        if pull:
            assert torch.equal(g.x_stage[:m].view(torch.int16), x.view(torch.int16))
        assert int(g.panel_flags.sum()) == 0 and int(g.sched.sum()) == 0


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (256, 384, 512), (512, 1024, 4096)])
@pytest.mark.parametrize("pull", [False, True, "warps"])
def test_block_scaled_fp8_matches_fp32(cuda_device, m, n, k, pull):
    from execution_ucx_b200.ops import remote_gemm as rg
    torch.manual_seed(m * 3 + n + k)
    x = torch.randn(m, k, device=cuda_device)
    w = torch.randn(k, n, device=cuda_device) * 0.02
    g = rg.RemoteGemmFp8(w, m)
    xq, xs = rg.quantize_rows_1x128(x)
    y = torch.zeros(m, n, dtype=torch.bfloat16, device=cuda_device)
    done = torch.zeros(1, dtype=torch.int64, device=cuda_device)
    for rnd in range(2):
        y.zero_()
        g(xq.data_ptr(), xs.data_ptr(), m, y.data_ptr(), x_is_local=not pull, done_flag_ptr=done.data_ptr(), done_value=rnd + 1,
          copy_ctas=2 if pull else 0, copy_warps=pull == "warps")
        torch.cuda.synchronize()
        g.check_status()
        assert int(done.item()) == rnd + 1
        ref = rg.dequantized_reference(xq, xs, g.w_q_t, g.w_scale)
        # the kernel differs from the reference only by fp32 summation order and the bf16 output rounding
        torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
        # and the quantised product stays close to the unquantised one
        if pull:
            assert torch.equal(g.x_scale_stage[:m], xs)
        full = x @ w
        assert float((y.float() - full).abs().max()) < 0.15 * float(full.abs().max()) + 0.05
        assert int(g.panel_flags.sum()) == 0 and int(g.sched.sum()) == 0


@pytest.mark.parametrize("pull", [False, True, "warps"])
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (512, 768, 1024), (1024, 512, 2048), (5120, 512, 128)])
def test_bf16_cta_pairs(cuda_device, m, n, k, pull):
    """The kernel that computes 256 x 256 tiles on pairs of CTAs (tcgen05 cta_group::2) against fp32 PyTorch,
    with X read in place, with X streamed in by copying pairs that then join the GEMM, and with X
    streamed in by two warps of every CTA."""
    from execution_ucx_b200.ops.remote_gemm import RemoteGemm
    torch.manual_seed(m + n + k)
    x = torch.randn(m, k, device=cuda_device).to(torch.bfloat16)
    w = (torch.randn(k, n, device=cuda_device) * 0.02).to(torch.bfloat16)
    g = RemoteGemm(w, m)
    y = torch.zeros(m, n, dtype=torch.bfloat16, device=cuda_device)
    done = torch.zeros(1, dtype=torch.int64, device=cuda_device)
    for call in range(2):      # twice: the scratch counters are left clean
        g(x.data_ptr(), m, y.data_ptr(), x_is_local=not pull, cta_pairs=True, done_flag_ptr=done.data_ptr(), done_value=call + 1,
          copy_ctas=4 if pull else 0, copy_warps=pull == "warps")
        torch.cuda.synchronize()
        g.check_status()
        assert int(done.item()) == call + 1
        torch.testing.assert_close(y.float(), x.float() @ w.float(), rtol=2e-2, atol=2e-2)
        if pull:
            assert torch.equal(g.x_stage[:m].view(torch.int16), x.view(torch.int16))
        assert int(g.panel_flags.sum()) == 0 and int(g.sched.sum()) == 0
        y.zero_()


@pytest.mark.parametrize("pull", [False, True, "warps"])
@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (512, 768, 1024), (1024, 512, 4096)])
def test_mxfp8_cta_pairs(cuda_device, m, n, k, pull):
    """MXFP8 (e4m3 with a power-of-two scale per 32 elements, scaled inside tcgen05.mma) against the fp32
    product of the dequantised operands, and loosely against the unquantised product."""
    from execution_ucx_b200.ops import remote_gemm as rg
    torch.manual_seed(m + 5 * n + k)
    # block magnitudes spread over several powers of two, so that a wrong or misplaced scale shows
    x = torch.randn(m, k, device=cuda_device) * torch.exp2(torch.randint(-3, 4, (m, k // 32), device=cuda_device).float()).repeat_interleave(32, 1)
    w = torch.randn(k, n, device=cuda_device) * 0.02 * torch.exp2(torch.randint(-2, 3, (k // 32, n), device=cuda_device).float()).repeat_interleave(32, 0)
    g = rg.RemoteGemmMx(w, m)
    xq, xsf = rg.quantize_mx(x)
    xc = rg.mx_scale_chunks(xsf, False)
    y = torch.zeros(m, n, dtype=torch.bfloat16, device=cuda_device)
    done = torch.zeros(1, dtype=torch.int64, device=cuda_device)
    ref = rg.mx_dequantized_reference(xq, xsf, g.w_q_t, g.w_sf)
    for rnd in range(2):
        y.zero_()
        g(xq.data_ptr(), xc.data_ptr(), m, y.data_ptr(), x_is_local=not pull, done_flag_ptr=done.data_ptr(), done_value=rnd + 1,
          copy_ctas=4 if pull else 0, copy_warps=pull == "warps")
        torch.cuda.synchronize()
        g.check_status()
        assert int(done.item()) == rnd + 1
        torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2 * float(ref.abs().max()) / 8)
        if pull:
            assert torch.equal(g.x_scale_stage[: xc.numel()], xc)
        full = x @ w
        assert float((y.float() - full).abs().max()) < 0.1 * float(full.abs().max())
        assert int(g.panel_flags.sum()) == 0 and int(g.sched.sum()) == 0
