"""K2 remote GEMM (tcgen05) against a plain PyTorch fp32 matmul."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 256), (1024, 1024, 1024), (384, 768, 4096)])
@pytest.mark.parametrize("pull", [False, True])
def test_gemm_matches_fp32(cuda_device, m, n, k, pull):
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
          copy_ctas=3 if pull else 0)
        torch.cuda.synchronize()
        g.check_status()
        assert int(done.item()) == rnd + 1
        ref = x.float() @ w.float()
        torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
        if pull:
            assert torch.equal(g.x_stage[:m].view(torch.int16), x.view(torch.int16))
        assert int(g.panel_flags.sum()) == 0 and int(g.sched.sum()) == 0
