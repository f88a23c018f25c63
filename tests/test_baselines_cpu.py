"""The library baselines are plain torch: their single-rank logic is checked on the CPU."""
import torch

from execution_ucx_b200.models import baselines as bl


def test_all_to_all_moe_single_rank_matches_weighted_sum():
    torch.manual_seed(0)
    t, h, k, e = 64, 256, 4, 16
    x = torch.randn(t, h).to(torch.bfloat16)
    idx = torch.rand(t, e).topk(k, dim=-1).indices.to(torch.int32)
    w = torch.softmax(torch.randn(t, k), dim=-1)
    out = bl.AllToAllMoe(0, 1, x, idx, w, e).step()
    want = x.float() * w.sum(-1, keepdim=True)
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2)


def test_echo_and_gemm_single_rank():
    src = torch.randn(1024).to(torch.bfloat16)
    echo = bl.NcclEcho(0, 1, 2048, "cpu")
    assert torch.equal(echo.step(src), src)
    g = bl.RecvGemmSend(0, 1, 32, 64, 128, "cpu")
    torch.testing.assert_close(g.step().float(), g.x.float() @ g.w.float(), rtol=3e-2, atol=3e-2)
