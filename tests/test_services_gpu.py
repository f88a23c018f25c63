"""The runtime's services on real GPUs: remote GEMM as an Axon function and MoE dispatch / combine on
buffers exchanged through the runtime, first with both runtimes of one process on GPU 0, then as one
process per GPU under torch.distributed.run when the box has two or more (NVLS off, plain peer access)."""
import asyncio
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_remote_gemm_and_moe_through_the_runtime_one_gpu(cuda_device):
    from execution_ucx_b200.models.workloads import AxonTensorRpc, MoeAxon, RemoteGemmAxon
    from execution_ucx_b200.parallel.peer import PeerGroup

    async def main():
        api = AxonTensorRpc(PeerGroup(0, 1, cuda_device), timeout_ms=20000)
        await api.start()
        for fmt in ("bf16", "fp8_block", "mxfp8", "fp8_block_pow2"):
            w = RemoteGemmAxon(api, 512, 768, 1024, fmt=fmt)
            for _ in range(2):
                y = await w.step()
            assert y.shape == (512, 768)
            assert w.max_abs_err(256) < 0.25, fmt
            if fmt == "fp8_block_pow2":
                # power-of-two block scales, applied by the tensor core (the MX kernel): not an approximation of the
                # block-scaled product but the same numbers, up to the order of the fp32 additions
                assert w.max_abs_err(256) < 2e-2, w.max_abs_err(256)
        assert api.server.gemm_launches() == 8
        # M that is not a multiple of 256 takes the one-CTA-per-tile kernel
        w = RemoteGemmAxon(api, 384, 512, 512, fmt="bf16", weight_id=9)
        await w.step()
        assert w.max_abs_err(128) < 0.25
        # a call for a weight nobody serves ends as an error at the caller, and the next call still works
        with pytest.raises(RuntimeError):
            await api.client.remote_gemm(w.x, w.ys[0], worker_name=api.partner_name, weight_id=77)
        await w.step()
        m = await MoeAxon.create(api, n_tokens=128, hidden=1024, topk=4, n_experts=8)
        out = m.step()
        torch.cuda.synchronize()
        m.a2a.check_status()
        torch.testing.assert_close(out.float(), m.reference(), rtol=2e-2, atol=2e-2)
        await m.close()
        api.stop()

    asyncio.run(main())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_services_one_process_per_gpu():
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
                        "--master-port", "29533", str(ROOT / "tests" / "mp_services_gpu.py")],
                       capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert r.returncode == 0 and "SERVICES_OK" in r.stdout, (r.stdout[-2000:] + r.stderr[-4000:])
