"""Small, self-ending cases of each data-plane kernel, for profiler captures.

    python -m execution_ucx_b200.models.profile_case --kernel gemm        (CTA pairs; gemm_1cta: one CTA per tile)
    python -m execution_ucx_b200.models.profile_case --kernel gemm_fp8   (or gemm_mx)
    python -m execution_ucx_b200.models.profile_case --kernel xfer
    python -m execution_ucx_b200.models.profile_case --kernel moe
    python -m execution_ucx_b200.models.profile_case --kernel pull_batch  (the transport's batched small pulls)
    python -m execution_ucx_b200.models.profile_case --kernel gemm_pull   (two GPUs, one process: the GEMM on GPU 0 reads X out of GPU 1's memory;
                                                                           gemm_mx_pull, gemm_fp8_pull: the same for the fp8 kernels)
    python -m execution_ucx_b200.models.profile_case --kernel xfer_peer   (two GPUs, one process: the transfer kernel on GPU 0 writes into GPU 1's memory)
    python -m execution_ucx_b200.models.profile_case --kernel xfer_gather (a transposed matrix gathered into a dense buffer)

Each case keeps well under a few GB on the device, uses inputs larger than L2
where DRAM figures matter, and launches the kernel of interest a handful of times.
"""
from __future__ import annotations

import argparse

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", choices=["gemm", "gemm_1cta", "gemm_fp8", "gemm_mx", "xfer", "pull_batch", "moe", "moe_fp8", "gemm_pull", "gemm_mx_pull", "gemm_fp8_pull", "xfer_peer", "xfer_gather"], required=True)
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    if args.kernel in ("gemm", "gemm_1cta"):
        from ..ops.remote_gemm import RemoteGemm
        m, n, k = 4096, 4096, 4096  # 3 x 32 MiB operands/result: > L2 in total, milliseconds per launch
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        w = (torch.randn(k, n, device=dev) * 0.02).to(torch.bfloat16)
        g = RemoteGemm(w, m)
        y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        for _ in range(args.iters):
            g(x.data_ptr(), m, y.data_ptr(), x_is_local=True, cta_pairs=args.kernel == "gemm")
        torch.cuda.synchronize()
        g.check_status()
    elif args.kernel in ("gemm_pull", "gemm_mx_pull", "gemm_fp8_pull", "xfer_peer"):
        # One process, two GPUs: the peer's memory is an ordinary allocation on GPU 1 that GPU 0 may access.
        # Nothing in the profiled kernels waits for the other GPU, so a replayed launch cannot stall.
        from ..ops import _native
        if torch.cuda.device_count() < 2:
            raise SystemExit("this case needs two GPUs")
        _native.check(_native.load().eux_enable_peer_access(0, 1), "peer access 0 -> 1")
        torch.cuda.set_device(0)
        if args.kernel == "gemm_pull":
            from ..ops.remote_gemm import RemoteGemm
            m, n, k = 4096, 4096, 4096
            x_remote = torch.randn(m, k, device="cuda:1").to(torch.bfloat16)   # complete before any launch below
            torch.cuda.synchronize(1)
            w = (torch.randn(k, n, device=dev) * 0.02).to(torch.bfloat16)
            g = RemoteGemm(w, m)
            y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
            for _ in range(args.iters):
                g(x_remote.data_ptr(), m, y.data_ptr(), x_is_local=False)
            torch.cuda.synchronize(0)
            g.check_status()
            ref = x_remote[:128].to(dev).float() @ w.float()
            assert float((y[:128].float() - ref).abs().max()) < 0.25
        elif args.kernel in ("gemm_mx_pull", "gemm_fp8_pull"):
            from ..ops import remote_gemm as g
            m, n, k = 4096, 4096, 4096
            x = torch.randn(m, k, device=dev)
            w = torch.randn(k, n, device=dev) * 0.02
            if args.kernel == "gemm_mx_pull":
                gemm = g.RemoteGemmMx(w, m)
                xq, xsf = g.quantize_mx(x)
                xs = g.mx_scale_chunks(xsf, False)
                ref = g.mx_dequantized_reference(xq[:128], xsf[:128], gemm.w_q_t, gemm.w_sf)
            else:
                gemm = g.RemoteGemmFp8(w.to(torch.bfloat16), m)
                xq, xs = g.quantize_rows_1x128(x.to(torch.bfloat16))
                ref = g.dequantized_reference(xq[:128], xs[:128], gemm.w_q_t, gemm.w_scale)
            xq_remote, xs_remote = xq.to("cuda:1"), xs.to("cuda:1")    # values and scales lie on GPU 1, complete before any launch
            torch.cuda.synchronize(1)
            y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
            for _ in range(args.iters):
                gemm(xq_remote.data_ptr(), xs_remote.data_ptr(), m, y.data_ptr(), x_is_local=False)
            torch.cuda.synchronize(0)
            gemm.check_status()
            assert float((y[:128].float() - ref).abs().max()) < 0.25
        else:
            from ..ops import tensor_xfer as tx
            n = 256 << 20
            src = torch.randn(n // 2, device=dev).to(torch.bfloat16)
            dst = torch.empty(n // 2, dtype=torch.bfloat16, device="cuda:1")
            flag = torch.zeros(1, dtype=torch.int64, device=dev)
            for i in range(args.iters):
                tx.push(src, dst, flag_ptr=flag.data_ptr(), flag_value=i + 1)
            torch.cuda.synchronize(0)
            assert torch.equal(dst[:4096].to(dev), src[:4096])
    elif args.kernel == "xfer_gather":
        from ..ops import tensor_xfer as tx
        a = torch.randn(8192, 8192, device=dev)            # 256 MiB; its transpose is read with a stride of 8192 elements
        dst = torch.empty(8192 * 8192, device=dev)
        for _ in range(args.iters):
            tx.push(a.t(), dst)
        torch.cuda.synchronize()
        assert torch.equal(dst.view(8192, 8192)[:64], a.t()[:64].contiguous())
    elif args.kernel == "gemm_fp8":
        from ..ops.remote_gemm import RemoteGemmFp8, quantize_rows_1x128
        m, n, k = 4096, 4096, 4096
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        w = (torch.randn(k, n, device=dev) * 0.02).to(torch.bfloat16)
        g = RemoteGemmFp8(w, m)
        xq, xs = quantize_rows_1x128(x)
        y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        for _ in range(args.iters):
            g(xq.data_ptr(), xs.data_ptr(), m, y.data_ptr(), x_is_local=True)
        torch.cuda.synchronize()
        g.check_status()
    elif args.kernel == "gemm_mx":
        from ..ops.remote_gemm import RemoteGemmMx, quantize_mx, mx_scale_chunks
        m, n, k = 4096, 4096, 4096
        x = torch.randn(m, k, device=dev)
        w = torch.randn(k, n, device=dev) * 0.02
        g = RemoteGemmMx(w, m)
        xq, xsf = quantize_mx(x)
        xc = mx_scale_chunks(xsf, False)
        y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        for _ in range(args.iters):
            g(xq.data_ptr(), xc.data_ptr(), m, y.data_ptr(), x_is_local=True)
        torch.cuda.synchronize()
        g.check_status()
    elif args.kernel == "xfer":
        from ..ops import tensor_xfer as tx
        n = 256 << 20  # 256 MiB source + 256 MiB destination
        src = torch.randn(n // 2, device=dev).to(torch.bfloat16)
        dst = torch.empty_like(src)
        flag = torch.zeros(1, dtype=torch.int64, device=dev)
        for i in range(args.iters):
            tx.push(src, dst, flag_ptr=flag.data_ptr(), flag_value=i + 1)
        torch.cuda.synchronize()
    elif args.kernel == "pull_batch":
        from ..ops import _native, tensor_xfer as tx
        # one launch of the size the RPC storm produces: 48 messages, sizes log-uniform in 256 B - 64 KiB
        g = torch.Generator(device="cpu").manual_seed(5)
        sizes = [int(256 * (256.0 ** float(u))) // 4 * 4 for u in torch.rand(_native.PULL_BATCH_MAX, generator=g)]
        flags = torch.zeros(len(sizes), dtype=torch.int64, device=dev)
        srcs = [torch.randint(0, 255, (n,), dtype=torch.uint8, device=dev) for n in sizes]
        dsts = [torch.empty_like(s) for s in srcs]
        for it in range(args.iters):
            tx.pull_batch([(s.data_ptr(), d.data_ptr(), s.numel(), flags.data_ptr() + 8 * i, it + 1)
                           for i, (s, d) in enumerate(zip(srcs, dsts))])
        torch.cuda.synchronize()
        assert all(torch.equal(s, d) for s, d in zip(srcs, dsts))
    else:
        from ..ops import moe
        fp8 = args.kernel == "moe_fp8"
        t, h, k, e = 4096, 7168, 8, 256  # the named configuration: 470 MB of rows per direction
        (rk,) = moe.MoeAllToAll.emulated(1, t, h, k, e, fp8=fp8)
        x = torch.randn(t, h, device=dev).to(torch.bfloat16)
        idx = torch.rand(t, e, device=dev).topk(k, dim=-1).indices.to(torch.int32)
        w = torch.softmax(torch.randn(t, k, device=dev), -1)
        for _ in range(args.iters):
            rk.dispatch(x, idx, w)
            rk.expert_ready()
            rk.combine()
        torch.cuda.synchronize()
        rk.check_status()
    print("ok")


if __name__ == "__main__":
    main()
