"""Small, self-ending cases of each data-plane kernel, for profiler captures.

    python -m execution_ucx_b200.models.profile_case --kernel gemm        (CTA pairs; gemm_1cta: one CTA per tile)
    python -m execution_ucx_b200.models.profile_case --kernel gemm_fp8   (or gemm_mx)
    python -m execution_ucx_b200.models.profile_case --kernel xfer
    python -m execution_ucx_b200.models.profile_case --kernel moe
    python -m execution_ucx_b200.models.profile_case --kernel pull_batch  (the transport's batched small pulls)

Each case keeps well under a few GB on the device, uses inputs larger than L2
where DRAM figures matter, and launches the kernel of interest a handful of times.
"""
from __future__ import annotations

import argparse

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", choices=["gemm", "gemm_1cta", "gemm_fp8", "gemm_mx", "xfer", "pull_batch", "moe", "moe_fp8"], required=True)
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
