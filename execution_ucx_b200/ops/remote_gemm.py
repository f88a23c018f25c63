"""Remote-GEMM RPC kernel (tcgen05 / TMEM / TMA) as a Python op.

``RemoteGemm`` is the callee side: it holds the resident weight in K-major
form and, per call, consumes the caller's activation (local, or pulled from
peer memory by the kernel's copy CTAs while the tensor cores already work on
the panels that have arrived) and writes Y into the caller's memory.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _native

_launches = 0


def launch_count() -> int:
    return _launches


class RemoteGemm:
    def __init__(self, w: torch.Tensor, max_m: int):
        """``w`` is W[K,N] (bf16); it is stored once as Wt[N,K] for the kernel."""
        assert w.dtype == torch.bfloat16 and w.dim() == 2
        self.K, self.N = w.shape
        self.w_t = w.t().contiguous()
        dev = w.device
        self.max_m = max_m
        self.x_stage = torch.empty(max_m, self.K, dtype=torch.bfloat16, device=dev)
        self.panel_flags = torch.zeros(max(1, max_m // 128), dtype=torch.int32, device=dev)
        self.sched = torch.zeros(4, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)

    def __call__(self, x_ptr: int, m: int, y_ptr: int, *, x_is_local: bool, done_flag_ptr: int = 0,
                 done_value: int = 0, copy_ctas: int = 0, timeout_ns: int = 2_000_000_000,
                 cta_pairs: bool = True, head_blocks: Optional[int] = None,
                 copy_warps: Optional[bool] = None) -> None:
        """Y[m,N] (at ``y_ptr``) = X[m,K] (at ``x_ptr``) @ W. Both addresses may be peer memory.
        ``cta_pairs`` selects the kernel that computes 256 x 256 tiles on pairs of CTAs
        (tcgen05 cta_group::2) whenever ``m`` is a multiple of 256; other shapes, and
        ``cta_pairs=False``, run the kernel with one CTA per 128 x 256 tile. ``head_blocks``
        overrides the height (in row blocks) of the first group of tiles when X is remote.
        A remote X is copied into the staging buffer by two spare warps of every CTA while the
        other warps compute (``copy_warps``, the default), or, when ``copy_ctas`` > 0 is given, by
        that many CTAs that copy first and compute afterwards."""
        global _launches
        if m > self.max_m:
            raise ValueError("m exceeds the staging buffer")
        d = _native.GemmDesc()
        d.x_src = x_ptr
        d.x_stage = x_ptr if x_is_local else self.x_stage.data_ptr()
        d.w_t, d.y_dst = self.w_t.data_ptr(), y_ptr
        d.M, d.N, d.K, d.fp8 = m, self.N, self.K, 0
        d.panel_flags, d.sched = self.panel_flags.data_ptr(), self.sched.data_ptr()
        d.done_flag, d.done_value = done_flag_ptr or None, done_value
        d.wait_timeout_ns, d.status, d.copy_ctas = timeout_ns, self.status.data_ptr(), copy_ctas
        if copy_warps is None:
            copy_warps = copy_ctas == 0
        d.flags = (1 if cta_pairs else 0) | (2 if copy_warps else 0) | (0 if head_blocks is None else ((head_blocks + 1) & 0xff) << 8)
        _native.check(_native.load().eux_gemm_launch(C.byref(d), C.c_void_p(_native.current_stream_ptr())),
                      "eux_gemm_launch")
        _launches += 1

    def check_status(self) -> None:
        s = int(self.status.item())
        if s:
            raise RuntimeError(f"remote gemm status code={s & 0xff} where={s >> 8}")


def _block_scale(amax: torch.Tensor, pow2: bool) -> torch.Tensor:
    scale = amax.clamp_min(2.0 ** -100) * (1.0 / 448.0)
    # a power of two at or above what the block needs: at most one bit of e4m3's range is given up, and the
    # scale can then be applied by the tensor core (see block_scales_to_mx)
    return torch.exp2(torch.ceil(torch.log2(scale))) if pow2 else scale


def quantize_rows_1x128(x: torch.Tensor, pow2: bool = False):
    """X[M,K] -> (e4m3 values [M,K], fp32 scales [M,K/128]): one scale per row per 128 columns.
    ``pow2``: every scale is a power of two."""
    m, k = x.shape
    g = x.float().view(m, k // 128, 128)
    scale = _block_scale(g.abs().amax(-1), pow2)
    q = (g * (1.0 / scale).unsqueeze(-1)).to(torch.float8_e4m3fn).view(m, k)
    return q.contiguous(), scale.contiguous()


def quantize_blocks_128x128(w_t: torch.Tensor, pow2: bool = False):
    """Wt[N,K] -> (e4m3 values [N,K], fp32 scales [N/128,K/128]): one scale per 128x128 block.
    ``pow2``: every scale is a power of two."""
    n, k = w_t.shape
    g = w_t.float().view(n // 128, 128, k // 128, 128)
    scale = _block_scale(g.abs().amax(dim=(1, 3)), pow2)
    q = (g * (1.0 / scale)[:, None, :, None]).to(torch.float8_e4m3fn).view(n, k)
    return q.contiguous(), scale.contiguous()


def scales_are_pow2(scale: torch.Tensor) -> bool:
    """True when every fp32 scale is a normal power of two (reads the tensor back: for set-up, not per call)."""
    bits = scale.contiguous().view(torch.int32)
    exp = (bits >> 23) & 0xFF
    return bool((((bits & 0x7FFFFF) == 0) & (bits > 0) & (exp > 0) & (exp < 255)).all())


def block_scales_to_mx(scale: torch.Tensor, rows_per_scale: int) -> torch.Tensor:
    """Power-of-two fp32 block scales -> UE8M0 exponents [R, K/32]: the scale of a 128-wide block of K stands
    for each of its four 32-wide blocks, and (for 128x128 weight blocks, ``rows_per_scale`` = 128) for each of
    its rows. With such scales the block-scaled product and the MX product are the same numbers, so the
    tensor core can apply them (the MX kernel) instead of the epilogue."""
    e8 = ((scale.contiguous().view(torch.int32) >> 23) & 0xFF).to(torch.uint8)   # the biased exponent is the UE8M0 code
    if rows_per_scale > 1:
        e8 = e8.repeat_interleave(rows_per_scale, dim=0)
    return e8.repeat_interleave(4, dim=1).contiguous()


def dequantized_reference(xq, xs, wq_t, ws) -> torch.Tensor:
    """fp32 statement of the block-scaled product: (xq * xs) @ (wq * ws)^T."""
    m, k = xq.shape
    n = wq_t.shape[0]
    x = xq.float().view(m, k // 128, 128) * xs.unsqueeze(-1)
    w = wq_t.float().view(n // 128, 128, k // 128, 128) * ws[:, None, :, None]
    return x.view(m, k) @ w.view(n, k).t()


class RemoteGemmFp8:
    """Block-scaled e4m3 variant: X with 1x128 scales (sent by the caller), W with 128x128 scales (resident)."""

    def __init__(self, w: torch.Tensor, max_m: int):
        assert w.dim() == 2 and w.shape[0] % 128 == 0 and w.shape[1] % 128 == 0
        self.K, self.N = w.shape
        self.w_q_t, self.w_scale = quantize_blocks_128x128(w.t().contiguous())
        dev = w.device
        self.max_m = max_m
        self.x_stage = torch.empty(max_m, self.K, dtype=torch.uint8, device=dev)
        self.x_scale_stage = torch.empty(max_m, self.K // 128, dtype=torch.float32, device=dev)
        self.panel_flags = torch.zeros(max(1, max_m // 128), dtype=torch.int32, device=dev)
        self.sched = torch.zeros(4, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)

    def __call__(self, xq_ptr: int, xs_ptr: int, m: int, y_ptr: int, *, x_is_local: bool, done_flag_ptr: int = 0,
                 done_value: int = 0, copy_ctas: int = 0, timeout_ns: int = 2_000_000_000,
                 copy_warps: Optional[bool] = None, head_blocks: Optional[int] = None) -> None:
        global _launches
        if m > self.max_m:
            raise ValueError("m exceeds the staging buffer")
        d = _native.GemmDesc()
        if copy_warps is None:
            copy_warps = copy_ctas == 0
        d.flags = (2 if copy_warps else 0) | (0 if head_blocks is None else ((head_blocks + 1) & 0xff) << 8)
        d.x_src = xq_ptr
        d.x_stage = xq_ptr if x_is_local else self.x_stage.data_ptr()
        d.x_scale = xs_ptr
        d.x_scale_stage = xs_ptr if x_is_local else self.x_scale_stage.data_ptr()
        d.w_t, d.w_scale, d.y_dst = self.w_q_t.data_ptr(), self.w_scale.data_ptr(), y_ptr
        d.M, d.N, d.K, d.fp8 = m, self.N, self.K, 1
        d.panel_flags, d.sched = self.panel_flags.data_ptr(), self.sched.data_ptr()
        d.done_flag, d.done_value = done_flag_ptr or None, done_value
        d.wait_timeout_ns, d.status, d.copy_ctas = timeout_ns, self.status.data_ptr(), copy_ctas
        _native.check(_native.load().eux_gemm_launch(C.byref(d), C.c_void_p(_native.current_stream_ptr())),
                      "eux_gemm_launch(fp8)")
        _launches += 1

    def check_status(self) -> None:
        s = int(self.status.item())
        if s:
            raise RuntimeError(f"remote gemm (fp8) status code={s & 0xff} where={s >> 8}")


def quantize_mx(x: torch.Tensor):
    """X[R,K] -> (e4m3 values [R,K], UE8M0 exponents [R,K/32] as uint8): the OCP MXFP8 form, one
    power-of-two scale per 32 elements along K, chosen so that the block's largest value fits e4m3."""
    r, k = x.shape
    g = x.float().view(r, k // 32, 32)
    amax = g.abs().amax(-1).clamp_min(2.0 ** -100)
    e = torch.ceil(torch.log2(amax * (1.0 / 448.0))).clamp(-127, 127)
    q = (g * torch.exp2(-e).unsqueeze(-1)).to(torch.float8_e4m3fn).view(r, k)
    return q.contiguous(), (e + 127).to(torch.uint8).contiguous()


def mx_scale_chunks(sf: torch.Tensor, k_step_major: bool) -> torch.Tensor:
    """Exponents [R,K/32] -> the 512-byte chunks the kernel loads: one chunk per 128 rows and 128
    elements of K, byte (r % 32) * 16 + (r // 32) * 4 + j for row r and 32-element block j. Chunks are
    ordered row block first (X: a panel's scales are contiguous) or K-step first (Wt: the two chunks of
    a 256-row tile are adjacent)."""
    r, kb = sf.shape
    v = sf.view(r // 128, 4, 32, kb // 4, 4)            # [row block, r // 32, r % 32, K-step, j]
    v = v.permute(3, 0, 2, 1, 4) if k_step_major else v.permute(0, 3, 2, 1, 4)
    return v.contiguous().view(-1)


def mx_dequantized_reference(xq, xsf, wq_t, wsf) -> torch.Tensor:
    """fp32 statement of the MX product: (xq * 2^(xsf-127)) @ (wq * 2^(wsf-127))^T."""
    def deq(q, sf):
        r, k = q.shape
        return (q.float().view(r, k // 32, 32) * torch.exp2(sf.float() - 127).unsqueeze(-1)).view(r, k)
    return deq(xq, xsf) @ deq(wq_t, wsf).t()


class RemoteGemmMx:
    """MXFP8 variant: e4m3 values with one UE8M0 scale per 32 elements of K on both operands, applied by
    the tensor core (tcgen05.mma kind::mxf8f6f4.block_scale) on pairs of CTAs. The caller sends X's values
    and its scale chunks (``mx_scale_chunks(sf, False)``); the weight is resident. M and N in multiples
    of 256, K of 128."""

    def __init__(self, w: torch.Tensor, max_m: int):
        assert w.dim() == 2 and w.shape[0] % 128 == 0 and w.shape[1] % 256 == 0 and max_m % 256 == 0
        self.K, self.N = w.shape
        self.w_q_t, self.w_sf = quantize_mx(w.t().contiguous())
        self.w_chunks = mx_scale_chunks(self.w_sf, True)
        dev = w.device
        self.max_m = max_m
        self.x_stage = torch.empty(max_m, self.K, dtype=torch.uint8, device=dev)
        self.x_scale_stage = torch.empty(max_m * self.K // 32, dtype=torch.uint8, device=dev)
        self.panel_flags = torch.zeros(max_m // 128, dtype=torch.int32, device=dev)
        self.sched = torch.zeros(4, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)

    def __call__(self, xq_ptr: int, xs_ptr: int, m: int, y_ptr: int, *, x_is_local: bool, done_flag_ptr: int = 0,
                 done_value: int = 0, copy_ctas: int = 0, timeout_ns: int = 2_000_000_000,
                 copy_warps: Optional[bool] = None, head_blocks: Optional[int] = None) -> None:
        global _launches
        if m > self.max_m or m % 256:
            raise ValueError("m exceeds the staging buffer or is not a multiple of 256")
        d = _native.GemmDesc()
        if copy_warps is None:
            copy_warps = copy_ctas == 0
        d.flags = (2 if copy_warps else 0) | (0 if head_blocks is None else ((head_blocks + 1) & 0xff) << 8)
        d.x_src = xq_ptr
        d.x_stage = xq_ptr if x_is_local else self.x_stage.data_ptr()
        d.x_scale = xs_ptr
        d.x_scale_stage = xs_ptr if x_is_local else self.x_scale_stage.data_ptr()
        d.w_t, d.w_scale, d.y_dst = self.w_q_t.data_ptr(), self.w_chunks.data_ptr(), y_ptr
        d.M, d.N, d.K, d.fp8 = m, self.N, self.K, 2
        d.panel_flags, d.sched = self.panel_flags.data_ptr(), self.sched.data_ptr()
        d.done_flag, d.done_value = done_flag_ptr or None, done_value
        d.wait_timeout_ns, d.status, d.copy_ctas = timeout_ns, self.status.data_ptr(), copy_ctas
        _native.check(_native.load().eux_gemm_launch(C.byref(d), C.c_void_p(_native.current_stream_ptr())),
                      "eux_gemm_launch(mx)")
        _launches += 1

    def check_status(self) -> None:
        s = int(self.status.item())
        if s:
            raise RuntimeError(f"remote gemm (mx) status code={s & 0xff} where={s >> 8}")


def smoke(device) -> None:
    """The pair kernel (bf16) with X pulled by the copy warps, the one-CTA kernel, and the MXFP8 kernel, on tiny shapes."""
    x = torch.randn(256, 256, device=device).to(torch.bfloat16)
    w = (torch.randn(256, 512, device=device) * 0.05).to(torch.bfloat16)
    g = RemoteGemm(w, 256)
    y = torch.empty(256, 512, dtype=torch.bfloat16, device=device)
    for kw in (dict(x_is_local=True), dict(x_is_local=False), dict(x_is_local=True, cta_pairs=False)):
        y.zero_()
        g(x.data_ptr(), 256, y.data_ptr(), **kw)
        torch.cuda.synchronize()
        g.check_status()
        torch.testing.assert_close(y.float(), x.float() @ w.float(), rtol=2e-2, atol=2e-2)
    gx = RemoteGemmMx(w.float(), 256)
    xq, xsf = quantize_mx(x.float())
    chunks = mx_scale_chunks(xsf, False)
    y.zero_()
    gx(xq.data_ptr(), chunks.data_ptr(), 256, y.data_ptr(), x_is_local=True)
    torch.cuda.synchronize()
    gx.check_status()
    torch.testing.assert_close(y.float(), mx_dequantized_reference(xq, xsf, gx.w_q_t, gx.w_sf), rtol=2e-2, atol=2e-2)
