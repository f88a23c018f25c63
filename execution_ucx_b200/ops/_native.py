"""ctypes view of ``libeux_kernels.so`` (the C ABI in ``csrc/kernels/eux_kernels.h``).

The library is built in-tree by :mod:`execution_ucx_b200._build`. On a machine
with a GPU the ops refuse to run without it: there is no eager fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent.parent / "_lib" / "libeux_kernels.so"
_lib = None

EUX_MAX_DIMS = 8
DT_BYTES, DT_F32, DT_F16, DT_BF16, DT_F8E4M3 = 0, 1, 2, 3, 4
OP_NONE, OP_ADD, OP_MUL = 0, 1, 2
ST_OK, ST_TIMEOUT, ST_BAD_ARG, ST_OVERFLOW = 0, 1, 2, 3


PULL_BATCH_MAX = 48


class PullItem(C.Structure):
    """eux_pull_item: one dense copy of a batch whose descriptors travel in the launch parameters."""
    _fields_ = [("src", C.c_void_p), ("dst", C.c_void_p), ("nbytes", C.c_uint64), ("flag", C.c_void_p),
                ("flag_value", C.c_uint64), ("flag2", C.c_void_p), ("flag2_value", C.c_uint64)]


class XferDesc(C.Structure):
    _fields_ = [
        ("src", C.c_void_p), ("dst", C.c_void_p), ("n_elems", C.c_uint64),
        ("src_dtype", C.c_int32), ("dst_dtype", C.c_int32), ("op", C.c_int32), ("op_arg", C.c_float),
        ("ndim", C.c_int32), ("reserved0", C.c_int32),
        ("shape", C.c_int64 * EUX_MAX_DIMS), ("stride", C.c_int64 * EUX_MAX_DIMS),
        ("flag", C.c_void_p), ("flag_value", C.c_uint64),
        ("wait_flag", C.c_void_p), ("wait_value", C.c_uint64), ("wait_timeout_ns", C.c_uint64),
        ("status", C.c_void_p), ("flag2", C.c_void_p), ("flag2_value", C.c_uint64),
    ]


class PingPongDesc(C.Structure):
    _fields_ = [
        ("local_buf", C.c_void_p), ("peer_buf", C.c_void_p), ("nbytes", C.c_uint64),
        ("local_flag", C.c_void_p), ("peer_flag", C.c_void_p), ("grid_bar", C.c_void_p),
        ("ts_out", C.c_void_p), ("status", C.c_void_p),
        ("iters", C.c_int32), ("initiator", C.c_int32), ("base_seq", C.c_uint64),
        ("wait_timeout_ns", C.c_uint64),
    ]


class MoeDesc(C.Structure):
    _fields_ = [
        ("rank", C.c_int32), ("world", C.c_int32), ("n_tokens", C.c_int32), ("hidden", C.c_int32),
        ("topk", C.c_int32), ("n_experts", C.c_int32), ("fp8", C.c_int32), ("capacity", C.c_int32),
        ("x", C.c_void_p), ("topk_idx", C.c_void_p), ("topk_w", C.c_void_p),
        ("arena_peer", C.c_void_p), ("meta_peer", C.c_void_p), ("flag_peer", C.c_void_p),
        ("slot_of", C.c_void_p), ("counters", C.c_void_p), ("out", C.c_void_p),
        ("seq", C.c_uint64), ("wait_timeout_ns", C.c_uint64), ("status", C.c_void_p),
    ]


class GemmDesc(C.Structure):
    _fields_ = [
        ("x_src", C.c_void_p), ("x_stage", C.c_void_p), ("w_t", C.c_void_p), ("y_dst", C.c_void_p),
        ("x_scale", C.c_void_p), ("x_scale_stage", C.c_void_p), ("w_scale", C.c_void_p),
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32), ("fp8", C.c_int32),
        ("panel_flags", C.c_void_p), ("sched", C.c_void_p),
        ("done_flag", C.c_void_p), ("done_value", C.c_uint64), ("wait_timeout_ns", C.c_uint64),
        ("status", C.c_void_p), ("copy_ctas", C.c_int32), ("flags", C.c_int32),
    ]


def lib_path() -> Path:
    return _LIB_PATH


def load():
    """Load the kernels library; raise with build advice if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        if os.environ.get("EUX_NO_AUTOBUILD") == "1":
            raise RuntimeError(f"{_LIB_PATH} is missing: run `python -m execution_ucx_b200._build`")
        from .. import _build
        _build.build_kernels()
    lib = C.CDLL(str(_LIB_PATH), mode=C.RTLD_GLOBAL)
    P, I, U64 = C.c_void_p, C.c_int, C.c_uint64
    lib.eux_xfer_launch.argtypes = [C.POINTER(XferDesc), P, I, P]
    lib.eux_xfer_bulk_launch.argtypes = [C.POINTER(XferDesc), P, I, P]
    lib.eux_xfer_rpc_step_launch.argtypes = [C.POINTER(XferDesc), C.POINTER(XferDesc), C.POINTER(XferDesc), P, I, P]
    lib.eux_xfer_batch_launch.argtypes = [P, I, P]
    lib.eux_xfer_pull_batch_launch.argtypes = [C.POINTER(PullItem), I, P]
    lib.eux_pingpong_launch.argtypes = [C.POINTER(PingPongDesc), I, P]
    lib.eux_memcpy_peer_async.argtypes = [P, I, P, I, C.c_size_t, P]
    lib.eux_ipc_export.argtypes = [P, C.c_char_p]
    lib.eux_ipc_open.argtypes = [C.c_char_p, C.POINTER(P)]
    lib.eux_ipc_close.argtypes = [P]
    lib.eux_enable_peer_access.argtypes = [I, I]
    lib.eux_device_malloc.argtypes = [C.POINTER(P), C.c_size_t]
    lib.eux_device_free.argtypes = [P]
    lib.eux_host_alloc_mapped.argtypes = [C.POINTER(P), C.POINTER(P), C.c_size_t]
    lib.eux_host_free.argtypes = [P]
    lib.eux_error_string.argtypes = [I]
    lib.eux_error_string.restype = C.c_char_p
    lib.eux_moe_row_bytes.argtypes = [I, I]
    lib.eux_moe_row_bytes.restype = C.c_size_t
    lib.eux_moe_dispatch_launch.argtypes = [C.POINTER(MoeDesc), I, P]
    lib.eux_moe_expert_ready_launch.argtypes = [C.POINTER(MoeDesc), P]
    lib.eux_moe_combine_launch.argtypes = [C.POINTER(MoeDesc), I, P]
    if hasattr(lib, "eux_gemm_launch"):
        lib.eux_gemm_launch.argtypes = [C.POINTER(GemmDesc), P]
        lib.eux_gemm_num_sms.argtypes = []
    if hasattr(lib, "eux_gemm_bf16_noalloc"):
        lib.eux_gemm_bf16_noalloc.argtypes = [P, P, P, I, I, I, P, U64, P]
        lib.eux_gemm_bf16_noalloc.restype = I
    _lib = lib
    _preload(lib)
    return lib


def _preload(lib) -> None:
    """Load every kernel on the current device now. With the driver's lazy loading a kernel is loaded by
    its first launch, which may have to wait for kernels that are running; a first launch made while some
    library's kernel spins on a peer (a collective's barrier) that in turn waits for this launch is a
    deadlock. Nothing is done where CUDA has not been brought up (CPU-only use of the package)."""
    try:
        import torch
        if not (torch.cuda.is_available() and torch.cuda.is_initialized()):
            return
    except Exception:
        return
    for fn in ("eux_xfer_preload", "eux_moe_preload", "eux_gemm_preload"):
        if hasattr(lib, fn):
            getattr(lib, fn)()


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().eux_error_string(rc).decode()
        raise RuntimeError(f"{what} failed: {msg} ({rc})")


_DTYPE_CODES = None


def torch_dtype_code(dtype) -> int:
    global _DTYPE_CODES
    if _DTYPE_CODES is None:
        import torch
        _DTYPE_CODES = {torch.float32: DT_F32, torch.float16: DT_F16, torch.bfloat16: DT_BF16,
                        torch.float8_e4m3fn: DT_F8E4M3, torch.uint8: DT_BYTES, torch.int8: DT_BYTES}
    try:
        return _DTYPE_CODES[dtype]
    except KeyError:
        raise TypeError(f"dtype {dtype} is not supported by the transfer kernels") from None


def current_stream_ptr() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream
