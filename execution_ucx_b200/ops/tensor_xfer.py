"""Tensor send/recv kernels (pack + cast + handler + flag) as Python ops.

``push`` is the data plane of one Axon tensor message: it reads a (possibly
strided) source tensor, optionally applies the elementwise handler and a dtype
cast, writes densely into a destination that may live on another GPU, and
release-stores a sequence flag. The reference moves the same bytes with
``ucp_am_send_nbx`` over UCX cuda_ipc (ucx_context/ucx_connection.cpp:353-374)
and ignores strides (rpc_core/utils/tensor_meta.hpp:91-104).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _native
from ._native import OP_ADD, OP_MUL, OP_NONE, XferDesc

_launches = 0


def launch_count() -> int:
    """Number of kernels this module has launched (for bench accounting)."""
    return _launches


def _is_dense(t: torch.Tensor) -> bool:
    return t.is_contiguous()


_scratch = {}


def _scratch_counter(device) -> torch.Tensor:
    key = (device.index, torch.cuda.current_stream().cuda_stream)
    if key not in _scratch:
        _scratch[key] = torch.zeros(64, dtype=torch.int32, device=device)
    return _scratch[key]


def make_desc(src: torch.Tensor, dst_ptr: int, dst_dtype: torch.dtype, op: int = OP_NONE, op_arg: float = 0.0,
              flag_ptr: int = 0, flag_value: int = 0, wait_flag_ptr: int = 0, wait_value: int = 0,
              wait_timeout_ns: int = 0, status_ptr: int = 0) -> XferDesc:
    d = XferDesc()
    d.src = src.data_ptr()
    d.dst = dst_ptr
    d.n_elems = src.numel()
    d.src_dtype = _native.torch_dtype_code(src.dtype)
    d.dst_dtype = _native.torch_dtype_code(dst_dtype)
    d.op, d.op_arg = op, op_arg
    if _is_dense(src):
        d.ndim = 0
    else:
        if src.dim() > _native.EUX_MAX_DIMS:
            raise ValueError("at most 8 dimensions")
        d.ndim = src.dim()
        for i in range(src.dim()):
            d.shape[i] = src.shape[i]
            d.stride[i] = src.stride(i)
    d.flag, d.flag_value = flag_ptr or None, flag_value
    d.wait_flag, d.wait_value, d.wait_timeout_ns = wait_flag_ptr or None, wait_value, wait_timeout_ns
    d.status = status_ptr or None
    return d


def push(src: torch.Tensor, dst, *, dst_dtype: Optional[torch.dtype] = None, op: int = OP_NONE,
         op_arg: float = 0.0, flag_ptr: int = 0, flag_value: int = 0, wait_flag_ptr: int = 0,
         wait_value: int = 0, wait_timeout_ns: int = 0, status_ptr: int = 0, max_ctas: int = 0,
         bulk: bool = False) -> None:
    """Launch one transfer on the current stream.

    ``dst`` is a tensor (its dtype is the destination dtype) or a raw device
    address (then ``dst_dtype`` is required); it may be peer memory. ``bulk`` moves a dense
    same-type copy of 16-byte aligned buffers with the bulk-copy engine instead of register
    loads and stores.
    """
    global _launches
    if not src.is_cuda:
        raise ValueError("push() moves device tensors; host tensors travel on the control plane")
    if isinstance(dst, torch.Tensor):
        if dst.numel() < src.numel() or not dst.is_contiguous():
            raise ValueError("destination must be dense and large enough")
        dst_ptr, dst_dtype = dst.data_ptr(), dst.dtype
    else:
        dst_ptr = int(dst)
        dst_dtype = dst_dtype or src.dtype
    d = make_desc(src, dst_ptr, dst_dtype, op, op_arg, flag_ptr, flag_value, wait_flag_ptr, wait_value,
                  wait_timeout_ns, status_ptr)
    counter = _scratch_counter(src.device)
    lib = _native.load()
    fn = lib.eux_xfer_bulk_launch if bulk else lib.eux_xfer_launch
    _native.check(fn(C.byref(d), C.c_void_p(counter.data_ptr()), max_ctas,
                     C.c_void_p(_native.current_stream_ptr())), "eux_xfer_bulk_launch" if bulk else "eux_xfer_launch")
    _launches += 1


def rpc_echo_step(src: torch.Tensor, req_dst_ptr: int, req_flag_ptr: int, request: torch.Tensor, resp_dst_ptr: int,
                  resp_flag_ptr: int, local_req_flag_ptr: int, local_resp_flag_ptr: int, seq: int, *, op: int = OP_NONE,
                  op_arg: float = 0.0, status_ptr: int = 0, wait_timeout_ns: int = 0, max_ctas: int = 0) -> None:
    """One echo step of a tensor RPC in ONE launch: push ``src`` into the partner's request slot and publish
    ``seq`` there; wait for the partner's request (``request``, this rank's request slot), apply the handler
    and push the result into the partner's response slot, publishing ``seq``; wait for this rank's response
    flag. ``src`` and ``request`` are dense, 16-byte aligned and of one dtype. The partner launches the same
    step on its GPU."""
    global _launches
    if not (src.is_cuda and src.is_contiguous() and request.is_contiguous() and src.dtype == request.dtype):
        raise ValueError("rpc_echo_step() wants dense tensors of one dtype")
    step = RpcEchoStep(src, req_dst_ptr, req_flag_ptr, request, resp_dst_ptr, resp_flag_ptr, local_req_flag_ptr,
                       local_resp_flag_ptr, op=op, op_arg=op_arg, status_ptr=status_ptr, wait_timeout_ns=wait_timeout_ns,
                       max_ctas=max_ctas)
    step.launch(seq)


class RpcEchoStep:
    """The descriptors of ``rpc_echo_step`` built once: ``launch(seq)`` only writes the sequence number into
    them and makes the one native call, which is what a small-message loop can afford per step."""

    def __init__(self, src: torch.Tensor, req_dst_ptr: int, req_flag_ptr: int, request: torch.Tensor, resp_dst_ptr: int,
                 resp_flag_ptr: int, local_req_flag_ptr: int, local_resp_flag_ptr: int, *, op: int = OP_NONE,
                 op_arg: float = 0.0, status_ptr: int = 0, wait_timeout_ns: int = 0, max_ctas: int = 0):
        if not (src.is_cuda and src.is_contiguous() and request.is_contiguous() and src.dtype == request.dtype):
            raise ValueError("rpc_echo_step() wants dense tensors of one dtype")
        self.req = make_desc(src, req_dst_ptr, src.dtype, OP_NONE, 0.0, req_flag_ptr, 0, 0, 0, wait_timeout_ns, status_ptr)
        self.resp = make_desc(request, resp_dst_ptr, request.dtype, op, op_arg, resp_flag_ptr, 0, local_req_flag_ptr, 0,
                              wait_timeout_ns, status_ptr)
        self.done = make_desc(request[:0], resp_dst_ptr, request.dtype, OP_NONE, 0.0, 0, 0, local_resp_flag_ptr, 0,
                              wait_timeout_ns, status_ptr)
        self._keep = (src, request)
        self._device = src.device
        self._fn = _native.load().eux_xfer_rpc_step_launch
        self._refs = (C.byref(self.req), C.byref(self.resp), C.byref(self.done))
        self._max_ctas = max_ctas

    def launch(self, seq: int) -> None:
        global _launches
        self.req.flag_value = seq
        self.resp.flag_value = seq
        self.resp.wait_value = seq
        self.done.wait_value = seq
        counter = _scratch_counter(self._device)
        _native.check(self._fn(*self._refs, C.c_void_p(counter.data_ptr() + 16), self._max_ctas,
                               C.c_void_p(_native.current_stream_ptr())), "eux_xfer_rpc_step_launch")
        _launches += 1


def push_batch(descs, stream_ptr: Optional[int] = None) -> None:
    """Many small transfers in one launch (one CTA per descriptor)."""
    global _launches
    n = len(descs)
    if n == 0:
        return
    arr = (XferDesc * n)(*descs)
    host = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8)
    dev = host.cuda()
    lib = _native.load()
    _native.check(lib.eux_xfer_batch_launch(C.c_void_p(dev.data_ptr()), n,
                                            C.c_void_p(stream_ptr or _native.current_stream_ptr())),
                  "eux_xfer_batch_launch")
    dev.record_stream(torch.cuda.current_stream())
    _launches += 1


def pull_batch(items, stream_ptr: Optional[int] = None) -> None:
    """Up to 48 dense copies in one launch, one CTA each, the descriptors in the launch parameters (nothing
    is read from memory to find the work). `items`: (src_ptr, dst_ptr, nbytes, flag_ptr or 0, flag_value); a
    copy's flag is written when that copy is done. This is what the transport uses for the small messages of
    one pass of its loop."""
    global _launches
    n = len(items)
    if n == 0:
        return
    arr = (_native.PullItem * n)()
    for i, (src, dst, nbytes, flag, value) in enumerate(items):
        arr[i].src, arr[i].dst, arr[i].nbytes, arr[i].flag, arr[i].flag_value = src, dst, nbytes, flag or None, value
    lib = _native.load()
    _native.check(lib.eux_xfer_pull_batch_launch(arr, n, C.c_void_p(stream_ptr or _native.current_stream_ptr())),
                  "eux_xfer_pull_batch_launch")
    _launches += 1


def pingpong(local_buf: torch.Tensor, peer_buf_ptr: int, nbytes: int, local_flag_ptr: int, peer_flag_ptr: int,
             grid_bar: torch.Tensor, iters: int, initiator: int, base_seq: int = 0, ts_out: Optional[torch.Tensor] = None,
             status: Optional[torch.Tensor] = None, ctas: int = 0, wait_timeout_ns: int = 2_000_000_000) -> None:
    """Device-driven ping-pong (see tensor_xfer.cu); one launch per GPU."""
    global _launches
    d = _native.PingPongDesc()
    d.local_buf, d.peer_buf, d.nbytes = local_buf.data_ptr(), peer_buf_ptr, nbytes
    d.local_flag, d.peer_flag = local_flag_ptr or None, peer_flag_ptr or None
    d.grid_bar = grid_bar.data_ptr()
    d.ts_out = ts_out.data_ptr() if ts_out is not None else None
    d.status = status.data_ptr() if status is not None else None
    d.iters, d.initiator, d.base_seq, d.wait_timeout_ns = iters, initiator, base_seq, wait_timeout_ns
    lib = _native.load()
    _native.check(lib.eux_pingpong_launch(C.byref(d), ctas, C.c_void_p(_native.current_stream_ptr())),
                  "eux_pingpong_launch")
    _launches += 1


__all__ = ["push", "rpc_echo_step", "RpcEchoStep", "push_batch", "pingpong", "make_desc", "launch_count", "OP_NONE", "OP_ADD", "OP_MUL"]
