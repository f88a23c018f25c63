"""axon: GPU tensor RPC for Python on the native runtime.

Same surface as the reference's ``axon`` package (``axon/python/axon/__init__.py``
and the nanobind module behind it)::

    rt = axon.AxonRuntime("worker", device=axon.cuda(0))
    rt.register_function(my_async_fn)            # annotations drive the wire signature
    rt.start()
    await rt.connect_endpoint_async(peer.get_local_address(), "peer")
    out = await rt.invoke(tensor, 3, worker_name="peer", session_id=1, function="my_async_fn")

Tensors are anything that speaks DLPack (``torch.Tensor``, ``numpy.ndarray``, ...).
They travel as the message payload without a copy on the sending side; large
ones are received straight into the tensors a ``memory_policy`` returns, and the
caller gets those very objects back.
"""
from __future__ import annotations

import asyncio
import inspect
import struct
import typing
from typing import Any, Callable, List, Optional, Sequence

from .. import _build as _build_mod


def _load_native():
    try:
        from . import _axon  # type: ignore
        return _axon
    except ImportError:
        _build_mod.build_kernels()
        _build_mod.build_runtime()
        _build_mod.build_python_module()
        from . import _axon  # type: ignore
        return _axon


_axon = _load_native()

from ._axon import (CudaMemoryResourceManager, DefaultUcxMemoryResourceManager, DLDataType, DLDevice,  # noqa: E402
                    DLPackCapsuleWrapper, MemoryType, ParamType, PayloadType, RpcErrc, RpcFunctionSignature,
                    RpcRequestHeader, RpcResponseHeader, TensorMeta, UcxBuffer, UcxBufferVec,
                    UcxMemoryResourceManager, deserialize_signatures, function_id_from_name,
                    get_default_resource_manager, get_device_context_handle)
from .device import (CpuDevice, CudaDevice, Device, DeviceType, RocmDevice, SyclDevice, auto_detect, cpu, cuda,  # noqa: E402
                     rocm, sycl)

_GROUP_SIZES = "__ntl_group_sizes"   # name of the param that carries nested-tensor-list group sizes


def _is_tensor(x: Any) -> bool:
    return hasattr(x, "__dlpack__") and not isinstance(x, (UcxBuffer, UcxBufferVec))


def _is_tensor_type(t: Any) -> bool:
    name = getattr(t, "__module__", "") + "." + getattr(t, "__qualname__", str(t))
    return name in ("torch.Tensor", "numpy.ndarray", "jax.Array", "jaxlib.xla_extension.ArrayImpl") or name.endswith(".Tensor")


def _default_from_dlpack(sample: Any = None) -> Callable:
    """from_dlpack of the framework the sample (a tensor or a tensor type) belongs to; numpy otherwise."""
    mod = (type(sample).__module__ if sample is not None and not isinstance(sample, type) else getattr(sample, "__module__", "")) or ""
    if mod.startswith("torch"):
        import torch
        return torch.from_dlpack
    if mod.startswith("jax"):
        import jax.dlpack
        return jax.dlpack.from_dlpack
    import numpy
    return numpy.from_dlpack


# ---- nested lists and string lists travel as tagged blobs (STRING params) ----------------------
def _encode_nested(lst: Sequence[Sequence], code: str) -> bytes:
    """[u32 groups][u32 size...][items...], items i64 / f64 / u8."""
    fmt = {"nli64": "q", "nlf64": "d", "nlb": "B"}[code]
    out = [struct.pack("<I", len(lst))] + [struct.pack("<I", len(g)) for g in lst]
    for g in lst:
        out.append(struct.pack("<%d%s" % (len(g), fmt), *[int(v) if fmt != "d" else float(v) for v in g]))
    return b"".join(out)


def _decode_nested(blob: bytes, code: str) -> List[list]:
    fmt = {"nli64": "q", "nlf64": "d", "nlb": "B"}[code]
    (n,) = struct.unpack_from("<I", blob, 0)
    sizes = struct.unpack_from("<%dI" % n, blob, 4)
    off, out = 4 + 4 * n, []
    width = struct.calcsize(fmt)
    for s in sizes:
        vals = list(struct.unpack_from("<%d%s" % (s, fmt), blob, off))
        out.append([bool(v) for v in vals] if code == "nlb" else vals)
        off += s * width
    return out


def _encode_str_list(lst: Sequence[str]) -> bytes:
    out = [struct.pack("<I", len(lst))]
    for s in lst:
        b = s.encode()
        out += [struct.pack("<I", len(b)), b]
    return b"".join(out)


def _decode_str_list(blob: bytes) -> List[str]:
    (n,) = struct.unpack_from("<I", blob, 0)
    off, out = 4, []
    for _ in range(n):
        (ln,) = struct.unpack_from("<I", blob, off)
        out.append(blob[off + 4: off + 4 + ln].decode())
        off += 4 + ln
    return out


def _add_value(add: Callable, v: Any) -> None:
    """Append one non-tensor Python value through `add(value, name)` / typed variants."""
    if isinstance(v, (list, tuple)) and v and all(isinstance(g, (list, tuple)) for g in v):
        flat = [x for g in v for x in g]
        code = "nlb" if flat and all(isinstance(x, bool) for x in flat) else ("nlf64" if any(isinstance(x, float) for x in flat) else "nli64")
        add(_encode_nested(v, code), code, ParamType.STRING)
    elif isinstance(v, (list, tuple)) and v and all(isinstance(x, str) for x in v):
        add(_encode_str_list(v), "ls", ParamType.STRING)
    else:
        add(v, "", None)


def _decode_value(ptype, value, name):
    if ptype == ParamType.STRING and name in ("nli64", "nlf64", "nlb"):
        return _decode_nested(value if isinstance(value, bytes) else value.encode("latin-1"), name)
    if ptype == ParamType.STRING and name == "ls":
        return _decode_str_list(value if isinstance(value, bytes) else value.encode("latin-1"))
    return value


def _classify(args: Sequence[Any]):
    """Split call arguments into plain values and tensors (flat, list, or nested list of tensors)."""
    values, tensors, groups = [], [], None
    for a in args:
        if _is_tensor(a):
            tensors.append(a)
        elif isinstance(a, (list, tuple)) and a and all(_is_tensor(x) for x in a):
            tensors.extend(a)
            groups = (groups or []) + [len(a)] if groups is not None else [len(a)]
        elif isinstance(a, (list, tuple)) and a and all(isinstance(g, (list, tuple)) and g and all(_is_tensor(x) for x in g) for g in a):
            for g in a:
                tensors.extend(g)
            groups = (groups or []) + [len(g) for g in a]
        else:
            values.append(a)
    return values, tensors, groups


def _contiguous(t):
    """Dense row-major form of the tensor, ready to be read by another stream or process."""
    if hasattr(t, "is_contiguous") and not t.is_contiguous():
        t = t.contiguous()
    if getattr(t, "is_cuda", False):
        # the transfer kernel runs on the runtime's own stream (possibly in another process):
        # everything queued on the producer's stream must have finished writing the tensor
        import torch
        torch.cuda.current_stream(t.device).synchronize()
        return t
    if hasattr(t, "is_contiguous"):
        return t
    flags = getattr(t, "flags", None)
    if flags is not None:
        import numpy
        if not flags["C_CONTIGUOUS"]:
            t = numpy.ascontiguousarray(t)
        if not t.flags["WRITEABLE"]:
            # DLPack cannot say "read only": numpy refuses to export such an array (a view of a received
            # tensor, for instance), so it travels as a copy
            t = t.copy()
    return t


def _tensors_from_payload(payload, metas: List[TensorMeta], from_dlpack_fn: Optional[Callable]):
    """Payload object + metadata -> list of framework tensors (policy-supplied objects come back as they are)."""
    out = []
    if payload is None:
        return out
    if isinstance(payload, UcxBufferVec):
        for i, m in enumerate(metas):
            owner = payload.owner(i)
            out.append(owner if owner is not None else (from_dlpack_fn or _default_from_dlpack())(payload.to_dlpack(i, m)))
        return out
    owner = payload.owner()
    if owner is not None:
        return [owner]
    if len(metas) == 1:
        return [(from_dlpack_fn or _default_from_dlpack())(payload.to_dlpack(metas[0]))]
    # several tensors received back to back in one host buffer
    fn = from_dlpack_fn or _default_from_dlpack()
    whole = fn(payload)  # uint8 view
    off = 0
    for m in metas:
        n = m.nbytes()
        piece = whole[off: off + n]
        off += n
        out.append(_reinterpret(piece, m, fn))
    return out


def _reinterpret(piece, meta: TensorMeta, fn):
    """uint8 1-D view -> tensor of meta's dtype and shape (numpy or torch)."""
    code, bits = meta.dtype.code, meta.dtype.bits
    mod = type(piece).__module__
    if mod.startswith("torch"):
        import torch
        table = {(2, 32): torch.float32, (2, 64): torch.float64, (2, 16): torch.float16, (4, 16): torch.bfloat16,
                 (0, 64): torch.int64, (0, 32): torch.int32, (0, 16): torch.int16, (0, 8): torch.int8, (1, 8): torch.uint8, (6, 8): torch.bool}
        return piece.view(table[(code, bits)]).reshape(list(meta.shape))
    import numpy
    kinds = {0: "i", 1: "u", 2: "f", 6: "b"}
    return numpy.asarray(piece).view(numpy.dtype("%s%d" % (kinds.get(code, "u"), bits // 8))).reshape(list(meta.shape))


class AxonRuntime(_axon.AxonRuntime):
    """Runtime with the annotation-driven ``register_function`` and the variadic ``invoke``."""

    def __init__(self, worker_name: str, thread_pool_size: int = 0, timeout=None, device=None, resource_manager=None):
        super().__init__(worker_name, thread_pool_size, timeout, device, resource_manager)
        self._functions = {}

    # ---- server side ------------------------------------------------------------------------
    def register_function(self, fn: Callable, function_id: Optional[int] = None, function_name: Optional[str] = None,
                          memory_policy: Optional[Callable] = None, lifecycle_policy: Optional[Callable] = None,
                          from_dlpack_fn: Optional[Callable] = None) -> int:
        """Register ``async def fn(...)``. Every parameter and the return need annotations:
        ``int`` (INT64), ``float`` (FLOAT64), ``bool``, ``str``, tensor types, ``List[...]`` of those;
        ``Tuple[...]`` only as the return annotation."""
        if not inspect.iscoroutinefunction(fn):
            raise TypeError("register_function needs an `async def` function")
        name = function_name or fn.__name__
        fid = function_id if function_id is not None else function_id_from_name(name, self.worker_name)
        hints = typing.get_type_hints(fn)
        sig = inspect.signature(fn)
        param_types, tensor_params, in_payload = [], [], PayloadType.NO_PAYLOAD
        for pname in sig.parameters:
            if pname not in hints:
                raise TypeError(f"parameter '{pname}' of {name} needs a type annotation")
            kind, ptype = _annotation_kind(hints[pname])
            if kind == "tensor":
                tensor_params.append((pname, False))
            elif kind == "tensor_list":
                tensor_params.append((pname, True))
            else:
                param_types.append(ptype)
            if kind in ("tensor", "tensor_list") and from_dlpack_fn is None:
                from_dlpack_fn = _default_from_dlpack(_tensor_type_of(hints[pname]))
        if tensor_params:
            many = len(tensor_params) > 1 or tensor_params[0][1]
            param_types.append(ParamType.TENSOR_META_VEC if many else ParamType.TENSOR_META)
            in_payload = PayloadType.UCX_BUFFER_VEC if many else PayloadType.UCX_BUFFER
        ret = hints.get("return", None)
        return_types, out_payload = _return_types(ret)
        order = list(sig.parameters)
        tensor_is_list = dict(tensor_params)   # parameter name -> takes a list of tensors

        async def wrapper(header, payload):
            values, metas, groups = [], [], None
            for ptype, value, pname in header.params:
                if ptype == ParamType.TENSOR_META:
                    metas = [value]
                elif ptype == ParamType.TENSOR_META_VEC:
                    metas = list(value)
                elif pname == _GROUP_SIZES:
                    groups = list(value)
                else:
                    values.append(_decode_value(ptype, value, pname))
            tensors = _tensors_from_payload(payload, metas, from_dlpack_fn)
            kwargs, vi, ti = {}, 0, 0
            for pname in order:
                is_list = tensor_is_list.get(pname)
                if is_list is not None:
                    if is_list:
                        take = groups.pop(0) if groups else len(tensors) - ti
                        kwargs[pname] = tensors[ti: ti + take]
                        ti += take
                    else:
                        kwargs[pname] = tensors[ti]
                        ti += 1
                else:
                    kwargs[pname] = values[vi]
                    vi += 1
            result = await fn(**kwargs)
            return _pack_results(result)

        ok = self.register_function_raw(fid, name, param_types, return_types, in_payload, out_payload, wrapper, memory_policy, lifecycle_policy)
        if not ok:
            raise ValueError(f"function id {fid} ({name}) is already registered")
        self._functions[name] = fid
        return fid

    # ---- client side --------------------------------------------------------------------------
    def invoke(self, *args, worker_name: str, session_id: int, function, workflow_id: int = 0,
               memory_policy: Optional[Callable] = None, from_dlpack_fn: Optional[Callable] = None):
        """Call ``function`` (an id, or a name hashed with the worker name) on ``worker_name``.
        Returns a future of the result: a single value, a tuple of values, tensors included."""
        fid = function if isinstance(function, int) else function_id_from_name(function, worker_name)
        header = RpcRequestHeader()
        header.session_id, header.function_id, header.workflow_id = session_id, fid, workflow_id
        values, tensors, groups = _classify(args)

        def add(v, name, ptype):
            if ptype is None:
                header.AddParam(v, name)
            else:
                header.add_param_typed(ptype, v, name)
        for v in values:
            _add_value(add, v)
        payload = None
        sample = tensors[0] if tensors else None
        if tensors:
            tensors = [_contiguous(t) for t in tensors]
            metas = [TensorMeta.from_tensor(t) for t in tensors]
            if groups is not None and len(groups) > 1:
                header.add_param_typed(ParamType.VECTOR_UINT32, groups, _GROUP_SIZES)
            # the tensor metadata goes last so the receiver finds it at once
            if len(tensors) == 1 and groups is None:
                header.add_param_typed(ParamType.TENSOR_META, metas[0], "")
                payload = tensors[0]
            else:
                header.add_param_typed(ParamType.TENSOR_META_VEC, metas, "")
                payload = tensors
        fn = from_dlpack_fn or (_default_from_dlpack(sample) if sample is not None else None)
        # the response is unpacked on the loop thread by the binding itself and settles the future
        return self.invoke_raw(worker_name, header, payload, memory_policy, False,
                               lambda resp, pay: _unpack_response(resp, pay, fn, fid, session_id))


def _unpack_response(resp, payload, from_dlpack_fn, fid, session_id):
    if not resp.ok:
        what = next((v for t, v, n in resp.results if t == ParamType.STRING), f"{resp.status_category} error {resp.status_value}")
        raise RuntimeError(f"{what} (function_id: {fid}) (session_id: {session_id})")
    values, metas = [], []
    for ptype, value, name in resp.results:
        if ptype == ParamType.TENSOR_META:
            metas = [value]
            values.append(("tensor", 0))
        elif ptype == ParamType.TENSOR_META_VEC:
            metas = list(value)
            values.append(("tensors", len(metas)))
        else:
            values.append(("value", _decode_value(ptype, value, name)))
    tensors = _tensors_from_payload(payload, metas, from_dlpack_fn)
    out = []
    for kind, v in values:
        if kind == "tensor":
            out.append(tensors[0])
        elif kind == "tensors":
            out.append(list(tensors))
        else:
            out.append(v)
    if not out:
        return None
    return out[0] if len(out) == 1 else tuple(out)


def _pack_results(result):
    """Handler return value -> (list of result params, payload)."""
    if result is None:
        return [], None
    items = list(result) if isinstance(result, tuple) else [result]
    header = RpcResponseHeader()
    tensors, listy = [], False
    for it in items:
        if _is_tensor(it):
            tensors.append(_contiguous(it))
        elif isinstance(it, (list, tuple)) and it and all(_is_tensor(x) for x in it):
            tensors.extend(_contiguous(x) for x in it)
            listy = True
        else:
            def add(v, name, ptype):
                if ptype is None:
                    header.AddResult(v, name)
                else:
                    header.add_result_typed(ptype, v, name)
            _add_value(add, it)
    payload = None
    if tensors:
        metas = [TensorMeta.from_tensor(t) for t in tensors]
        if len(tensors) == 1 and not listy:
            header.add_result_typed(ParamType.TENSOR_META, metas[0], "")
            payload = tensors[0]
        else:
            header.add_result_typed(ParamType.TENSOR_META_VEC, metas, "")
            payload = tensors
    return header, payload


def _tensor_type_of(ann):
    args = typing.get_args(ann)
    return args[0] if args else ann


def _annotation_kind(ann):
    if ann is bool:
        return "value", ParamType.PRIMITIVE_BOOL
    if ann is int:
        return "value", ParamType.PRIMITIVE_INT64
    if ann is float:
        return "value", ParamType.PRIMITIVE_FLOAT64
    if ann is str:
        return "value", ParamType.STRING
    if ann is bytes:
        return "value", ParamType.VECTOR_UINT8
    if _is_tensor_type(ann):
        return "tensor", None
    origin = typing.get_origin(ann)
    if origin in (list, List):
        (inner,) = typing.get_args(ann) or (None,)
        if inner is bool:
            return "value", ParamType.VECTOR_BOOL
        if inner is int:
            return "value", ParamType.VECTOR_INT64
        if inner is float:
            return "value", ParamType.VECTOR_FLOAT64
        if inner is str:
            return "value", ParamType.STRING
        if _is_tensor_type(inner):
            return "tensor_list", None
        if typing.get_origin(inner) in (list, List):
            return "value", ParamType.STRING
    raise TypeError(f"unsupported annotation {ann!r}: use int, float, bool, str, bytes, a tensor type, or List[...] of those")


def _return_types(ann):
    if ann is None or ann is type(None) or ann is inspect.Signature.empty:
        return [], PayloadType.NO_PAYLOAD
    anns = list(typing.get_args(ann)) if typing.get_origin(ann) in (tuple, typing.Tuple) else [ann]
    types, n_tensors, listy = [], 0, False
    for a in anns:
        kind, ptype = _annotation_kind(a)
        if kind == "tensor":
            n_tensors += 1
        elif kind == "tensor_list":
            n_tensors += 2
            listy = True
        else:
            types.append(ptype)
    payload = PayloadType.NO_PAYLOAD
    if n_tensors == 1 and not listy:
        types.append(ParamType.TENSOR_META)
        payload = PayloadType.UCX_BUFFER
    elif n_tensors:
        types.append(ParamType.TENSOR_META_VEC)
        payload = PayloadType.UCX_BUFFER_VEC
    return types, payload


__all__ = [
    "AxonRuntime", "ParamType", "PayloadType", "RpcErrc", "TensorMeta", "DLDevice", "DLDataType", "UcxBuffer", "UcxBufferVec",
    "DLPackCapsuleWrapper", "RpcRequestHeader", "RpcResponseHeader", "RpcFunctionSignature", "deserialize_signatures",
    "UcxMemoryResourceManager", "DefaultUcxMemoryResourceManager", "CudaMemoryResourceManager", "get_default_resource_manager",
    "get_device_context_handle", "function_id_from_name", "MemoryType",
    "Device", "DeviceType", "CpuDevice", "CudaDevice", "RocmDevice", "SyclDevice", "cpu", "cuda", "rocm", "sycl", "auto_detect",
]
