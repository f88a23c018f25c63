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
from .loop import SpinningSelector, new_event_loop, run  # noqa: E402

_GROUP_SIZES = "__ntl_group_sizes"   # name of the VECTOR_UINT32 param that carries nested-tensor-list group sizes
_NESTED_TAGS = {"nli64": "q", "nlf64": "d", "nlb": "B"}
_STR_LIST_TAG = "vs"                 # List[str] blob (reference: param_conversion.cpp:543)
_SUPPORTED = "Supported types: int, float, bool, str, List[T], Tuple[...], Dlpack compatible Tensor/Array"


def _is_tensor(x: Any) -> bool:
    return hasattr(x, "__dlpack__") and not isinstance(x, (UcxBuffer, UcxBufferVec, type))


def _is_seq(x: Any) -> bool:
    return isinstance(x, (list, tuple))


def _type_name(t: Any) -> str:
    return getattr(t, "__module__", "") + "." + getattr(t, "__qualname__", str(t))


def _is_tensor_type(t: Any) -> bool:
    """A bare class that is (or looks like) a DLPack tensor type: never a generic alias."""
    if hasattr(t, "__origin__"):
        return False
    if hasattr(t, "__dlpack__"):
        return True
    name = _type_name(t)
    if name in ("torch.Tensor", "numpy.ndarray", "jax.Array", "jaxlib.xla_extension.ArrayImpl"):
        return True
    text = str(t)
    return any(k in text for k in ("numpy.ndarray", "torch.Tensor", "jax.Array", "jaxlib.xla_extension.ArrayImpl"))


def _default_from_dlpack(sample: Any = None) -> Callable:
    """from_dlpack of the framework the sample (a tensor or a tensor type) belongs to; numpy otherwise."""
    if isinstance(sample, type):
        fn = getattr(sample, "from_dlpack", None)
        if callable(fn):
            return fn
        mod = getattr(sample, "__module__", "") or ""
    else:
        mod = (type(sample).__module__ if sample is not None else "") or ""
    if mod.startswith("torch"):
        import torch
        return torch.from_dlpack
    if mod.startswith("jax"):
        import jax.dlpack
        return jax.dlpack.from_dlpack
    import numpy
    return numpy.from_dlpack


def _takes_capsule(fn: Callable) -> bool:
    """torch.from_dlpack accepts the bare capsule and then skips its device and stream queries: the bytes
    are complete when the runtime hands them over, so nothing needs to be ordered."""
    import sys
    t = sys.modules.get("torch")
    return t is not None and fn is t.from_dlpack


# ---- nested lists and string lists travel as tagged blobs (STRING params) ----------------------
def _encode_nested(lst: Sequence[Sequence], code: str) -> bytes:
    """[u32 groups][u32 size...][items...], items i64 / f64 / u8."""
    fmt = _NESTED_TAGS[code]
    out = [struct.pack("<I", len(lst))] + [struct.pack("<I", len(g)) for g in lst]
    for g in lst:
        out.append(struct.pack("<%d%s" % (len(g), fmt), *[float(v) if fmt == "d" else int(v) for v in g]))
    return b"".join(out)


def _decode_nested(blob: bytes, code: str) -> List[list]:
    fmt = _NESTED_TAGS[code]
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


def _nested_code(v: Sequence[Sequence]) -> str:
    """Wire tag of a list of lists, from its first element; raises TypeError for anything but numbers and bools."""
    for g in v:
        if not _is_seq(g):
            raise TypeError("Heterogeneous sequences are not supported as RPC arguments: every element of a nested list must be a list")
    flat = [x for g in v for x in g]
    for x in flat:
        if not isinstance(x, (bool, int, float)):
            raise TypeError(f"unsupported element type in nested list: {type(x).__name__} (supported: int, float, bool, Tensor)")
    if flat and all(isinstance(x, bool) for x in flat):
        return "nlb"
    return "nlf64" if any(isinstance(x, float) for x in flat) else "nli64"


def _add_inferred(add_typed: Callable, add_plain: Callable, v: Any) -> None:
    """Append one non-tensor Python value, choosing the wire form from the value itself."""
    if _is_seq(v) and v and _is_seq(v[0]):
        code = _nested_code(v)
        add_typed(ParamType.STRING, _encode_nested(v, code), code)
    elif _is_seq(v) and v and isinstance(v[0], str):
        if not all(isinstance(x, str) for x in v):
            raise TypeError("unsupported element type: a list that starts with a str must hold only str")
        add_typed(ParamType.STRING, _encode_str_list(v), _STR_LIST_TAG)
    else:
        add_plain(v)


def _add_declared(add_typed: Callable, add_plain: Callable, ptype, v: Any) -> None:
    """Append a value under the wire type the function declared (UNKNOWN: infer; VOID: nothing)."""
    if ptype == ParamType.VOID:
        return
    if ptype == ParamType.UNKNOWN or ptype == ParamType.STRING and not isinstance(v, (str, bytes)):
        _add_inferred(add_typed, add_plain, v)
    else:
        add_typed(ptype, v, "")


def _contiguous(t, strided_ok: bool = False):
    """The tensor in a form the native layer can send. Host tensors: dense row-major. Device tensors are
    handed on without waiting for their producer (the native layer records an event on the producer's stream
    and the transport orders itself after it), and a single strided one (``strided_ok``) as it lies when its
    strides are not negative: the transfer kernel gathers it on the way."""
    if getattr(t, "is_cuda", False):
        if not t.is_contiguous() and not (strided_ok and 1 <= t.dim() <= 8 and all(s >= 0 for s in t.stride()) and t.numel() > 0
                                          and t.element_size() in (1, 2, 4, 8, 16)):
            t = t.contiguous()
        return t
    if hasattr(t, "is_contiguous") and not t.is_contiguous():
        t = t.contiguous()
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


def _dtype_name(dtype) -> str:
    """'float16' for torch.float16, numpy.float16, numpy.dtype('float16') and 'float16'."""
    name = getattr(dtype, "__name__", None) or getattr(dtype, "name", None) or str(dtype)
    return str(name).rsplit(".", 1)[-1]


def _wire_code(wire_dtype) -> int:
    """Kernel code of the type in which a device tensor's elements shall travel (0: as they are)."""
    if wire_dtype is None:
        return 0
    name = _dtype_name(wire_dtype)
    code = {"float32": 1, "float16": 2, "half": 2, "bfloat16": 3}.get(name)
    if code is None:
        raise ValueError(f"wire_dtype must be float32, float16 or bfloat16, not {wire_dtype}")
    return code


def _apply_wire_dtype(payload, wire_dtype):
    """What the transfer kernel cannot convert on the way (host tensors, lists of tensors) is converted here."""
    if wire_dtype is None or payload is None:
        return payload

    def convert(t, even_on_device):
        if hasattr(t, "is_floating_point"):                      # torch
            if t.is_floating_point() and (even_on_device or not getattr(t, "is_cuda", False)):
                import torch
                target = getattr(torch, _dtype_name(wire_dtype))
                return t.to(target).contiguous() if even_on_device else t.to(target)
            return t
        kind = getattr(getattr(t, "dtype", None), "kind", None)   # numpy
        if kind == "f":
            name = _dtype_name(wire_dtype)
            if name == "bfloat16":
                raise ValueError("numpy has no bfloat16: send the array as float16 or float32, or as a torch tensor")
            return t.astype(name)
        return t

    if isinstance(payload, list):
        return [convert(t, True) for t in payload]
    return convert(payload, False)


_TORCH_DTYPES = {(2, 32): "float32", (2, 64): "float64", (2, 16): "float16", (4, 16): "bfloat16", (0, 64): "int64", (0, 32): "int32",
                 (0, 16): "int16", (0, 8): "int8", (1, 8): "uint8", (6, 8): "bool"}
_NUMPY_KINDS = {0: "i", 1: "u", 2: "f", 6: "b"}


def _reinterpret(piece, meta: TensorMeta, fn):
    """uint8 1-D view -> tensor of meta's dtype and shape (numpy or torch)."""
    code, bits = meta.dtype.code, meta.dtype.bits
    mod = type(piece).__module__
    if mod.startswith("torch"):
        import torch
        return piece.view(getattr(torch, _TORCH_DTYPES[(code, bits)])).reshape(list(meta.shape))
    import numpy
    return numpy.asarray(piece).view(numpy.dtype("%s%d" % (_NUMPY_KINDS.get(code, "u"), bits // 8))).reshape(list(meta.shape))


def _payload_nbytes(meta: TensorMeta) -> int:
    """Bytes the tensor takes in a payload: ``meta.nbytes()``, except that a rank-0 tensor is one element there."""
    if meta.ndim == 0:
        return (meta.dtype.bits * (meta.dtype.lanes or 1) + 7) // 8
    return meta.nbytes()


def _empty_tensor(meta: TensorMeta, fn: Optional[Callable]):
    """A tensor without elements never travels (a message of no bytes has no payload): it is made here, in host
    memory, with the shape and type that its description gives."""
    code, bits = meta.dtype.code, meta.dtype.bits
    f = fn or _default_from_dlpack()
    if _takes_capsule(f) or (code, bits) == (4, 16):
        import torch
        return torch.empty(list(meta.shape), dtype=getattr(torch, _TORCH_DTYPES[(code, bits)]))
    import numpy
    made = numpy.empty(list(meta.shape), dtype=numpy.dtype("%s%d" % (_NUMPY_KINDS.get(code, "u"), bits // 8)))
    return made if f is numpy.from_dlpack else f(made)


class _TensorStream:
    """The tensors of one message, in order: payload object + metadata -> framework tensors.

    A tensor whose memory came from a memory policy is handed back as the very object the policy
    returned; everything else goes through a ``from_dlpack`` function (the one given for that
    position, else the framework default)."""

    def __init__(self, payload, metas: List[TensorMeta]):
        self.payload, self.metas, self.pos = payload, metas, 0
        self._whole = None

    def __len__(self) -> int:
        if self.payload is not None:
            return len(self.metas)
        # no payload at all: tensors without elements are still there
        return len(self.metas) if self.metas and all(_payload_nbytes(m) == 0 for m in self.metas) else 0

    def remaining(self) -> int:
        return len(self) - self.pos

    def take(self, fn: Optional[Callable]):
        i, self.pos = self.pos, self.pos + 1
        if i >= len(self):
            raise RuntimeError("the message carries fewer tensors than the function takes")
        p, m = self.payload, self.metas[i]
        if p is None:
            return _empty_tensor(m, fn)
        if isinstance(p, UcxBufferVec):
            owner = p.owner(i)
            if owner is not None:
                return owner
            f = fn or _default_from_dlpack()
            return f(p.to_capsule(i, m)) if _takes_capsule(f) else f(p.to_dlpack(i, m))
        if len(self.metas) == 1:
            owner = p.owner()
            if owner is not None:
                return owner
            f = fn or _default_from_dlpack()
            return f(p.to_capsule(m)) if _takes_capsule(f) else f(p.to_dlpack(m))
        # several tensors received back to back in one host buffer
        f = fn or _default_from_dlpack()
        if self._whole is None:
            self._whole = f(p)  # uint8 view
        off = sum(_payload_nbytes(x) for x in self.metas[:i])
        return _reinterpret(self._whole[off: off + _payload_nbytes(m)], m, f)


def _split_params(meta_list):
    """(type, value, name) triples -> (non-tensor triples in order, tensor metas)."""
    plain, metas = [], []
    for ptype, value, name in meta_list:
        if ptype == ParamType.TENSOR_META:
            metas = [value]
        elif ptype == ParamType.TENSOR_META_VEC:
            metas = list(value)
        else:
            plain.append((ptype, value, name))
    return plain, metas


# ---- signatures ---------------------------------------------------------------------------------
class _Sig:
    """What a registered function takes and returns, in wire terms (reference: FunctionSignatureInfo,
    axon/python/src/python_helpers.cpp:405-560)."""

    __slots__ = ("param_types", "return_types", "in_payload", "out_payload", "encoded", "param_from_dlpack",
                 "n_tensor_params", "tensor_return_indices", "non_tensor_indices", "non_tensor_types", "mode", "plan",
                 "pack_kind")

    def __init__(self):
        self.param_types: List[Any] = []
        self.return_types: List[Any] = []
        self.in_payload = PayloadType.NO_PAYLOAD
        self.out_payload = PayloadType.NO_PAYLOAD
        self.encoded: dict = {}              # parameter index -> "vs" | "nli64" | "nlf64" | "nlb" | "ntl"
        self.param_from_dlpack: dict = {}    # parameter index -> from_dlpack callable or None
        self.n_tensor_params = 0
        self.tensor_return_indices: List[int] = []   # positions in the returned tuple
        self.non_tensor_indices: List[int] = []
        self.non_tensor_types: List[Any] = []
        self.mode = "void"                   # void | single | tensor | tensor_list | tuple
        self.plan = None                     # native counterpart of _params_to_args for this signature (see _register)
        self.pack_kind = None                # which branch of _pack_results this signature takes (see _register)


def _is_list_alias(t: Any) -> bool:
    return t is typing.List or typing.get_origin(t) in (list, typing.List) or getattr(t, "__origin__", None) is list


def _annotation_info(ann: Any):
    """Annotation -> (ParamType, blob tag or None, tensor type or None). TypeError for forms that can
    never be carried; UNKNOWN for types this layer does not know."""
    if ann is None or ann is type(None):
        return ParamType.UNKNOWN, None, None
    if ann is bool:
        return ParamType.PRIMITIVE_BOOL, None, None
    if ann is int:
        return ParamType.PRIMITIVE_INT64, None, None
    if ann is float:
        return ParamType.PRIMITIVE_FLOAT64, None, None
    if ann is str:
        return ParamType.STRING, None, None
    if hasattr(ann, "__dlpack__"):
        return ParamType.TENSOR_META, None, ann
    if _is_list_alias(ann):
        args = typing.get_args(ann)
        if not args:
            raise TypeError("List without type argument is not supported. Use List[int], List[float], List[str], List[bool], "
                            "List[Tensor], List[List[int]], List[List[float]], List[List[bool]], List[List[Tensor]] instead.")
        elem = args[0]
        if elem is int:
            return ParamType.VECTOR_INT64, None, None
        if elem is float:
            return ParamType.VECTOR_FLOAT64, None, None
        if elem is bool:
            return ParamType.VECTOR_BOOL, None, None
        if elem is str:
            return ParamType.STRING, _STR_LIST_TAG, None
        if _is_tensor_type(elem):
            return ParamType.TENSOR_META_VEC, None, elem
        if _is_list_alias(elem):
            inner = typing.get_args(elem)
            if not inner:
                raise TypeError("List[List[...]] requires explicit element type annotation (e.g. List[List[int]])")
            it = inner[0]
            if it is int:
                return ParamType.STRING, "nli64", None
            if it is float:
                return ParamType.STRING, "nlf64", None
            if it is bool:
                return ParamType.STRING, "nlb", None
            if _is_tensor_type(it):
                return ParamType.STRING, "ntl", it
            raise TypeError(f"Unsupported inner element type in List[List[...]]: '{it}'. Supported: int, float, bool, Tensor")
        raise TypeError(f"Unsupported List element type: '{elem}'. Supported: int, float, bool, str, Tensor, List[int], "
                        "List[float], List[bool], List[Tensor]")
    if isinstance(ann, type):
        for mod, cls in (("torch", "Tensor"), ("numpy", "ndarray"), ("jax", "Array"), ("tensorflow", "Tensor")):
            import sys
            m = sys.modules.get(mod)
            base = getattr(m, cls, None) if m is not None else None
            try:
                if base is not None and issubclass(ann, base):
                    return ParamType.TENSOR_META, None, ann
            except TypeError:
                pass
    return ParamType.UNKNOWN, None, None


def _callable_for_signature(fn: Callable):
    return fn if inspect.isfunction(fn) or inspect.ismethod(fn) else getattr(fn, "__call__", fn)


def _is_async_callable(fn: Any) -> bool:
    return inspect.iscoroutinefunction(fn) or inspect.iscoroutinefunction(getattr(fn, "__call__", None))


def _parse_signature(fn: Callable) -> _Sig:
    """Wire signature of ``fn`` from its annotations; parameters without one are UNKNOWN."""
    sig = _Sig()
    target = _callable_for_signature(fn)
    try:
        hints = typing.get_type_hints(target)
    except Exception:
        hints = {}
    isig = inspect.signature(fn)
    n_tensors, any_list = 0, False
    for idx, (pname, par) in enumerate(isig.parameters.items()):
        ann = hints.get(pname, par.annotation)
        if ann is inspect.Parameter.empty:
            sig.param_types.append(ParamType.UNKNOWN)
            continue
        ptype, tag, ttype = _annotation_info(ann)
        sig.param_types.append(ptype)
        if tag is not None:
            sig.encoded[idx] = tag
        if ptype in (ParamType.TENSOR_META, ParamType.TENSOR_META_VEC) or tag == "ntl":
            sig.param_from_dlpack[idx] = _default_from_dlpack(ttype) if isinstance(ttype, type) and not hasattr(ttype, "__dlpack__") or _is_known_framework(ttype) else getattr(ttype, "from_dlpack", None)
            sig.n_tensor_params += 1
            n_tensors += 1 if ptype == ParamType.TENSOR_META else 2
    if n_tensors == 1:
        sig.in_payload = PayloadType.UCX_BUFFER
    elif n_tensors > 1:
        sig.in_payload = PayloadType.UCX_BUFFER_VEC
    ret = hints.get("return", isig.return_annotation)
    if ret is inspect.Signature.empty:
        return sig
    if ret is None or ret is type(None):
        sig.return_types = [ParamType.VOID]
        return sig
    is_tuple = typing.get_origin(ret) in (tuple, typing.Tuple)
    anns = list(typing.get_args(ret)) if is_tuple else [ret]
    if ret is tuple:
        anns, is_tuple = [], True
        sig.non_tensor_types.append(ParamType.UNKNOWN)
        sig.non_tensor_indices.append(0)
    has_vec = False
    for i, a in enumerate(anns):
        ptype, _tag, _tt = _annotation_info(a)
        if ptype == ParamType.TENSOR_META:
            sig.tensor_return_indices.append(i)
        elif ptype == ParamType.TENSOR_META_VEC:
            has_vec = True
            sig.tensor_return_indices.append(i)
        else:
            sig.non_tensor_types.append(ptype)
            sig.non_tensor_indices.append(i)
    sig.return_types = list(sig.non_tensor_types)
    if len(sig.tensor_return_indices) == 1 and not has_vec:
        sig.return_types.append(ParamType.TENSOR_META)
        sig.out_payload = PayloadType.UCX_BUFFER
    elif sig.tensor_return_indices:
        sig.return_types.append(ParamType.TENSOR_META_VEC)
        sig.out_payload = PayloadType.UCX_BUFFER_VEC
    sig.mode = _return_mode(sig.return_types, bool(sig.tensor_return_indices), has_vec, is_tuple)
    return sig


def _is_known_framework(t: Any) -> bool:
    mod = getattr(t, "__module__", "") or ""
    return mod.startswith(("torch", "numpy", "jax"))


def _return_mode(return_types, has_tensors: bool, has_vec: bool, is_tuple: bool) -> str:
    if not return_types or (len(return_types) == 1 and return_types[0] == ParamType.VOID):
        return "void"
    if len(return_types) == 1 and not is_tuple:
        if has_tensors:
            return "tensor_list" if has_vec else "tensor"
        return "single"
    return "tuple"


def _sig_from_types(param_types, return_types, in_payload, out_payload, from_dlpack_fn) -> _Sig:
    """Signature of a function registered with explicit wire types (register_function_raw, long form)."""
    sig = _Sig()
    sig.param_types, sig.return_types = list(param_types), list(return_types)
    n_in = sum(1 if t == ParamType.TENSOR_META else 2 for t in sig.param_types if t in (ParamType.TENSOR_META, ParamType.TENSOR_META_VEC))
    sig.in_payload = PayloadType.UCX_BUFFER if n_in == 1 else PayloadType.UCX_BUFFER_VEC if n_in > 1 else in_payload
    for i, t in enumerate(sig.param_types):
        if t in (ParamType.TENSOR_META, ParamType.TENSOR_META_VEC):
            sig.param_from_dlpack[i] = from_dlpack_fn
            sig.n_tensor_params += 1
    has_vec = False
    for i, t in enumerate(sig.return_types):
        if t in (ParamType.TENSOR_META, ParamType.TENSOR_META_VEC):
            sig.tensor_return_indices.append(i)
            has_vec = has_vec or t == ParamType.TENSOR_META_VEC
        else:
            sig.non_tensor_indices.append(i)
            sig.non_tensor_types.append(t)
    n_out = len(sig.tensor_return_indices) + (1 if has_vec else 0)
    sig.out_payload = PayloadType.UCX_BUFFER if n_out == 1 else PayloadType.UCX_BUFFER_VEC if n_out > 1 else out_payload
    sig.mode = _return_mode(sig.return_types, bool(sig.tensor_return_indices), has_vec, len(sig.return_types) > 1)
    return sig


# ---- server side: header + payload -> positional arguments -> results ---------------------------
def _params_to_args(sig: _Sig, header, payload) -> list:
    """Positional arguments of the handler, in declaration order (reference:
    bindings_runtime_wrapper.cpp:97-329): every tensor-typed parameter draws from one stream of
    tensors, every other parameter from the non-tensor params in their order on the wire. The native plan does
    the same without the interpreter and leaves the rare forms (NotImplemented) to the code below."""
    if sig.plan is not None:
        args = sig.plan.args(header, payload)
        if args is not NotImplemented:
            return args
    plain, metas = _split_params(header.params_meta)
    stream = _TensorStream(payload, metas)
    args, pi = [], 0
    if not sig.param_types and payload is not None and not metas:
        return args
    for idx, ptype in enumerate(sig.param_types):
        tag = sig.encoded.get(idx)
        fn = sig.param_from_dlpack.get(idx)
        if tag == "ntl":
            if pi >= len(plain):
                raise RuntimeError(f"Missing group-sizes param for nested tensor list at index {idx}")
            sizes = plain[pi][1]
            pi += 1
            args.append([[stream.take(fn) for _ in range(int(n))] for n in sizes])
        elif ptype == ParamType.TENSOR_META:
            if stream.remaining() <= 0:
                raise RuntimeError(f"Tensor meta not found for parameter {idx}")
            args.append(stream.take(fn))
        elif ptype == ParamType.TENSOR_META_VEC:
            args.append([stream.take(fn) for _ in range(stream.remaining())])
        elif pi < len(plain):
            while pi < len(plain) and plain[pi][2] == _GROUP_SIZES:
                pi += 1          # sizes of a nested tensor list sent to a function that takes a flat list
            if pi < len(plain):
                args.append(plain[pi][1])
                pi += 1
    return args


def _tensor_payload(tensors: list, as_vec: bool):
    """(payload object, add_meta) for the tensors of a message. The native layer describes the tensors in
    the header itself (1: one TENSOR_META, 2: one TENSOR_META_VEC; always the last param), from the same
    DLPack export it takes the bytes from."""
    if not tensors:
        return None, 0
    if len(tensors) == 1 and not as_vec:
        return _contiguous(tensors[0], strided_ok=True), 1
    return [_contiguous(t) for t in tensors], 2


def _pack_kind(sig: _Sig) -> str:
    """The branch of ``_pack_results`` a signature takes: its return mode, or "inferred" when an annotation is
    missing or unknown and the wire form follows the value."""
    if sig.mode == "void" and not (sig.return_types and sig.return_types[0] == ParamType.UNKNOWN):
        return "void"
    if any(t == ParamType.UNKNOWN for t in sig.return_types) or not sig.return_types:
        return "inferred"
    return sig.mode


def _pack_results(sig: _Sig, result):
    """Handler return value -> (RpcResponseHeader with the plain result params, payload, add_meta)."""
    header = RpcResponseHeader()
    kind = sig.pack_kind or _pack_kind(sig)
    if kind == "tensor":
        if result is None:
            raise TypeError("the function returned None where its annotation promises a tensor")
        return header, _contiguous(result, strided_ok=True), 1
    if kind == "void":
        return header, None, 0

    add_typed, add_plain = header.add_result_typed, header.AddResult
    if kind == "inferred":
        return _pack_inferred(result, header, add_typed, add_plain)
    if kind == "single":
        _add_declared(add_typed, add_plain, sig.return_types[0], result)
        return header, None, 0
    if kind == "tensor_list":
        return (header, *_tensor_payload(list(result), True))
    items = tuple(result) if isinstance(result, (tuple, list)) else (result,)
    for ptype, i in zip(sig.non_tensor_types, sig.non_tensor_indices):
        _add_declared(add_typed, add_plain, ptype, items[i])
    tensors, as_vec = [], len(sig.tensor_return_indices) > 1
    for i in sig.tensor_return_indices:
        if _is_seq(items[i]):
            tensors.extend(items[i])
            as_vec = True
        else:
            tensors.append(items[i])
    return (header, *_tensor_payload(tensors, as_vec))


def _pack_inferred(result, header, add_typed, add_plain):
    """No usable return annotation: the wire form follows the value."""
    if result is None:
        return header, None, 0
    items = list(result) if isinstance(result, tuple) else [result]
    tensors, as_vec = [], False
    for it in items:
        if _is_tensor(it):
            tensors.append(it)
        elif _is_seq(it) and it and all(_is_tensor(x) for x in it):
            tensors.extend(it)
            as_vec = True
        else:
            _add_inferred(add_typed, add_plain, it)
    return (header, *_tensor_payload(tensors, as_vec or len(tensors) > 1))


# ---- client side --------------------------------------------------------------------------------
def _error_text(resp, fid: int, session_id: int) -> str:
    what = next((v for t, v, _n in resp.results_meta if t == ParamType.STRING), None)
    if not what:
        what = f"RPC invocation failed: {resp.status_category} error {resp.status_value}"
    if fid:
        what += f" (function_id: {fid})"
    if session_id:
        what += f" (session_id: {session_id})"
    return what


def _results_to_python(resp, payload, from_dlpack_fn, fid: int, session_id: int):
    """Response -> what the awaiting caller gets (reference: param_conversion.hpp:83-176): nothing ->
    None, one result -> the value (a tensor, or the list of tensors), several -> a tuple with the tensors
    spliced in after the plain values. The native function does the same without the interpreter and leaves
    failed responses and the rare forms (NotImplemented) to the code below."""
    out = _axon._results_to_python(resp, payload, from_dlpack_fn)
    if out is not NotImplemented:
        return out
    if not resp.ok:
        raise RuntimeError(_error_text(resp, fid, session_id))
    results = resp.results_meta
    plain, metas = _split_params(results)
    stream = _TensorStream(payload, metas)
    if len(results) == 1:
        ptype, value, _ = results[0]
        if ptype == ParamType.TENSOR_META:
            return stream.take(from_dlpack_fn)
        if ptype == ParamType.TENSOR_META_VEC:
            return [stream.take(from_dlpack_fn) for _ in range(len(metas))]
        return value
    out = []
    for ptype, value, _ in results:
        if ptype == ParamType.TENSOR_META:
            out.append(stream.take(from_dlpack_fn))
        elif ptype == ParamType.TENSOR_META_VEC:
            out.extend(stream.take(from_dlpack_fn) for _ in range(len(metas)))
        else:
            out.append(value)
    return tuple(out) if out else None


def _classify(obj: Any) -> str:
    """'tensor' | 'flat' | 'nested' | 'value' (reference: ClassifyArg, bindings_runtime_helpers.hpp:264-334)."""
    if _is_tensor(obj):
        return "tensor"
    if not _is_seq(obj):
        return "value"
    if len(obj) == 0:
        return "flat"
    first = obj[0]
    if _is_tensor(first):
        return "flat"
    if _is_seq(first):
        for inner in obj:
            if not _is_seq(inner):
                raise TypeError("Heterogeneous sequences are not supported as RPC arguments: expected all elements to be "
                                "sequences (list/tuple) for List[List[Tensor]]")
            if len(inner) == 0:
                continue
            head = inner[0]
            if _is_tensor(head):
                return "nested"
            if isinstance(head, (bool, int, float, str)):
                return "value"
            raise TypeError("Unsupported element type inside nested sequence: expected a DLPack-compatible tensor, int, "
                            "float, bool, or str for List[List[T]] argument")
    return "value"


class AxonRuntime(_axon.AxonRuntime):
    """The runtime as Python sees it: annotation-driven registration, raw registration with explicit
    wire types, ``invoke`` with natural arguments and ``invoke_raw`` with a prepared header
    (reference: axon/python/src/bindings_runtime.cpp:404-1018)."""

    def __init__(self, worker_name: str, thread_pool_size: int = 0, timeout=None, device=None, resource_manager=None):
        super().__init__(worker_name, thread_pool_size or 0, timeout, device, resource_manager)
        self._functions = {}

    # ---- server side ------------------------------------------------------------------------
    def _register(self, fid: int, name: str, sig: _Sig, fn: Callable, memory_policy, lifecycle_policy, wire_dtype=None) -> int:
        code = _wire_code(wire_dtype)
        sig.pack_kind = _pack_kind(sig)
        sig.plan = _axon._ArgPlan(list(sig.param_types), [i for i, tag in sig.encoded.items() if tag == "ntl"],
                                  [sig.param_from_dlpack.get(i) for i in range(len(sig.param_types))])
        if code:
            async def handler(header, payload):
                head, pay, add_meta = _pack_results(sig, await fn(*_params_to_args(sig, header, payload)))
                return head, _apply_wire_dtype(pay, wire_dtype), add_meta, code
        else:
            async def handler(header, payload):
                return _pack_results(sig, await fn(*_params_to_args(sig, header, payload)))

        ok = self._register_native(fid, name, sig.param_types, sig.return_types, sig.in_payload, sig.out_payload, handler,
                                   memory_policy, lifecycle_policy)
        if not ok:
            raise ValueError(f"function id {fid} ({name}) is already registered")
        self._functions[name] = fid
        return fid

    @staticmethod
    def _name_of(fn: Callable, function_name: Optional[str], fid: Optional[int]) -> str:
        return function_name or getattr(fn, "__name__", None) or f"function_{fid or 0}"

    def register_function(self, callable: Callable, function_id: Optional[int] = None, function_name: Optional[str] = None,
                          memory_policy: Optional[Callable] = None, lifecycle_policy: Optional[Callable] = None,
                          from_dlpack_fn: Optional[Callable] = None, wire_dtype=None) -> int:
        """Register ``async def callable(...)`` under ``function_id`` (default: the hash of its name and
        this worker's name). ``wire_dtype`` (float32, float16 or bfloat16; not in the reference): the floating-point
        tensors the function returns travel in that type; a single CUDA tensor is converted by the transfer
        kernel on its way, anything else before it is sent. Every parameter and the return need an annotation this layer can carry:
        ``int`` (INT64), ``float`` (FLOAT64), ``bool``, ``str``, a DLPack tensor type, ``List[...]`` of
        those, ``List[List[int|float|bool|Tensor]]``; ``Tuple[...]`` only as the return annotation."""
        if not _is_async_callable(callable):
            raise RuntimeError("register_function only accepts async functions. Please use 'async def' to define your function.")
        name = self._name_of(callable, function_name, function_id)
        fid = function_id if function_id is not None else function_id_from_name(name, self.worker_name)
        sig = _parse_signature(callable)
        for i, t in enumerate(sig.param_types):
            if t == ParamType.UNKNOWN:
                raise TypeError(f"Unsupported or missing type annotation for parameter {i} in function '{name}'. {_SUPPORTED}.")
        if any(t == ParamType.UNKNOWN for t in sig.return_types):
            raise TypeError(f"Unsupported or missing return type annotation for function '{name}'. {_SUPPORTED}, None.")
        # Small messages arrive in host memory without the memory_policy being asked, so they need a
        # from_dlpack function. The reference demands an explicit one here; this layer only does so when
        # the annotations give it nothing to derive one from (torch / numpy / jax types do).
        if memory_policy is not None and from_dlpack_fn is None and any(f is None for f in sig.param_from_dlpack.values()):
            raise RuntimeError(
                f"Function '{name}' has tensor parameters and custom memory_policy is set, but from_dlpack_fn is not provided. "
                "from_dlpack_fn is required for small messages, which arrive in host memory without the memory_policy being "
                "asked. Please provide from_dlpack_fn (e.g., numpy.from_dlpack, torch.from_dlpack, jax.dlpack.from_dlpack).")
        if from_dlpack_fn is not None:
            sig.param_from_dlpack = {i: from_dlpack_fn for i in sig.param_from_dlpack}
        return self._register(fid, name, sig, callable, memory_policy, lifecycle_policy, wire_dtype)

    def register_function_raw(self, function_id: int, *args, **kwargs) -> int:
        """Two forms, as in the reference:

        ``register_function_raw(function_id, function_name, param_types, return_types, input_payload_type,
        return_payload_type, callable, memory_policy=None, lifecycle_policy=None, from_dlpack_fn=None)``
        registers under explicit wire types;

        ``register_function_raw(function_id, callable, function_name=None, memory_policy=None,
        lifecycle_policy=None)`` infers them from the annotations (missing ones become UNKNOWN and the
        values decide at run time)."""
        long_names = ("function_name", "param_types", "return_types", "input_payload_type", "return_payload_type", "callable",
                      "memory_policy", "lifecycle_policy", "from_dlpack_fn")
        short_names = ("callable", "function_name", "memory_policy", "lifecycle_policy")
        is_long = "param_types" in kwargs or (args and isinstance(args[0], str))
        names = long_names if is_long else short_names
        if len(args) > len(names):
            raise TypeError("register_function_raw(): too many positional arguments")
        bound = dict(zip(names, args))
        for k, v in kwargs.items():
            if k not in names or k in bound:
                raise TypeError(f"register_function_raw(): unexpected or repeated argument '{k}'")
            bound[k] = v
        fn = bound.get("callable")
        required = long_names[:6] if is_long else ("callable",)
        missing = [k for k in required if k not in bound]
        if missing:
            raise TypeError(f"register_function_raw(): missing argument(s) {', '.join(missing)}")
        if not _is_async_callable(fn):
            raise RuntimeError("register_function_raw only accepts async functions. Please use 'async def' to define your function.")
        memory_policy, lifecycle_policy = bound.get("memory_policy"), bound.get("lifecycle_policy")
        if is_long:
            name = bound["function_name"]
            sig = _sig_from_types(bound["param_types"], bound["return_types"], bound["input_payload_type"],
                                  bound["return_payload_type"], bound.get("from_dlpack_fn"))
        else:
            name = self._name_of(fn, bound.get("function_name"), function_id)
            sig = _parse_signature(fn)
            if not sig.return_types:
                sig.return_types = [ParamType.UNKNOWN]
        return self._register(function_id, name, sig, fn, memory_policy, lifecycle_policy)

    # ---- remote GEMM: a weight resident on this runtime's GPU, callable by peers -----------------
    GEMM_FORMATS = {"bf16": 0, "fp8_block": 1, "mxfp8": 2}

    MX_SIBLING = 0x40000000   # weight_id | MX_SIBLING: the same fp8_block weight with its scales in the MX form

    def serve_gemm(self, weight_id: int, w, fmt: str = "bf16", max_m: int = 8192, pow2_scales: bool = True) -> None:
        """Make ``W[K, N]`` (a bf16 or fp32 tensor on this runtime's GPU) callable by peers as ``weight_id``.

        ``fmt``: ``"bf16"``; ``"fp8_block"`` (e4m3 with one fp32 scale per 128x128 block of W, callers send e4m3
        rows with one fp32 scale per 128 elements); ``"mxfp8"`` (e4m3 with one power-of-two scale per 32 elements
        of K on both operands, scaled inside the tensor core). The weight is converted once, here. A call is served by
        one kernel that reads the caller's X across NVLink while it computes and writes Y into the caller's memory.

        ``pow2_scales`` (``"fp8_block"``): the weight's block scales are chosen as powers of two. They are still
        fp32 scales per 128x128 block, and any caller is served as before; a caller whose own scales are powers
        of two as well (``remote_gemm(..., x_scale_pow2=True)``) is served by the MX kernel, which lets the tensor
        core apply the scales and is the faster of the two."""
        import torch

        from ..ops import remote_gemm as g
        code = self.GEMM_FORMATS[fmt]
        k, n = w.shape
        keep = []
        if fmt == "bf16":
            w_t, scale = w.to(torch.bfloat16).t().contiguous(), None
        elif fmt == "fp8_block":
            w_t, scale = g.quantize_blocks_128x128(w.to(torch.bfloat16).t().contiguous(), pow2=pow2_scales)
            if pow2_scales and n % 256 == 0 and max_m % 256 == 0 and weight_id < self.MX_SIBLING:
                chunks = g.mx_scale_chunks(g.block_scales_to_mx(scale, 128), True)
                self._gemm_add_weight(weight_id | self.MX_SIBLING, w_t.data_ptr(), n, k, self.GEMM_FORMATS["mxfp8"], max_m, chunks.data_ptr())
                keep.append(chunks)
        else:
            w_t, sf = g.quantize_mx(w.float().t().contiguous())
            scale = g.mx_scale_chunks(sf, True)
        self._gemm_add_weight(weight_id, w_t.data_ptr(), n, k, code, max_m, scale.data_ptr() if scale is not None else 0)
        if not hasattr(self, "_gemm_weights"):
            self._gemm_weights = {}
        self._gemm_weights[weight_id] = (w_t, scale, keep)      # the kernel reads them for as long as the weight is served

    def remote_gemm(self, x, y, *, worker_name: str, weight_id: int, x_scale=None, x_scale_pow2: bool = False):
        """``y[M, N] = x[M, K] @ W`` on ``worker_name``, where W is what that worker serves as ``weight_id``.
        ``x`` and ``y`` (and ``x_scale`` for the fp8 formats) are device tensors of this process that the callee's
        kernel reads and writes directly; they must stay untouched until the returned future resolves (to the
        kernel's status word, 0 when all went well). The request leaves once whatever produces ``x`` on the current
        stream has finished; that is waited for on a helper thread, not on the event loop.

        ``x_scale_pow2`` (an ``"fp8_block"`` weight served with ``pow2_scales``): ``x_scale`` [M, K/128] holds
        powers of two (``quantize_rows_1x128(x, pow2=True)``); the call is routed to the MX kernel. The result
        is the same block-scaled product. ``x_scale`` may also be given already in the MX form (uint8:
        ``mx_scale_chunks(block_scales_to_mx(scale, 1), False)``), which saves the conversion per call."""
        import torch
        if x_scale_pow2:
            if x_scale.dtype != torch.uint8:      # fp32 scales: brought into the MX form here; a caller that quantises
                from ..ops import remote_gemm as g    # X once and calls often converts once itself and passes the bytes
                x_scale = g.mx_scale_chunks(g.block_scales_to_mx(x_scale, 1), False)
            weight_id |= self.MX_SIBLING
        nb = lambda t: t.numel() * t.element_size()  # noqa: E731

        def call():
            fut = self._remote_gemm(worker_name, weight_id, x.shape[0], x.data_ptr(), nb(x), y.data_ptr(), nb(y),
                                    x_scale.data_ptr() if x_scale is not None else 0, nb(x_scale) if x_scale is not None else 0)
            if x_scale_pow2:
                fut.add_done_callback(lambda _f, keep=x_scale: None)   # the converted scales live until the kernel has read them
            return fut

        # the callee's kernel reads x as soon as the request arrives: the request leaves when x is complete
        producer = torch.cuda.current_stream(x.device)
        if producer.query():
            return call()

        async def when_produced():
            # the producer is waited for on a helper thread, so that this runtime's handlers keep running meanwhile
            await asyncio.get_running_loop().run_in_executor(None, producer.synchronize)
            return await call()

        return asyncio.ensure_future(when_produced())

    # ---- client side --------------------------------------------------------------------------
    def invoke_raw(self, worker_name: str, request_header: RpcRequestHeader, payload=None, memory_policy: Optional[Callable] = None):
        """Send a prepared header (and an optional payload: a tensor, a list of tensors, a ``UcxBuffer`` or
        ``UcxBufferVec``). The future resolves to the function's return value(s), as ``invoke`` does."""
        if request_header is None:
            raise RuntimeError("request_header cannot be None")
        fid, sid = request_header.function_id, request_header.session_id
        if payload is not None and not isinstance(payload, (UcxBuffer, UcxBufferVec)):
            payload = [_contiguous(t) for t in payload] if _is_seq(payload) else _contiguous(payload, strided_ok=True)
        return self._invoke_native(worker_name, request_header, payload, memory_policy, False,
                                   lambda resp, pay: _results_to_python(resp, pay, None, fid, sid))

    def invoke(self, *args, worker_name: str, session_id: int, function, workflow_id: int = 0,
               memory_policy: Optional[Callable] = None, from_dlpack_fn: Optional[Callable] = None, wire_dtype=None):
        """Call ``function`` (an id, or a name hashed with the worker name) on ``worker_name`` with natural
        arguments: values, tensors, lists of tensors, lists of lists of tensors. ``wire_dtype`` (float32, float16
        or bfloat16; not in the reference): floating-point tensor arguments travel in that type, a single CUDA
        tensor converted by the transfer kernel on its way (no converted copy is made first). Returns a future of the
        result: a single value, or a tuple of values, tensors included."""
        if isinstance(function, bool) or not isinstance(function, (int, str)):
            raise ValueError("function must be int (ID) or str (name)")
        fid = function if isinstance(function, int) else function_id_from_name(function, worker_name)
        header = RpcRequestHeader()
        header.session_id, header.function_id, header.workflow_id = session_id, fid, workflow_id
        tensors: list = []
        for a in args:
            kind = _classify(a)
            if kind == "tensor":
                tensors.append(a)
            elif kind == "flat":
                tensors.extend(a)
            elif kind == "nested":
                header.add_param_typed(ParamType.VECTOR_UINT32, [len(g) for g in a], _GROUP_SIZES)
                for g in a:
                    tensors.extend(g)
            else:
                _add_inferred(header.add_param_typed, header.AddParam, a)
        sample = tensors[0] if tensors else None
        payload, add_meta = _tensor_payload(tensors, len(tensors) > 1)
        fn = from_dlpack_fn or (_default_from_dlpack(sample) if sample is not None else None)
        code = 0
        if wire_dtype is not None:
            payload, code = _apply_wire_dtype(payload, wire_dtype), _wire_code(wire_dtype)
        # the response is unpacked on the loop thread by the binding itself and settles the future
        return self._invoke_native(worker_name, header, payload, memory_policy, False,
                                   lambda resp, pay: _results_to_python(resp, pay, fn, fid, session_id), add_meta, code)



__all__ = [
    "AxonRuntime", "ParamType", "PayloadType", "RpcErrc", "TensorMeta", "DLDevice", "DLDataType", "UcxBuffer", "UcxBufferVec",
    "DLPackCapsuleWrapper", "RpcRequestHeader", "RpcResponseHeader", "RpcFunctionSignature", "deserialize_signatures",
    "UcxMemoryResourceManager", "DefaultUcxMemoryResourceManager", "CudaMemoryResourceManager", "get_default_resource_manager",
    "get_device_context_handle", "function_id_from_name", "MemoryType",
    "SpinningSelector", "new_event_loop", "run",
    "Device", "DeviceType", "CpuDevice", "CudaDevice", "RocmDevice", "SyclDevice", "cpu", "cuda", "rocm", "sycl", "auto_detect",
]
