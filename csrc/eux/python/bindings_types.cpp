// Python bindings, part 1: enums, DLPack/tensor metadata, buffers, RPC headers,
// signatures, parameter conversion (reference: axon/python/src/bindings_enums.cpp,
// bindings_types.cpp, param_conversion.cpp).
#include "bindings_common.hpp"

namespace eux::python {

using rpc::ParamMeta;
using rpc::ParamType;
using rpc::TensorMeta;

// ---- ParamMeta <-> Python ---------------------------------------------------------------
namespace {
// Nested lists and string lists travel as STRING parameters whose `name` says how to read the bytes
// (reference: axon/python/src/param_conversion.cpp:38-67, 104-146):
//   "nli64" / "nlf64" / "nlb":  [u32 groups][u32 size of each group][items: i64 / f64 / u8]
//   "vs":                       [u32 count]{[u32 length][bytes]}
// Returns a null object when the tag is not one of these or the bytes do not add up.
py::object decode_tagged_blob(std::string_view tag, const char* d, size_t n) {
  auto u32_at = [&](size_t off, uint32_t* v) {
    if (off + 4 > n) return false;
    std::memcpy(v, d + off, 4);
    return true;
  };
  if (tag == "vs") {
    uint32_t count = 0;
    if (!u32_at(0, &count)) return {};
    size_t off = 4;
    py::list out;
    for (uint32_t i = 0; i < count; ++i) {
      uint32_t len = 0;
      if (!u32_at(off, &len) || off + 4 + len > n) return {};
      out.append(py::str(d + off + 4, len));
      off += 4 + size_t(len);
    }
    return out;
  }
  const int kind = tag == "nli64" ? 0 : tag == "nlf64" ? 1 : tag == "nlb" ? 2 : -1;
  if (kind < 0) return {};
  uint32_t groups = 0;
  if (!u32_at(0, &groups) || 4 + size_t(groups) * 4 > n) return {};
  const size_t width = kind == 2 ? 1 : 8;
  size_t off = 4 + size_t(groups) * 4;
  py::list out;
  for (uint32_t g = 0; g < groups; ++g) {
    uint32_t sz = 0;
    u32_at(4 + size_t(g) * 4, &sz);
    if (off + size_t(sz) * width > n) return {};
    py::list inner;
    for (uint32_t i = 0; i < sz; ++i, off += width) {
      if (kind == 0) {
        int64_t v;
        std::memcpy(&v, d + off, 8);
        inner.append(py::int_(v));
      } else if (kind == 1) {
        double v;
        std::memcpy(&v, d + off, 8);
        inner.append(py::float_(v));
      } else {
        inner.append(py::bool_(d[off] != 0));
      }
    }
    out.append(std::move(inner));
  }
  return out;
}
}  // namespace

py::object param_to_python(const ParamMeta& p, bool decode_blobs) {
  return std::visit(
      [&](const auto& alt) -> py::object {
        using A = std::decay_t<decltype(alt)>;
        if constexpr (std::is_same_v<A, rpc::PrimitiveValue>) {
          return std::visit(
              [](auto x) -> py::object {
                using X = decltype(x);
                if constexpr (std::is_same_v<X, bool>) return py::bool_(x);
                else if constexpr (std::is_floating_point_v<X>) return py::float_(x);
                else return py::int_(x);
              },
              alt);
        } else if constexpr (std::is_same_v<A, rpc::VectorValue>) {
          return std::visit(
              [&](const auto& vec) -> py::object {
                using E = typename std::decay_t<decltype(vec)>::value_type;
                if constexpr (std::is_same_v<E, uint8_t>) {
                  return py::bytes(reinterpret_cast<const char*>(vec.data()), vec.size());
                } else {
                  py::list out;
                  for (auto x : vec) {
                    if constexpr (std::is_same_v<E, rpc::data::bool_t>) out.append(py::bool_(bool(x)));
                    else if constexpr (std::is_floating_point_v<E>) out.append(py::float_(x));
                    else out.append(py::int_(x));
                  }
                  return out;
                }
              },
              alt);
        } else if constexpr (std::is_same_v<A, rpc::data::string>) {
          if (decode_blobs && p.type == ParamType::STRING && !p.name.empty()) {
            py::object decoded = decode_tagged_blob(std::string_view(p.name.data(), p.name.size()), alt.data(), alt.size());
            if (decoded) return decoded;
          }
          PyObject* s = PyUnicode_DecodeUTF8(alt.data(), static_cast<Py_ssize_t>(alt.size()), nullptr);
          if (s) return py::reinterpret_steal<py::object>(s);
          PyErr_Clear();  // binary blob carried as a string parameter
          return py::bytes(alt.data(), alt.size());
        } else if constexpr (std::is_same_v<A, std::nullptr_t>) {
          return py::none();
        } else if constexpr (std::is_same_v<A, TensorMeta>) {
          return py::cast(alt);
        } else {
          py::list out;
          for (auto& m : alt) out.append(py::cast(m));
          return out;
        }
      },
      p.value);
}

namespace {
template <class T>
ParamMeta prim_param(ParamType t, T v) {
  return ParamMeta(t, rpc::ParamValue(std::in_place_type<rpc::PrimitiveValue>, rpc::PrimitiveValue(std::in_place_type<T>, v)));
}
template <class T, class Cast>
ParamMeta vec_param(ParamType t, py::handle seq, Cast cast) {
  rpc::data::vector<T> out;
  for (auto item : seq) out.push_back(cast(item));
  return ParamMeta(t, rpc::ParamValue(std::in_place_type<rpc::VectorValue>, rpc::VectorValue(std::in_place_type<rpc::data::vector<T>>, std::move(out))));
}
}  // namespace

// Convert with an explicit wire type.
ParamMeta python_to_param_typed(py::handle v, ParamType t) {
  auto i64 = [](py::handle h) { return h.cast<int64_t>(); };
  auto u64 = [](py::handle h) { return h.cast<uint64_t>(); };
  auto f64 = [](py::handle h) { return h.cast<double>(); };
  switch (t) {
    case ParamType::PRIMITIVE_BOOL: return prim_param<bool>(t, v.cast<bool>());
    case ParamType::PRIMITIVE_INT8: return prim_param<int8_t>(t, static_cast<int8_t>(i64(v)));
    case ParamType::PRIMITIVE_INT16: return prim_param<int16_t>(t, static_cast<int16_t>(i64(v)));
    case ParamType::PRIMITIVE_INT32: return prim_param<int32_t>(t, static_cast<int32_t>(i64(v)));
    case ParamType::PRIMITIVE_INT64: return prim_param<int64_t>(t, i64(v));
    case ParamType::PRIMITIVE_UINT8: return prim_param<uint8_t>(t, static_cast<uint8_t>(u64(v)));
    case ParamType::PRIMITIVE_UINT16: return prim_param<uint16_t>(t, static_cast<uint16_t>(u64(v)));
    case ParamType::PRIMITIVE_UINT32: return prim_param<uint32_t>(t, static_cast<uint32_t>(u64(v)));
    case ParamType::PRIMITIVE_UINT64: return prim_param<uint64_t>(t, u64(v));
    case ParamType::PRIMITIVE_FLOAT32: return prim_param<float>(t, static_cast<float>(f64(v)));
    case ParamType::PRIMITIVE_FLOAT64: return prim_param<double>(t, f64(v));
    case ParamType::VECTOR_BOOL: return vec_param<bool>(t, v, [](py::handle h) { return rpc::data::bool_t(h.cast<bool>()); });
    case ParamType::VECTOR_INT8: return vec_param<int8_t>(t, v, [&](py::handle h) { return static_cast<int8_t>(i64(h)); });
    case ParamType::VECTOR_INT16: return vec_param<int16_t>(t, v, [&](py::handle h) { return static_cast<int16_t>(i64(h)); });
    case ParamType::VECTOR_INT32: return vec_param<int32_t>(t, v, [&](py::handle h) { return static_cast<int32_t>(i64(h)); });
    case ParamType::VECTOR_INT64: return vec_param<int64_t>(t, v, i64);
    case ParamType::VECTOR_UINT8: {
      if (py::isinstance<py::bytes>(v) || py::isinstance<py::bytearray>(v)) {
        std::string s = py::isinstance<py::bytes>(v) ? std::string(v.cast<py::bytes>()) : std::string(py::bytes(v.cast<py::bytearray>()));
        rpc::data::vector<uint8_t> out(s.begin(), s.end());
        return ParamMeta(t, rpc::ParamValue(std::in_place_type<rpc::VectorValue>, rpc::VectorValue(std::in_place_type<rpc::data::vector<uint8_t>>, std::move(out))));
      }
      return vec_param<uint8_t>(t, v, [&](py::handle h) { return static_cast<uint8_t>(u64(h)); });
    }
    case ParamType::VECTOR_UINT16: return vec_param<uint16_t>(t, v, [&](py::handle h) { return static_cast<uint16_t>(u64(h)); });
    case ParamType::VECTOR_UINT32: return vec_param<uint32_t>(t, v, [&](py::handle h) { return static_cast<uint32_t>(u64(h)); });
    case ParamType::VECTOR_UINT64: return vec_param<uint64_t>(t, v, u64);
    case ParamType::VECTOR_FLOAT32: return vec_param<float>(t, v, [&](py::handle h) { return static_cast<float>(f64(h)); });
    case ParamType::VECTOR_FLOAT64: return vec_param<double>(t, v, f64);
    case ParamType::STRING: {
      std::string s = py::isinstance<py::bytes>(v) ? std::string(v.cast<py::bytes>()) : v.cast<std::string>();
      return ParamMeta(t, rpc::ParamValue(std::in_place_type<rpc::data::string>, std::move(s)));
    }
    case ParamType::VOID: return ParamMeta(t, rpc::ParamValue(nullptr));
    case ParamType::TENSOR_META: return ParamMeta(t, rpc::ParamValue(std::in_place_type<TensorMeta>, v.cast<TensorMeta>()));
    case ParamType::TENSOR_META_VEC: {
      rpc::TensorMetaVec out;
      for (auto item : v) out.push_back(item.cast<TensorMeta>());
      return ParamMeta(t, rpc::ParamValue(std::in_place_type<rpc::TensorMetaVec>, std::move(out)));
    }
    default: throw py::type_error("unsupported parameter type");
  }
}

// Infer the wire type from the Python value: bool, int -> INT64, float -> FLOAT64, str, bytes,
// None, TensorMeta, and flat lists of those (reference: bindings_types.cpp:266-278).
ParamMeta python_to_param(py::handle v) {
  if (v.is_none()) return python_to_param_typed(v, ParamType::VOID);
  if (py::isinstance<py::bool_>(v)) return python_to_param_typed(v, ParamType::PRIMITIVE_BOOL);
  if (py::isinstance<py::int_>(v)) return python_to_param_typed(v, ParamType::PRIMITIVE_INT64);
  if (py::isinstance<py::float_>(v)) return python_to_param_typed(v, ParamType::PRIMITIVE_FLOAT64);
  if (py::isinstance<py::str>(v)) return python_to_param_typed(v, ParamType::STRING);
  if (py::isinstance<py::bytes>(v) || py::isinstance<py::bytearray>(v)) return python_to_param_typed(v, ParamType::VECTOR_UINT8);
  if (py::isinstance<TensorMeta>(v)) return python_to_param_typed(v, ParamType::TENSOR_META);
  if (py::isinstance<py::list>(v) || py::isinstance<py::tuple>(v)) {
    py::sequence seq = py::reinterpret_borrow<py::sequence>(v);
    if (seq.size() == 0) return python_to_param_typed(v, ParamType::VECTOR_INT64);
    py::object first = seq[0];
    if (py::isinstance<TensorMeta>(first)) return python_to_param_typed(v, ParamType::TENSOR_META_VEC);
    if (py::isinstance<py::bool_>(first)) return python_to_param_typed(v, ParamType::VECTOR_BOOL);
    bool any_float = false;
    for (auto item : seq) {
      if (py::isinstance<py::float_>(item)) any_float = true;
      else if (!py::isinstance<py::int_>(item)) throw py::type_error("lists must hold only numbers, bools or TensorMeta");
    }
    return python_to_param_typed(v, any_float ? ParamType::VECTOR_FLOAT64 : ParamType::VECTOR_INT64);
  }
  throw py::type_error("value cannot be carried as an RPC parameter: " + std::string(py::str(py::type::of(v))));
}

// ---- buffers as Python objects ------------------------------------------------------------------
py::object PyBuffer::to_capsule_wrapper(const TensorMeta& meta) const {
  if (!buf) throw py::value_error("empty buffer");
  if (rpc::utils::CalculateTensorSize(meta) > buf->size()) throw py::value_error("the metadata describes more bytes than the buffer holds");
  TensorMeta m = meta;
  // the bytes are where this runtime received them: its device, whatever device the sender's tensor was on
  m.device = device_of(buf->type(), device_id);
  return py::cast(DLPackCapsuleWrapper(make_capsule(buf, buf->data(), m), m.device));
}
TensorMeta PyBuffer::bytes_meta() const {
  TensorMeta m;
  m.device = device_of(buf->type(), device_id);
  m.ndim = 1;
  m.dtype = {kDLUInt, 8, 1};
  m.shape = {static_cast<int64_t>(buf->size())};
  m.strides = {1};
  return m;
}

void bind_types(py::module_& m) {
  py::enum_<ParamType>(m, "ParamType")
      .value("PRIMITIVE_BOOL", ParamType::PRIMITIVE_BOOL).value("PRIMITIVE_INT8", ParamType::PRIMITIVE_INT8)
      .value("PRIMITIVE_INT16", ParamType::PRIMITIVE_INT16).value("PRIMITIVE_INT32", ParamType::PRIMITIVE_INT32)
      .value("PRIMITIVE_INT64", ParamType::PRIMITIVE_INT64).value("PRIMITIVE_UINT8", ParamType::PRIMITIVE_UINT8)
      .value("PRIMITIVE_UINT16", ParamType::PRIMITIVE_UINT16).value("PRIMITIVE_UINT32", ParamType::PRIMITIVE_UINT32)
      .value("PRIMITIVE_UINT64", ParamType::PRIMITIVE_UINT64).value("PRIMITIVE_FLOAT32", ParamType::PRIMITIVE_FLOAT32)
      .value("PRIMITIVE_FLOAT64", ParamType::PRIMITIVE_FLOAT64).value("VECTOR_BOOL", ParamType::VECTOR_BOOL)
      .value("VECTOR_INT8", ParamType::VECTOR_INT8).value("VECTOR_INT16", ParamType::VECTOR_INT16)
      .value("VECTOR_INT32", ParamType::VECTOR_INT32).value("VECTOR_INT64", ParamType::VECTOR_INT64)
      .value("VECTOR_UINT8", ParamType::VECTOR_UINT8).value("VECTOR_UINT16", ParamType::VECTOR_UINT16)
      .value("VECTOR_UINT32", ParamType::VECTOR_UINT32).value("VECTOR_UINT64", ParamType::VECTOR_UINT64)
      .value("VECTOR_FLOAT32", ParamType::VECTOR_FLOAT32).value("VECTOR_FLOAT64", ParamType::VECTOR_FLOAT64)
      .value("STRING", ParamType::STRING).value("VOID", ParamType::VOID).value("TENSOR_META", ParamType::TENSOR_META)
      .value("TENSOR_META_VEC", ParamType::TENSOR_META_VEC).value("UNKNOWN", ParamType::UNKNOWN);
  py::enum_<rpc::PayloadType>(m, "PayloadType")
      .value("UCX_BUFFER", rpc::PayloadType::UCX_BUFFER).value("UCX_BUFFER_VEC", rpc::PayloadType::UCX_BUFFER_VEC)
      .value("NO_PAYLOAD", rpc::PayloadType::NO_PAYLOAD)
      .value("MONOSTATE", rpc::PayloadType::MONOSTATE);
  py::enum_<rpc::RpcErrc>(m, "RpcErrc")
      .value("OK", rpc::RpcErrc::OK).value("CANCELLED", rpc::RpcErrc::CANCELLED).value("UNKNOWN", rpc::RpcErrc::UNKNOWN)
      .value("INVALID_ARGUMENT", rpc::RpcErrc::INVALID_ARGUMENT).value("DEADLINE_EXCEEDED", rpc::RpcErrc::DEADLINE_EXCEEDED)
      .value("NOT_FOUND", rpc::RpcErrc::NOT_FOUND).value("ALREADY_EXISTS", rpc::RpcErrc::ALREADY_EXISTS)
      .value("PERMISSION_DENIED", rpc::RpcErrc::PERMISSION_DENIED).value("RESOURCE_EXHAUSTED", rpc::RpcErrc::RESOURCE_EXHAUSTED)
      .value("FAILED_PRECONDITION", rpc::RpcErrc::FAILED_PRECONDITION).value("ABORTED", rpc::RpcErrc::ABORTED)
      .value("OUT_OF_RANGE", rpc::RpcErrc::OUT_OF_RANGE).value("UNIMPLEMENTED", rpc::RpcErrc::UNIMPLEMENTED)
      .value("INTERNAL", rpc::RpcErrc::INTERNAL).value("UNAVAILABLE", rpc::RpcErrc::UNAVAILABLE)
      .value("DATA_LOSS", rpc::RpcErrc::DATA_LOSS).value("UNAUTHENTICATED", rpc::RpcErrc::UNAUTHENTICATED);
  py::enum_<ucx_memory_type>(m, "MemoryType")
      .value("HOST", ucx_memory_type::HOST).value("CUDA", ucx_memory_type::CUDA).value("CUDA_MANAGED", ucx_memory_type::CUDA_MANAGED)
      .value("ROCM", ucx_memory_type::ROCM).value("UNKNOWN", ucx_memory_type::UNKNOWN);

  py::class_<DLDevice>(m, "DLDevice")
      .def(py::init([](int type, int id) { return DLDevice{static_cast<DLDeviceType>(type), id}; }), py::arg("device_type") = 1, py::arg("device_id") = 0)
      .def_property("device_type", [](const DLDevice& d) { return static_cast<int>(d.device_type); },
                    [](DLDevice& d, int t) { d.device_type = static_cast<DLDeviceType>(t); })
      .def_readwrite("device_id", &DLDevice::device_id)
      .def("__repr__", [](const DLDevice& d) { return "DLDevice(" + std::to_string(d.device_type) + ", " + std::to_string(d.device_id) + ")"; });
  py::class_<DLDataType>(m, "DLDataType")
      .def(py::init([](int code, int bits, int lanes) { return DLDataType{uint8_t(code), uint8_t(bits), uint16_t(lanes)}; }), py::arg("code") = 2,
           py::arg("bits") = 32, py::arg("lanes") = 1)
      .def_readwrite("code", &DLDataType::code).def_readwrite("bits", &DLDataType::bits).def_readwrite("lanes", &DLDataType::lanes)
      .def("__repr__", [](const DLDataType& d) { return "DLDataType(" + std::to_string(d.code) + ", " + std::to_string(d.bits) + ", " + std::to_string(d.lanes) + ")"; });
  py::class_<TensorMeta>(m, "TensorMeta")
      .def(py::init<>())
      .def_readwrite("device", &TensorMeta::device).def_readwrite("ndim", &TensorMeta::ndim).def_readwrite("dtype", &TensorMeta::dtype)
      .def_readwrite("byte_offset", &TensorMeta::byte_offset)
      .def_property("shape", [](const TensorMeta& t) { return std::vector<int64_t>(t.shape.begin(), t.shape.end()); },
                    [](TensorMeta& t, std::vector<int64_t> v) { t.shape.assign(v.begin(), v.end()); t.ndim = int32_t(v.size()); })
      .def_property("strides", [](const TensorMeta& t) { return std::vector<int64_t>(t.strides.begin(), t.strides.end()); },
                    [](TensorMeta& t, std::vector<int64_t> v) { t.strides.assign(v.begin(), v.end()); })
      .def("nbytes", [](const TensorMeta& t) { return rpc::utils::CalculateTensorSize(t); })
      .def_static("from_tensor", [](py::handle obj) {
        ImportedTensor t = import_tensor(obj);
        TensorMeta meta = t.meta;
        if (t.managed && t.managed->deleter) t.managed->deleter(t.managed);
        return meta;
      })
      .def("__repr__", [](const TensorMeta& t) {
        std::string s = "TensorMeta(shape=[";
        for (size_t i = 0; i < t.shape.size(); ++i) s += (i ? ", " : "") + std::to_string(t.shape[i]);
        return s + "], bits=" + std::to_string(t.dtype.bits) + ", device=" + std::to_string(t.device.device_type) + ":" + std::to_string(t.device.device_id) + ")";
      });

  py::class_<DLPackCapsuleWrapper>(m, "DLPackCapsuleWrapper")
      .def("__dlpack__", &DLPackCapsuleWrapper::dlpack)
      .def("__dlpack_device__", &DLPackCapsuleWrapper::dlpack_device)
      .def_property_readonly("consumed", &DLPackCapsuleWrapper::consumed);

  py::class_<PyBuffer>(m, "UcxBuffer")
      .def_property_readonly("size", [](const PyBuffer& b) { return b.buf ? b.buf->size() : 0; })
      .def_property_readonly("memory_type", [](const PyBuffer& b) { return b.buf ? b.buf->type() : ucx_memory_type::UNKNOWN; })
      .def_property_readonly("data_ptr", [](const PyBuffer& b) { return b.buf ? reinterpret_cast<uintptr_t>(b.buf->data()) : 0; })
      .def("to_dlpack", &PyBuffer::to_capsule_wrapper, py::arg("meta"), "A single-use DLPack holder that views this buffer as the tensor `meta` describes.")
      .def("to_capsule", [](const PyBuffer& b, const TensorMeta& meta) {
        if (!b.buf) throw py::value_error("empty buffer");
        if (rpc::utils::CalculateTensorSize(meta) > b.buf->size()) throw py::value_error("the metadata describes more bytes than the buffer holds");
        TensorMeta m = meta;
        m.device = device_of(b.buf->type(), b.device_id);
        return make_capsule(b.buf, b.buf->data(), m);
      }, py::arg("meta"), "The bare 'dltensor' capsule of the same view, for consumers that take capsules (torch.from_dlpack does, and skips its stream handling then).")
      .def("__dlpack__", [](const PyBuffer& b, py::args, py::kwargs) {
        auto m = b.bytes_meta();
        return make_capsule(b.buf, b.buf->data(), m);
      })
      .def("__dlpack_device__", [](const PyBuffer& b) {
        auto d = device_of(b.buf->type(), b.device_id);
        return py::make_tuple(static_cast<int>(d.device_type), d.device_id);
      })
      .def("owner", [](const PyBuffer& b) { return b.buf ? take_owner(b.buf->data()) : py::object(py::none()); },
           "The Python object that supplied this memory through a memory policy, if any (returned once).")
      .def("tobytes", [](const PyBuffer& b) {
        if (!b.buf || b.buf->type() != ucx_memory_type::HOST) throw py::value_error("tobytes() needs a host buffer");
        return py::bytes(static_cast<const char*>(b.buf->data()), b.buf->size());
      });
  py::class_<PyBufferVec>(m, "UcxBufferVec")
      .def("__len__", [](const PyBufferVec& v) { return v.vec ? v.vec->size() : 0; })
      .def_property_readonly("memory_type", [](const PyBufferVec& v) { return v.vec ? v.vec->type() : ucx_memory_type::UNKNOWN; })
      .def("sizes", [](const PyBufferVec& v) { return v.vec ? v.vec->data_sizes() : std::vector<size_t>{}; })
      .def("to_dlpack", [](const PyBufferVec& v, size_t i, const TensorMeta& meta) {
        if (!v.vec || i >= v.vec->size()) throw py::index_error("segment index out of range");
        if (rpc::utils::CalculateTensorSize(meta) > (*v.vec)[i].size) throw py::value_error("the metadata describes more bytes than the segment holds");
        TensorMeta m = meta;
        m.device = device_of(v.vec->type(), v.device_id);
        return DLPackCapsuleWrapper(make_capsule(v.vec, (*v.vec)[i].data, m), m.device);
      })
      .def("to_capsule", [](const PyBufferVec& v, size_t i, const TensorMeta& meta) {
        if (!v.vec || i >= v.vec->size()) throw py::index_error("segment index out of range");
        if (rpc::utils::CalculateTensorSize(meta) > (*v.vec)[i].size) throw py::value_error("the metadata describes more bytes than the segment holds");
        TensorMeta m = meta;
        m.device = device_of(v.vec->type(), v.device_id);
        return make_capsule(v.vec, (*v.vec)[i].data, m);
      })
      .def("owner", [](const PyBufferVec& v, size_t i) {
        if (!v.vec || i >= v.vec->size()) throw py::index_error("segment index out of range");
        return take_owner((*v.vec)[i].data);
      })
      .def("tobytes", [](const PyBufferVec& v, size_t i) {
        if (!v.vec || i >= v.vec->size()) throw py::index_error("segment index out of range");
        if (v.vec->type() != ucx_memory_type::HOST) throw py::value_error("tobytes() needs host memory");
        return py::bytes(static_cast<const char*>((*v.vec)[i].data), (*v.vec)[i].size);
      });

  // `params` / `results` give the values as Python objects (blobs decoded), which is what the
  // reference exposes (bindings_types.cpp:257, 299); `params_meta` / `results_meta` add the wire
  // type and the name tag for code that needs them.
  auto params_list = [](const rpc::data::vector<ParamMeta>& ps) {
    py::list out;
    for (auto& p : ps) out.append(param_to_python(p, true));
    return out;
  };
  auto params_meta_list = [](const rpc::data::vector<ParamMeta>& ps) {
    py::list out;
    for (auto& p : ps) out.append(py::make_tuple(p.type, param_to_python(p, true), py::str(p.name.data(), p.name.size())));
    return out;
  };
  py::class_<rpc::RpcRequestHeader>(m, "RpcRequestHeader")
      .def(py::init<>())
      .def_property("session_id", [](const rpc::RpcRequestHeader& h) { return h.session_id.v_; }, [](rpc::RpcRequestHeader& h, uint32_t v) { h.session_id.v_ = v; })
      .def_property("request_id", [](const rpc::RpcRequestHeader& h) { return h.request_id.v_; }, [](rpc::RpcRequestHeader& h, uint32_t v) { h.request_id.v_ = v; })
      .def_property("function_id", [](const rpc::RpcRequestHeader& h) { return h.function_id.v_; }, [](rpc::RpcRequestHeader& h, uint32_t v) { h.function_id.v_ = v; })
      .def_property("workflow_id", [](const rpc::RpcRequestHeader& h) { return h.workflow_id.v_; }, [](rpc::RpcRequestHeader& h, uint32_t v) { h.workflow_id.v_ = v; })
      .def_property_readonly("hlc", [](const rpc::RpcRequestHeader& h) { return h.hlc.Raw(); })
      .def("AddParam", [](rpc::RpcRequestHeader& h, py::handle v, const std::string& name) {
        ParamMeta p = python_to_param(v);
        p.name = rpc::data::string(name);
        h.params.push_back(std::move(p));
      }, py::arg("value"), py::arg("name") = "")
      .def("add_param_typed", [](rpc::RpcRequestHeader& h, ParamType t, py::handle v, const std::string& name) {
        ParamMeta p = python_to_param_typed(v, t);
        p.name = rpc::data::string(name);
        h.params.push_back(std::move(p));
      }, py::arg("type"), py::arg("value"), py::arg("name") = "")
      .def_property_readonly("params", [params_list](const rpc::RpcRequestHeader& h) { return params_list(h.params); })
      .def_property_readonly("params_meta", [params_meta_list](const rpc::RpcRequestHeader& h) { return params_meta_list(h.params); })
      .def("serialize", [](const rpc::RpcRequestHeader& h) {
        auto b = rpc::Serialize(h);
        return py::bytes(reinterpret_cast<const char*>(b.data()), b.size());
      })
      .def_static("deserialize", [](py::bytes data) {
        std::string s = data;
        return rpc::Deserialize<rpc::RpcRequestHeader>(s.data(), s.size());
      });
  py::class_<rpc::RpcResponseHeader>(m, "RpcResponseHeader")
      .def(py::init<>())
      .def_property("session_id", [](const rpc::RpcResponseHeader& h) { return h.session_id.v_; }, [](rpc::RpcResponseHeader& h, uint32_t v) { h.session_id.v_ = v; })
      .def_property("request_id", [](const rpc::RpcResponseHeader& h) { return h.request_id.v_; }, [](rpc::RpcResponseHeader& h, uint32_t v) { h.request_id.v_ = v; })
      .def_property("workflow_id", [](const rpc::RpcResponseHeader& h) { return h.workflow_id.v_; }, [](rpc::RpcResponseHeader& h, uint32_t v) { h.workflow_id.v_ = v; })
      .def_property_readonly("hlc", [](const rpc::RpcResponseHeader& h) { return h.hlc.Raw(); })
      .def_property_readonly("status_value", [](const rpc::RpcResponseHeader& h) { return h.status.value; })
      .def_property_readonly("status_category", [](const rpc::RpcResponseHeader& h) { return std::string(h.status.category_name); })
      .def_property_readonly("ok", [](const rpc::RpcResponseHeader& h) { return h.status.ok(); })
      .def("set_status", [](rpc::RpcResponseHeader& h, int value, const std::string& category) {
        h.status.value = value;
        h.status.category_name = rpc::data::string(category);
      })
      .def("AddResult", [](rpc::RpcResponseHeader& h, py::handle v, const std::string& name) {
        ParamMeta p = python_to_param(v);
        p.name = rpc::data::string(name);
        h.results.push_back(std::move(p));
      }, py::arg("value"), py::arg("name") = "")
      .def("add_result_typed", [](rpc::RpcResponseHeader& h, ParamType t, py::handle v, const std::string& name) {
        ParamMeta p = python_to_param_typed(v, t);
        p.name = rpc::data::string(name);
        h.results.push_back(std::move(p));
      }, py::arg("type"), py::arg("value"), py::arg("name") = "")
      .def_property_readonly("results", [params_list](const rpc::RpcResponseHeader& h) { return params_list(h.results); })
      .def_property_readonly("results_meta", [params_meta_list](const rpc::RpcResponseHeader& h) { return params_meta_list(h.results); })
      .def_property_readonly("status", [](const rpc::RpcResponseHeader& h) {
        py::dict d;
        d["value"] = py::int_(h.status.value);
        d["category_name"] = py::str(h.status.category_name.data(), h.status.category_name.size());
        return d;
      })
      .def("serialize", [](const rpc::RpcResponseHeader& h) {
        auto b = rpc::Serialize(h);
        return py::bytes(reinterpret_cast<const char*>(b.data()), b.size());
      })
      .def_static("deserialize", [](py::bytes data) {
        std::string s = data;
        return rpc::Deserialize<rpc::RpcResponseHeader>(s.data(), s.size());
      });
  py::class_<rpc::RpcFunctionSignature>(m, "RpcFunctionSignature")
      .def_property_readonly("instance_name", [](const rpc::RpcFunctionSignature& s) { return std::string(s.instance_name); })
      .def_property_readonly("id", [](const rpc::RpcFunctionSignature& s) { return s.id.v_; })
      .def_property_readonly("function_name", [](const rpc::RpcFunctionSignature& s) { return std::string(s.function_name); })
      .def_property_readonly("param_types", [](const rpc::RpcFunctionSignature& s) { return std::vector<ParamType>(s.param_types.begin(), s.param_types.end()); })
      .def_property_readonly("return_types", [](const rpc::RpcFunctionSignature& s) { return std::vector<ParamType>(s.return_types.begin(), s.return_types.end()); })
      .def_readonly("input_payload_type", &rpc::RpcFunctionSignature::input_payload_type)
      .def_readonly("return_payload_type", &rpc::RpcFunctionSignature::return_payload_type);
  m.def("deserialize_signatures", [](py::bytes data) {
    std::string s = data;
    auto sigs = rpc::RpcDispatcher::DeserializeSignatures(s.data(), s.size());
    return std::vector<rpc::RpcFunctionSignature>(sigs.begin(), sigs.end());
  });
  m.def("function_id_from_name", [](const std::string& fn, const std::string& worker) { return axon::utils::FunctionIdFromName(fn, worker); },
        "low 32 bits of MHash(function_name, worker_name)");
}

}  // namespace eux::python
