// Python bindings, part 3: what runs on every call between the wire form and a Python function's arguments and
// results (reference: axon/python/src/bindings_runtime_wrapper.cpp:97-329 for the handler's arguments,
// axon/python/src/param_conversion.hpp:83-176 for the caller's results).
//
// The package's Python layer holds the same logic in `_params_to_args` and `_results_to_python` and stays the
// definition of the behaviour; these functions do the common cases without the interpreter and answer
// NotImplemented for what they leave to it (several tensors packed into one host buffer, tensors without
// elements that came without a payload, a failed response, a payload object of a foreign type), always before
// anything has been taken out of the message.
#include "bindings_common.hpp"

namespace eux::python {

using rpc::ParamMeta;
using rpc::ParamType;
using rpc::TensorMeta;

namespace {

constexpr std::string_view kGroupSizes = "__ntl_group_sizes";

py::object not_implemented() { return py::reinterpret_borrow<py::object>(Py_NotImplemented); }

// numpy.from_dlpack, what a tensor without a from_dlpack of its own goes through
py::object default_from_dlpack() {
  static PyObject* fn = nullptr;  // kept for good: nothing of the interpreter's is released at exit
  if (!fn) fn = py::object(py::module_::import("numpy").attr("from_dlpack")).release().ptr();
  return py::reinterpret_borrow<py::object>(fn);
}

// torch.from_dlpack takes the bare capsule (and then leaves out its device and stream queries: the bytes are
// complete when the runtime hands them over); every other consumer gets an object with __dlpack__.
bool takes_capsule(py::handle fn) {
  static PyObject* torch_fn = nullptr;
  if (!torch_fn) {
    py::object modules = py::module_::import("sys").attr("modules");
    if (!modules.contains("torch")) return false;
    torch_fn = py::object(modules["torch"].attr("from_dlpack")).release().ptr();
  }
  return fn.ptr() == torch_fn;
}

// Non-tensor parameters in their order on the wire, and the tensor descriptions (the last TENSOR_META or
// TENSOR_META_VEC parameter wins, as in the Python layer).
struct Split {
  std::vector<const ParamMeta*> plain;
  std::vector<const TensorMeta*> metas;
};
Split split(const rpc::data::vector<ParamMeta>& params) {
  Split s;
  for (auto& p : params) {
    if (p.type == ParamType::TENSOR_META) {
      if (auto* m = std::get_if<TensorMeta>(&p.value)) {
        s.metas.clear();
        s.metas.push_back(m);
      }
    } else if (p.type == ParamType::TENSOR_META_VEC) {
      if (auto* v = std::get_if<rpc::TensorMetaVec>(&p.value)) {
        s.metas.clear();
        for (auto& m : *v) s.metas.push_back(&m);
      }
    } else {
      s.plain.push_back(&p);
    }
  }
  return s;
}

// The tensors of one message, in order. A tensor whose memory came from a memory policy is handed back as the
// very object the policy returned; everything else goes through `fn` (numpy.from_dlpack when there is none).
class TensorStream {
 public:
  TensorStream(py::handle payload, const std::vector<const TensorMeta*>& metas) : metas_(metas) {
    if (payload.is_none()) return;
    if (py::isinstance<PyBufferVec>(payload)) vec_ = &payload.cast<PyBufferVec&>();
    else if (py::isinstance<PyBuffer>(payload)) buf_ = &payload.cast<PyBuffer&>();
    else foreign_ = true;
  }
  // What this class leaves to the Python layer: a payload object of another type, several tensors packed into
  // one buffer, and tensors without elements that came without any payload (they are made there).
  bool unsupported() const {
    if (foreign_ || (buf_ && metas_.size() > 1)) return true;
    if (buf_ || vec_ || metas_.empty()) return false;
    for (auto* m : metas_)
      if (rpc::utils::TensorPayloadBytes(*m) != 0) return false;
    return true;
  }
  size_t size() const { return (buf_ || vec_) ? metas_.size() : 0; }
  size_t remaining() const { return size() > pos_ ? size() - pos_ : 0; }

  py::object take(py::handle fn) {
    const size_t i = pos_++;
    if (i >= size()) throw std::runtime_error("the message carries fewer tensors than the function takes");
    const TensorMeta& meta = *metas_[i];
    if (vec_) {
      if (!vec_->vec || i >= vec_->vec->size()) throw py::index_error("segment index out of range");
      const auto& seg = (*vec_->vec)[i];
      py::object owner = take_owner(seg.data);
      if (!owner.is_none()) return owner;
      if (rpc::utils::CalculateTensorSize(meta) > seg.size) throw py::value_error("the metadata describes more bytes than the segment holds");
      TensorMeta m = meta;
      m.device = device_of(vec_->vec->type(), vec_->device_id);
      return convert(fn, make_capsule(vec_->vec, seg.data, m), m);
    }
    if (buf_->buf) {
      py::object owner = take_owner(buf_->buf->data());
      if (!owner.is_none()) return owner;
    }
    if (!buf_->buf) throw py::value_error("empty buffer");
    if (rpc::utils::CalculateTensorSize(meta) > buf_->buf->size()) throw py::value_error("the metadata describes more bytes than the buffer holds");
    TensorMeta m = meta;
    m.device = device_of(buf_->buf->type(), buf_->device_id);
    return convert(fn, make_capsule(buf_->buf, buf_->buf->data(), m), m);
  }

 private:
  static py::object convert(py::handle fn, py::capsule capsule, const TensorMeta& m) {
    py::object f = (fn && !fn.is_none()) ? py::reinterpret_borrow<py::object>(fn) : default_from_dlpack();
    if (takes_capsule(f)) return f(capsule);
    return f(py::cast(DLPackCapsuleWrapper(std::move(capsule), m.device)));
  }
  const std::vector<const TensorMeta*>& metas_;
  PyBuffer* buf_ = nullptr;
  PyBufferVec* vec_ = nullptr;
  bool foreign_ = false;
  size_t pos_ = 0;
};

// How a registered function's parameters are drawn from a request: built once per registration.
class ArgPlan {
 public:
  ArgPlan(std::vector<ParamType> types, const std::vector<size_t>& nested_tensor_lists, std::vector<py::object> from_dlpack)
      : types_(std::move(types)), fns_(std::move(from_dlpack)), nested_(types_.size(), false) {
    fns_.resize(types_.size());
    for (size_t i : nested_tensor_lists)
      if (i < nested_.size()) nested_[i] = true;
  }

  // Positional arguments in declaration order: every tensor-typed parameter draws from one stream of tensors,
  // every other parameter from the non-tensor params in their order on the wire.
  py::object args(const rpc::RpcRequestHeader& header, py::handle payload) const {
    Split s = split(header.params);
    TensorStream stream(payload, s.metas);
    if (stream.unsupported()) return not_implemented();
    py::list out;
    size_t pi = 0;
    for (size_t idx = 0; idx < types_.size(); ++idx) {
      const ParamType t = types_[idx];
      py::handle fn = fns_[idx] ? py::handle(fns_[idx]) : py::handle();
      if (nested_[idx]) {
        if (pi >= s.plain.size()) throw std::runtime_error("Missing group-sizes param for nested tensor list at index " + std::to_string(idx));
        py::object sizes = param_to_python(*s.plain[pi++], true);
        py::list groups;
        for (auto n : sizes) {
          py::list group;
          const long count = py::int_(py::reinterpret_borrow<py::object>(n)).cast<long>();
          for (long k = 0; k < count; ++k) group.append(stream.take(fn));
          groups.append(std::move(group));
        }
        out.append(std::move(groups));
      } else if (t == ParamType::TENSOR_META) {
        if (stream.remaining() == 0) throw std::runtime_error("Tensor meta not found for parameter " + std::to_string(idx));
        out.append(stream.take(fn));
      } else if (t == ParamType::TENSOR_META_VEC) {
        py::list all;
        for (size_t k = stream.remaining(); k > 0; --k) all.append(stream.take(fn));
        out.append(std::move(all));
      } else if (pi < s.plain.size()) {
        // sizes of a nested tensor list sent to a function that takes a flat list
        while (pi < s.plain.size() && std::string_view(s.plain[pi]->name.data(), s.plain[pi]->name.size()) == kGroupSizes) ++pi;
        if (pi < s.plain.size()) out.append(param_to_python(*s.plain[pi++], true));
      }
    }
    return out;
  }

 private:
  std::vector<ParamType> types_;
  std::vector<py::object> fns_;
  std::vector<bool> nested_;
};

// Response -> what the awaiting caller gets: nothing -> None, one result -> the value (a tensor, or the list of
// tensors), several -> a tuple with the tensors spliced in where their description stands.
py::object results_to_python(const rpc::RpcResponseHeader& resp, py::handle payload, py::handle fn) {
  if (!resp.status.ok()) return not_implemented();  // the Python layer words the error
  Split s = split(resp.results);
  TensorStream stream(payload, s.metas);
  if (stream.unsupported()) return not_implemented();
  auto all_tensors = [&](py::list& into) {
    for (size_t k = s.metas.size(); k > 0; --k) into.append(stream.take(fn));
  };
  if (resp.results.size() == 1) {
    const ParamMeta& r = resp.results[0];
    if (r.type == ParamType::TENSOR_META) return stream.take(fn);
    if (r.type == ParamType::TENSOR_META_VEC) {
      py::list out;
      all_tensors(out);
      return out;
    }
    return param_to_python(r, true);
  }
  py::list out;
  for (auto& r : resp.results) {
    if (r.type == ParamType::TENSOR_META) out.append(stream.take(fn));
    else if (r.type == ParamType::TENSOR_META_VEC) all_tensors(out);
    else out.append(param_to_python(r, true));
  }
  if (out.empty()) return py::none();
  return py::tuple(out);
}

}  // namespace

void bind_call_conversion(py::module_& m) {
  py::class_<ArgPlan>(m, "_ArgPlan")
      .def(py::init<std::vector<ParamType>, const std::vector<size_t>&, std::vector<py::object>>(), py::arg("param_types"),
           py::arg("nested_tensor_lists"), py::arg("from_dlpack"))
      .def("args", &ArgPlan::args, py::arg("header"), py::arg("payload").none(true),
           "The handler's positional arguments, or NotImplemented for a message this path leaves to the Python layer.");
  m.def("_results_to_python", &results_to_python, py::arg("response"), py::arg("payload").none(true), py::arg("from_dlpack").none(true),
        "The caller's value(s) of a response, or NotImplemented for what this path leaves to the Python layer.");
}

}  // namespace eux::python
