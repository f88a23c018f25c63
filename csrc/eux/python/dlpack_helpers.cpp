#include "dlpack_helpers.hpp"

#include <cuda_runtime_api.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

namespace eux::python {

ucx_memory_type_t memory_type_of(const DLDevice& dev) {
  switch (dev.device_type) {
    case kDLCPU:
    case kDLCUDAHost: return ucx_memory_type::HOST;
    case kDLCUDA: return ucx_memory_type::CUDA;
    case kDLCUDAManaged: return ucx_memory_type::CUDA_MANAGED;
    case kDLROCM: return ucx_memory_type::ROCM;
    case kDLROCMHost: return ucx_memory_type::HOST;
    case kDLOneAPI: return ucx_memory_type::ZE_DEVICE;
    default: return ucx_memory_type::UNKNOWN;
  }
}

DLDevice device_of(ucx_memory_type_t type, int device_id) {
  switch (type) {
    case ucx_memory_type::CUDA: return {kDLCUDA, device_id < 0 ? 0 : device_id};
    case ucx_memory_type::CUDA_MANAGED: return {kDLCUDAManaged, device_id < 0 ? 0 : device_id};
    case ucx_memory_type::ROCM: return {kDLROCM, device_id < 0 ? 0 : device_id};
    default: return {kDLCPU, 0};
  }
}

namespace {
// What this layer asks torch for on every call, looked up once (under the GIL; the references are never given
// back, so that nothing is destroyed after the interpreter has gone).
struct TorchHooks {
  PyObject* tensor_type = nullptr;   // torch.Tensor
  PyObject* to_dlpack = nullptr;     // torch.utils.dlpack.to_dlpack: the capsule without the checks of Tensor.__dlpack__
  PyObject* raw_stream = nullptr;    // torch._C._cuda_getCurrentRawStream, where this torch has it
  PyObject* current_stream = nullptr;  // torch.cuda.current_stream
};
const TorchHooks* torch_hooks() {
  static TorchHooks hooks;
  static bool ready = false;
  if (ready) return &hooks;
  py::object modules = py::module_::import("sys").attr("modules");
  if (!modules.contains("torch")) return nullptr;  // not loaded (yet): asked again next time
  try {
    py::object torch = modules["torch"];
    hooks.tensor_type = py::object(torch.attr("Tensor")).release().ptr();
    hooks.current_stream = py::object(torch.attr("cuda").attr("current_stream")).release().ptr();
    py::object c = py::getattr(torch, "_C", py::none());
    if (!c.is_none() && py::hasattr(c, "_cuda_getCurrentRawStream")) hooks.raw_stream = py::object(c.attr("_cuda_getCurrentRawStream")).release().ptr();
    py::object dl = py::module_::import("torch.utils.dlpack");
    hooks.to_dlpack = py::object(dl.attr("to_dlpack")).release().ptr();
  } catch (py::error_already_set&) {
    PyErr_Clear();
  }
  ready = true;
  return &hooks;
}

// A plain torch.Tensor (no subclass) that Tensor.__dlpack__ would export without complaint: its capsule comes
// from torch.utils.dlpack.to_dlpack, which skips the Python-level checks of __dlpack__ (about ten times the cost
// of the export itself). Everything else goes through __dlpack__ and gets its errors from there.
py::object export_capsule(py::handle obj) {
  if (std::strcmp(Py_TYPE(obj.ptr())->tp_name, "Tensor") == 0) {
    const TorchHooks* h = torch_hooks();
    if (h && h->to_dlpack && reinterpret_cast<PyObject*>(Py_TYPE(obj.ptr())) == h->tensor_type) {
      try {
        if (!obj.attr("requires_grad").cast<bool>() && !obj.attr("is_conj")().cast<bool>())
          return py::reinterpret_steal<py::object>(PyObject_CallOneArg(h->to_dlpack, obj.ptr()));
      } catch (py::error_already_set&) {
        PyErr_Clear();
      }
    }
  }
  if (!py::hasattr(obj, "__dlpack__")) throw py::type_error("object does not implement __dlpack__");
  return obj.attr("__dlpack__")();
}
}  // namespace

uintptr_t torch_current_stream(py::handle obj, int device) {
  try {
    const TorchHooks* h = torch_hooks();
    if (!h) return 0;
    if (obj) {
      // a tensor of another library works on the legacy default stream as far as this layer knows
      if (reinterpret_cast<PyObject*>(Py_TYPE(obj.ptr())) != h->tensor_type &&
          py::type::handle_of(obj).attr("__module__").cast<std::string>().rfind("torch", 0) != 0)
        return 0;
    } else {
      // nobody showed a torch tensor: torch's stream counts only once torch has a CUDA context of its own
      static bool initialized = false;
      if (!initialized) {
        initialized = py::module_::import("torch").attr("cuda").attr("is_initialized")().cast<bool>();
        if (!initialized) return 0;
      }
    }
    if (h->raw_stream) {
      py::object s = py::reinterpret_steal<py::object>(PyObject_CallOneArg(h->raw_stream, py::int_(device).ptr()));
      if (s) return s.cast<uintptr_t>();
      PyErr_Clear();
    }
    if (h->current_stream) return py::handle(h->current_stream)(device).attr("cuda_stream").cast<uintptr_t>();
  } catch (const std::exception&) {
    PyErr_Clear();
  }
  return 0;
}

ImportedTensor import_tensor(py::handle obj, bool allow_strided, int wire_dtype) {
  py::object cap_obj = export_capsule(obj);
  if (!cap_obj) throw py::error_already_set();
  if (!PyCapsule_IsValid(cap_obj.ptr(), "dltensor")) throw py::value_error("__dlpack__ did not return an unused 'dltensor' capsule");
  auto* managed = static_cast<DLManagedTensor*>(PyCapsule_GetPointer(cap_obj.ptr(), "dltensor"));
  if (!managed) throw py::error_already_set();
  // consume-once protocol: rename the capsule and drop its destructor; the tensor is ours now
  PyCapsule_SetName(cap_obj.ptr(), "used_dltensor");
  PyCapsule_SetDestructor(cap_obj.ptr(), nullptr);
  ImportedTensor t;
  t.managed = managed;
  try {
    t.meta = rpc::utils::TensorMeta(managed->dl_tensor);
    if (!t.meta.is_compact()) {
      const auto& dl = managed->dl_tensor;
      const unsigned elem_bits = unsigned(dl.dtype.bits) * (dl.dtype.lanes ? dl.dtype.lanes : 1);
      bool ok = allow_strided && dl.device.device_type == kDLCUDA && dl.ndim >= 1 && dl.ndim <= ucxx::kSendAttrMaxDims &&
                (elem_bits == 8 || elem_bits == 16 || elem_bits == 32 || elem_bits == 64 || elem_bits == 128);
      for (int i = 0; ok && i < dl.ndim; ++i) ok = t.meta.strides[i] >= 0 && t.meta.shape[i] > 0;
      if (!ok) throw py::value_error("only dense row-major tensors can be sent; call .contiguous() first");
      t.strided = true;
      t.src_strides.assign(t.meta.strides.begin(), t.meta.strides.end());
      int64_t st = 1;  // what arrives is dense
      for (int i = dl.ndim - 1; i >= 0; --i) {
        t.meta.strides[i] = st;
        st *= t.meta.shape[i];
      }
    }
  } catch (...) {
    if (managed->deleter) managed->deleter(managed);
    throw;
  }
  t.data = static_cast<char*>(managed->dl_tensor.data) + managed->dl_tensor.byte_offset;
  if (wire_dtype >= 1 && wire_dtype <= 3 && managed->dl_tensor.device.device_type == kDLCUDA && t.meta.ndim >= 1 &&
      t.meta.ndim <= ucxx::kSendAttrMaxDims && t.meta.dtype.lanes <= 1) {
    auto code_of = [](const DLDataType& d) -> int {
      if (d.code == kDLFloat && d.bits == 32) return 1;
      if (d.code == kDLFloat && d.bits == 16) return 2;
      if (d.code == kDLBfloat && d.bits == 16) return 3;
      return 0;
    };
    const int src = code_of(managed->dl_tensor.dtype);
    bool sane = src != 0 && src != wire_dtype;
    for (int i = 0; sane && i < t.meta.ndim; ++i) sane = t.meta.shape[i] > 0;
    if (sane) {
      if (!t.strided) t.src_strides.assign(managed->dl_tensor.strides ? managed->dl_tensor.strides : nullptr,
                                           managed->dl_tensor.strides ? managed->dl_tensor.strides + t.meta.ndim : nullptr);
      if (t.src_strides.empty()) t.src_strides.assign(t.meta.strides.begin(), t.meta.strides.end());  // compact: the row-major strides
      bool nonneg = true;
      for (auto v : t.src_strides) nonneg = nonneg && v >= 0;
      if (nonneg) {
        t.src_dtype = static_cast<uint8_t>(src);
        t.dst_dtype = static_cast<uint8_t>(wire_dtype);
        t.src_elem_size = src == 1 ? 4 : 2;
        t.strided = true;  // described to the transport by a layout, dense or not
        t.meta.dtype = wire_dtype == 1 ? DLDataType{kDLFloat, 32, 1} : (wire_dtype == 2 ? DLDataType{kDLFloat, 16, 1} : DLDataType{kDLBfloat, 16, 1});
        int64_t st = 1;
        for (int i = t.meta.ndim - 1; i >= 0; --i) {
          t.meta.strides[i] = st;
          st *= t.meta.shape[i];
        }
      }
    }
  }
  t.nbytes = rpc::utils::TensorPayloadBytes(t.meta);  // a rank-0 tensor travels as its one element
  t.meta.byte_offset = 0;  // the payload starts at the first element
  return t;
}

bool stream_ordering_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("EUX_STREAM_ORDERING");
    return !(e && e[0] == '0');
  }();
  return on;
}

std::shared_ptr<const ucxx::UcxSendAttr> make_send_attr(const ImportedTensor* one, int device, uintptr_t stream) {
  auto attr = std::make_shared<ucxx::UcxSendAttr>();
  if (one && one->strided) {
    const auto& m = one->meta;
    attr->ndim = m.ndim;
    attr->elem_size = one->src_elem_size ? one->src_elem_size : (unsigned(m.dtype.bits) * (m.dtype.lanes ? m.dtype.lanes : 1) + 7) / 8;
    attr->src_dtype = one->src_dtype;
    attr->dst_dtype = one->dst_dtype;
    uint64_t last = 0;
    for (int i = 0; i < m.ndim; ++i) {
      attr->shape[i] = m.shape[i];
      attr->stride[i] = one->src_strides[i];
      last += uint64_t(m.shape[i] - 1) * uint64_t(one->src_strides[i]);
    }
    attr->span_bytes = (last + 1) * attr->elem_size;
    attr->dense_bytes = one->nbytes;
  }
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != device) cudaSetDevice(device);
  cudaStream_t producer = stream ? reinterpret_cast<cudaStream_t>(stream) : cudaStreamLegacy;
  if (!stream_ordering_enabled() || cudaStreamQuery(producer) == cudaSuccess) {
    // nothing is queued on the producer's stream: the tensor is complete (and free to be written) as it is
    if (prev != device && prev >= 0) cudaSetDevice(prev);
    if (attr->ndim == 0) return nullptr;
    return attr;
  }
  cudaGetLastError();
  cudaEvent_t ev = nullptr;
  if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) == cudaSuccess) {
    if (cudaEventRecord(ev, producer) == cudaSuccess) {
      attr->ready_event = ev;
      attr->device = device;
      attr->keep = std::shared_ptr<void>(ev, [device](void* e) {
        int cur = -1;
        cudaGetDevice(&cur);
        if (cur != device) cudaSetDevice(device);
        cudaEventDestroy(static_cast<cudaEvent_t>(e));
        if (cur != device && cur >= 0) cudaSetDevice(cur);
      });
    } else {
      cudaEventDestroy(ev);
    }
  }
  cudaGetLastError();
  if (prev != device && prev >= 0) cudaSetDevice(prev);
  if (!attr->ready_event) {
    // no event to go by: wait here, once, so that what is sent is at least complete
    cudaStreamSynchronize(producer);
    cudaGetLastError();
    if (attr->ndim == 0) return nullptr;
  }
  return attr;
}

namespace {
// the deleter may touch Python objects (the producer's tensor): take the GIL
ucxx::ucp_release_fn_t managed_deleter(DLManagedTensor* m) {
  auto holder = std::shared_ptr<DLManagedTensor>(m, [](DLManagedTensor* p) {
    if (!p || !p->deleter) return;
    if (Py_IsInitialized()) {
      py::gil_scoped_acquire gil;
      p->deleter(p);
    }
  });
  return [holder](void*) mutable { holder.reset(); };
}
}  // namespace

ucxx::UcxBuffer to_ucx_buffer(ucxx::UcxMemoryResourceManager& mr, ImportedTensor&& t) {
  auto type = memory_type_of(t.meta.device);
  if (type == ucx_memory_type::UNKNOWN) {
    if (t.managed && t.managed->deleter) t.managed->deleter(t.managed);
    throw py::value_error("tensors on this device type cannot be sent");
  }
  return ucxx::UcxBuffer(mr, type, t.data, t.nbytes, nullptr, true, managed_deleter(t.managed));
}

ucxx::UcxBufferVec to_ucx_buffer_vec(ucxx::UcxMemoryResourceManager& mr, std::vector<ImportedTensor>&& ts) {
  if (ts.empty()) return ucxx::UcxBufferVec(mr, ucx_memory_type::HOST, std::vector<size_t>{});
  const auto type = memory_type_of(ts.front().meta.device);
  std::vector<ucx_buffer_t> ranges;
  // one release function for the whole vector: it runs once per range, the owners go with the last one
  auto owners = std::make_shared<std::vector<ucxx::ucp_release_fn_t>>();
  for (auto& t : ts) {
    if (memory_type_of(t.meta.device) != type) {
      for (auto& u : ts)
        if (u.managed && u.managed->deleter) u.managed->deleter(u.managed);
      throw py::value_error("all tensors of one call must live on the same kind of device");
    }
    ranges.push_back({t.data, t.nbytes});
    owners->push_back(managed_deleter(t.managed));
  }
  return ucxx::UcxBufferVec(mr, type, std::move(ranges), nullptr, true, [owners](void*) mutable {
    if (owners) {
      for (auto& f : *owners) f(nullptr);
      owners.reset();
    }
  });
}

py::capsule DLPackCapsuleWrapper::dlpack(py::args, py::kwargs) {
  if (consumed_) throw py::value_error("this DLPack capsule was already consumed");
  consumed_ = true;
  return std::move(capsule_);
}

namespace {
struct ExportCtx {
  std::shared_ptr<void> keep;
  std::vector<int64_t> shape, strides;
  DLManagedTensor managed{};
};
void export_deleter(DLManagedTensor* self) { delete static_cast<ExportCtx*>(self->manager_ctx); }
}  // namespace

py::capsule make_capsule(std::shared_ptr<void> keep_alive, void* data, const rpc::utils::TensorMeta& meta) {
  // The description may have come from another process. What is handed to a tensor library here decides which
  // bytes that library will read, so only the shape and the type are taken from it: rank and shape must agree,
  // the element must be whole bytes, and the strides are always the dense ones (what travels is dense; strides
  // from the wire could point anywhere). The callers have checked the byte count against the buffer.
  const unsigned bits = unsigned(meta.dtype.bits) * (meta.dtype.lanes ? meta.dtype.lanes : 1);
  if (meta.ndim < 0 || meta.ndim > 64 || size_t(meta.ndim) != meta.shape.size() || bits == 0 || bits % 8 != 0 ||
      rpc::utils::CalculateTensorSize(meta) == static_cast<size_t>(-1))
    throw py::value_error("the metadata does not describe a tensor");
  auto* ctx = new ExportCtx();
  ctx->keep = std::move(keep_alive);
  ctx->shape.assign(meta.shape.begin(), meta.shape.end());
  ctx->strides.assign(size_t(meta.ndim), 1);
  for (int i = meta.ndim - 2; i >= 0; --i) ctx->strides[i] = ctx->strides[i + 1] * std::max<int64_t>(ctx->shape[i + 1], 1);
  DLTensor& t = ctx->managed.dl_tensor;
  t.data = data;
  t.device = meta.device;
  t.ndim = meta.ndim;
  t.dtype = meta.dtype;
  t.shape = ctx->shape.empty() ? nullptr : ctx->shape.data();
  t.strides = ctx->strides.empty() ? nullptr : ctx->strides.data();
  t.byte_offset = 0;
  ctx->managed.manager_ctx = ctx;
  ctx->managed.deleter = export_deleter;
  // if nobody consumes the capsule its destructor releases the tensor; a consumer renames it first
  return py::capsule(&ctx->managed, "dltensor", [](PyObject* cap) {
    if (PyCapsule_IsValid(cap, "dltensor")) {
      auto* m = static_cast<DLManagedTensor*>(PyCapsule_GetPointer(cap, "dltensor"));
      if (m && m->deleter) m->deleter(m);
    }
  });
}

namespace {
std::mutex& owners_mu() {
  static std::mutex m;
  return m;
}
std::unordered_map<const void*, py::object>& owners() {
  static auto* m = new std::unordered_map<const void*, py::object>();  // leaked: outlives interpreter shutdown order
  return *m;
}
}  // namespace

void remember_owner(const void* data, py::object owner) {
  std::lock_guard lk(owners_mu());
  owners()[data] = std::move(owner);
}
py::object take_owner(const void* data) {
  std::lock_guard lk(owners_mu());
  auto it = owners().find(data);
  if (it == owners().end()) return py::none();
  py::object o = std::move(it->second);
  owners().erase(it);
  return o;
}

}  // namespace eux::python
