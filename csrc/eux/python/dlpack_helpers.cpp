#include "dlpack_helpers.hpp"

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

ImportedTensor import_tensor(py::handle obj) {
  if (!py::hasattr(obj, "__dlpack__")) throw py::type_error("object does not implement __dlpack__");
  py::object cap_obj = obj.attr("__dlpack__")();
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
    if (!t.meta.is_compact()) throw py::value_error("only dense row-major tensors can be sent; call .contiguous() first");
  } catch (...) {
    if (managed->deleter) managed->deleter(managed);
    throw;
  }
  t.data = static_cast<char*>(managed->dl_tensor.data) + managed->dl_tensor.byte_offset;
  t.nbytes = rpc::utils::CalculateTensorSize(t.meta);
  if (t.meta.ndim == 0) t.nbytes = (t.meta.dtype.bits * (t.meta.dtype.lanes ? t.meta.dtype.lanes : 1) + 7) / 8;
  t.meta.byte_offset = 0;  // the payload starts at the first element
  return t;
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
  auto* ctx = new ExportCtx();
  ctx->keep = std::move(keep_alive);
  ctx->shape.assign(meta.shape.begin(), meta.shape.end());
  ctx->strides.assign(meta.strides.begin(), meta.strides.end());
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
