// DLPack interop for the Python bindings: tensors enter as zero-copy UcxBuffer
// views that keep their Python owner alive through the release function, and
// buffers leave as "dltensor" capsules following the consume-once protocol
// (reference: axon/python/src/dlpack_helpers.{hpp,cpp}).
#pragma once

#include "eux/ucxx/ucx_send_attr.hpp"

#include <pybind11/pybind11.h>

#include <memory>
#include <vector>

#include "eux/dlpack.h"
#include "eux/rpc/utils/tensor_meta.hpp"
#include "eux/ucxx/ucx_context_data.hpp"

namespace eux::python {

namespace py = pybind11;

ucx_memory_type_t memory_type_of(const DLDevice& dev);
DLDevice device_of(ucx_memory_type_t type, int device_id);

// The result of consuming obj.__dlpack__(): the managed tensor (owned by us now) and its metadata.
struct ImportedTensor {
  DLManagedTensor* managed = nullptr;
  rpc::utils::TensorMeta meta;
  void* data = nullptr;   // data pointer with byte_offset applied
  size_t nbytes = 0;      // size as a message: the elements, densely
  // a device tensor that is not dense row-major and was taken as it lies (`meta` then describes the dense
  // tensor that arrives at the other end; these are the strides it has here)
  bool strided = false;
  std::vector<int64_t> src_strides;
  // the elements travel in another floating-point type (kernel codes: 1 fp32, 2 fp16, 3 bf16; 0: as they are);
  // `meta` and `nbytes` then describe the converted tensor
  uint8_t src_dtype = 0, dst_dtype = 0;
  uint32_t src_elem_size = 0;
};
// Calls obj.__dlpack__() (any object that implements the protocol), takes the capsule's tensor.
// Throws when the tensor is not compact (dense row-major), unless `allow_strided` and it lives on a CUDA
// device with no negative stride and at most 8 dimensions: the transport gathers such a view itself.
// `wire_dtype` (1 fp32, 2 fp16, 3 bf16; 0: none): a CUDA tensor of another one of these types is announced in
// that type and converted by the transfer kernel on the way.
ImportedTensor import_tensor(py::handle obj, bool allow_strided = false, int wire_dtype = 0);
// torch's current stream on `device` as a cudaStream_t in an integer, when the tensor library in use is torch
// (`obj`: a tensor that tells, or null to go by whether torch is loaded at all); 0 otherwise: the legacy default
// stream, with which every blocking stream synchronises.
uintptr_t torch_current_stream(py::handle obj, int device);
// The remarks for the transport about a device tensor that is about to be sent: its layout when it was
// imported strided, and an event recorded now on the producer's stream (`stream`: a cudaStream_t as an
// integer; 0: the legacy default stream), so that nobody has to wait for the producer here. Null for host tensors.
// EUX_STREAM_ORDERING=0 turns off everything this layer does to order the transport after the tensor library's
// streams (events behind producers, behind the previous users of receive buffers, behind the consumers of ring
// slots), for applications that synchronise their streams themselves before they send and after they receive.
bool stream_ordering_enabled();
std::shared_ptr<const ucxx::UcxSendAttr> make_send_attr(const ImportedTensor* one, int device, uintptr_t stream);
// A non-copying buffer over the tensor; releasing it calls the DLPack deleter (under the GIL).
ucxx::UcxBuffer to_ucx_buffer(ucxx::UcxMemoryResourceManager& mr, ImportedTensor&& t);
// One buffer vector over several tensors (all on one device kind).
ucxx::UcxBufferVec to_ucx_buffer_vec(ucxx::UcxMemoryResourceManager& mr, std::vector<ImportedTensor>&& ts);

// A single-use holder of a DLPack capsule: frameworks' from_dlpack() call its __dlpack__().
class DLPackCapsuleWrapper {
 public:
  DLPackCapsuleWrapper(py::capsule capsule, DLDevice device) : capsule_(std::move(capsule)), device_(device) {}
  py::capsule dlpack(py::args, py::kwargs);  // __dlpack__(stream=None, ...)
  py::tuple dlpack_device() const { return py::make_tuple(static_cast<int>(device_.device_type), device_.device_id); }
  bool consumed() const { return consumed_; }

 private:
  py::capsule capsule_;
  DLDevice device_;
  bool consumed_ = false;
};

// Export `bytes [offset, offset+size)` of a shared buffer as a tensor described by `meta`.
// The capsule keeps the buffer alive until the consumer's deleter runs.
py::capsule make_capsule(std::shared_ptr<void> keep_alive, void* data, const rpc::utils::TensorMeta& meta);

// Python owners of buffers that were supplied by a Python memory policy: when such a buffer
// comes back with data, the very same Python object is handed to the caller.
void remember_owner(const void* data, py::object owner);
py::object take_owner(const void* data);  // None when unknown

}  // namespace eux::python
