// Shared declarations of the pybind11 module `_axon`.
#pragma once

#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <memory>

#include "dlpack_helpers.hpp"
#include "eux/axon/axon_runtime.hpp"
#include "python_wake_manager.hpp"

namespace eux::python {

namespace py = pybind11;

// Buffers as Python sees them: shared, so DLPack exports can keep them alive.
struct PyBuffer {
  std::shared_ptr<ucxx::UcxBuffer> buf;
  int device_id = 0;
  py::object to_capsule_wrapper(const rpc::utils::TensorMeta& meta) const;
  rpc::utils::TensorMeta bytes_meta() const;
};
struct PyBufferVec {
  std::shared_ptr<ucxx::UcxBufferVec> vec;
  int device_id = 0;
};

// A Python object that C++ closures may hold and drop on any thread: the last
// reference is released with the GIL taken.
inline std::shared_ptr<py::object> gil_shared(py::object o) {
  return std::shared_ptr<py::object>(new py::object(std::move(o)), [](py::object* p) {
    if (Py_IsInitialized()) {
      py::gil_scoped_acquire gil;
      delete p;
    } else {
      (void)p->release();  // interpreter gone: leak rather than touch it
      delete p;
    }
  });
}

// decode_blobs: nested-list / string-list blobs (STRING parameters with a name tag) come back as lists
py::object param_to_python(const rpc::ParamMeta& p, bool decode_blobs = true);
rpc::ParamMeta python_to_param(py::handle v);
rpc::ParamMeta python_to_param_typed(py::handle v, rpc::ParamType t);

void bind_types(py::module_& m);
void bind_runtime(py::module_& m);
void bind_call_conversion(py::module_& m);

}  // namespace eux::python
