// Entry point of the extension module (reference: axon/python/src/axon_python.cpp:31-39).
#include "bindings_common.hpp"

PYBIND11_MODULE(_axon, m) {
  m.doc() = "Axon tensor RPC runtime (native part)";
  eux::python::bind_types(m);
  eux::python::bind_runtime(m);
}
