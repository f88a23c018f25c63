// Device context: a factory of RAII guards that bind the calling thread to a
// device for the lifetime of the guard. The active-message context holds one
// guard while it is constructed and one for its whole run loop (reference:
// ucx_context/ucx_device_context.hpp:38-150, used at ucx_am_context.cpp:88-94, 237-240).
#pragma once

#include <memory>

namespace eux::ucxx {

class OperationRAII {
 public:
  virtual ~OperationRAII() = default;
};

class UcxAutoDeviceContext {
 public:
  virtual ~UcxAutoDeviceContext() = default;
  // Activate the device on the calling thread; the returned guard deactivates it.
  virtual std::unique_ptr<OperationRAII> operator()() = 0;
  virtual int device_id() const { return -1; }
};

// No device: guards do nothing.
class UcxAutoDefaultDeviceContext final : public UcxAutoDeviceContext {
 public:
  std::unique_ptr<OperationRAII> operator()() override { return std::make_unique<OperationRAII>(); }
};

}  // namespace eux::ucxx
