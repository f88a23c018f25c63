// CUDA device context: binds the worker thread to one GPU with cudaSetDevice
// (the reference pushes/pops a CUcontext instead,
// ucx_context/cuda/ucx_cuda_context.hpp:48-73; with one process per GPU and the
// runtime API's primary context, selecting the device is all that is needed).
#pragma once

#include "eux/ucxx/cuda/ucx_cuda_macro.h"
#include "eux/ucxx/ucx_device_context.hpp"

namespace eux::ucxx {

class UcxAutoCudaDeviceContext final : public UcxAutoDeviceContext {
 public:
  explicit UcxAutoCudaDeviceContext(int device) : device_(device) {}
  std::unique_ptr<OperationRAII> operator()() override {
    struct Guard final : OperationRAII {
      int prev = -1;
      explicit Guard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        EUX_CUDA_CHECK(cudaSetDevice(dev));
      }
      ~Guard() override {
        if (prev >= 0) cudaSetDevice(prev);
      }
    };
    return std::make_unique<Guard>(device_);
  }
  int device_id() const override { return device_; }

 private:
  int device_;
};

}  // namespace eux::ucxx
