/* Error-check helpers for CUDA runtime calls made by the host runtime. */
#ifndef EUX_UCX_CUDA_MACRO_H_
#define EUX_UCX_CUDA_MACRO_H_
#include <cuda_runtime_api.h>

#include <stdexcept>
#include <string>

#define EUX_CUDA_CHECK(expr)                                                                        \
  do {                                                                                              \
    cudaError_t eux_e_ = (expr);                                                                    \
    if (eux_e_ != cudaSuccess)                                                                      \
      throw std::runtime_error(std::string(#expr " failed: ") + cudaGetErrorString(eux_e_));        \
  } while (0)
#define EUX_CUDA_WARN(expr)                                                                         \
  do {                                                                                              \
    cudaError_t eux_e_ = (expr);                                                                    \
    (void)eux_e_;                                                                                   \
  } while (0)
#endif
