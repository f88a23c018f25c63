// Optional NVTX ranges around the phases of an RPC and of a device transfer, for timelines in
// Nsight Systems. Off unless EUX_NVTX=1 is set when the process starts; a range then costs one
// call into the (header-only) NVTX loader, which does nothing when no tool is attached.
// The reference has no tracing hooks beyond compile-time printf tracing
// (ucx_context/ucx_am_context/ucx_am_context.cpp:45-65).
#pragma once

#include <cstdlib>

#include <nvtx3/nvToolsExt.h>

namespace eux::ucxx {

inline bool nvtx_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("EUX_NVTX");
    return e && e[0] == '1';
  }();
  return on;
}

class NvtxRange {
 public:
  explicit NvtxRange(const char* name) : on_(nvtx_enabled()) {
    if (on_) nvtxRangePushA(name);
  }
  ~NvtxRange() {
    if (on_) nvtxRangePop();
  }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;

 private:
  bool on_;
};

inline void nvtx_mark(const char* name) {
  if (nvtx_enabled()) nvtxMarkA(name);
}

}  // namespace eux::ucxx
