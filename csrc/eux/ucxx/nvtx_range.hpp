// Optional NVTX ranges around the phases of an RPC and of a device transfer, for timelines in
// Nsight Systems. Off unless EUX_NVTX=1 is set when the process starts; a range then costs one
// call into the (header-only) NVTX loader, which does nothing when no tool is attached.
// The reference has no tracing hooks beyond compile-time printf tracing
// (ucx_context/ucx_am_context/ucx_am_context.cpp:45-65).
//
// EUX_TRACE=1 writes the same ranges and marks to stderr as text lines
// "eux-trace <B|E|M> <name> <steady-clock ns> <thread>", for machines without a timeline tool.
#pragma once

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <thread>

#include <nvtx3/nvToolsExt.h>

namespace eux::ucxx {

inline bool nvtx_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("EUX_NVTX");
    return e && e[0] == '1';
  }();
  return on;
}

inline bool trace_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("EUX_TRACE");
    return e && e[0] == '1';
  }();
  return on;
}
inline void trace_line(char kind, const char* name) {
  const auto ns = std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
  std::fprintf(stderr, "eux-trace %c %s %lld %zu\n", kind, name, static_cast<long long>(ns),
               std::hash<std::thread::id>{}(std::this_thread::get_id()) % 100000);
}

class NvtxRange {
 public:
  explicit NvtxRange(const char* name) : name_(name), on_(nvtx_enabled()), trace_(trace_enabled()) {
    if (on_) nvtxRangePushA(name);
    if (trace_) trace_line('B', name_);
  }
  ~NvtxRange() {
    if (on_) nvtxRangePop();
    if (trace_) trace_line('E', name_);
  }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;

 private:
  const char* name_;
  bool on_;
  bool trace_;
};

inline void nvtx_mark(const char* name) {
  if (nvtx_enabled()) nvtxMarkA(name);
  if (trace_enabled()) trace_line('M', name);
}

}  // namespace eux::ucxx
