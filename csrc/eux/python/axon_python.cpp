#include <execinfo.h>
#include <signal.h>
#include <unistd.h>

#include <cstdlib>

#include <cuda_runtime_api.h>

#include "bindings_common.hpp"
#include "dlpack_helpers.hpp"
#include "eux/ucxx/transport.hpp"

namespace {
// With EUX_BACKTRACE=1 in the environment a fatal signal prints the native call
// stack (module + offset per frame, resolvable with addr2line) before the
// default action runs. Off by default: Python's faulthandler owns the signals.
void fatal_signal_backtrace(int sig) {
  void* frames[64];
  int n = backtrace(frames, 64);
  const char msg[] = "eux: fatal signal, native frames:\n";
  (void)!write(2, msg, sizeof(msg) - 1);
  backtrace_symbols_fd(frames, n, 2);
  signal(sig, SIG_DFL);
  raise(sig);
}
}  // namespace

namespace {
namespace py = pybind11;
// Where the consumers of a received device tensor queue their work, as far as this layer can know: the tensor
// library's current stream on the thread that drops the tensor (it is dropped right after the code that used
// it). An event recorded there tells the transport when the ring slot under the tensor may be written again.
int consumer_event_on_torch_stream(int device, void** event) {
  namespace tr = eux::ucxx::transport;
  // not a Python thread, or no torch: the legacy default stream, with which blocking streams synchronise
  uintptr_t stream = 0;
  if (Py_IsInitialized() && PyGILState_Check()) {
    stream = eux::python::torch_current_stream(py::handle(), device);
  }
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != device && cudaSetDevice(device) != cudaSuccess) {
    cudaGetLastError();
    return tr::kConsumerDone;
  }
  cudaStream_t st = stream ? reinterpret_cast<cudaStream_t>(stream) : cudaStreamLegacy;
  int state = tr::kConsumerDone;
  if (cudaStreamQuery(st) == cudaErrorNotReady) {  // something is queued there: the slot waits for it
    cudaEvent_t ev = nullptr;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) == cudaSuccess) {
      if (cudaEventRecord(ev, st) == cudaSuccess) {
        *event = ev;
        state = tr::kConsumerEvent;
      } else {
        cudaEventDestroy(ev);
      }
    }
  }
  cudaGetLastError();
  if (prev != device && prev >= 0) cudaSetDevice(prev);
  return state;
}
}  // namespace

PYBIND11_MODULE(_axon, m) {
  m.doc() = "Axon tensor RPC runtime (native part)";
  if (eux::python::stream_ordering_enabled()) eux::ucxx::transport::set_consumer_event_hook(&consumer_event_on_torch_stream);
  if (const char* e = std::getenv("EUX_BACKTRACE"); e && e[0] == '1') {
    // its own stack, so that a stack overflow can still be reported
    static char alt_stack[1 << 16];
    stack_t ss{};
    ss.ss_sp = alt_stack;
    ss.ss_size = sizeof(alt_stack);
    sigaltstack(&ss, nullptr);
    struct sigaction sa{};
    sa.sa_handler = fatal_signal_backtrace;
    sa.sa_flags = SA_ONSTACK | SA_NODEFER;
    sigaction(SIGSEGV, &sa, nullptr);
    sigaction(SIGABRT, &sa, nullptr);
    sigaction(SIGBUS, &sa, nullptr);
  }
  eux::python::bind_types(m);
  eux::python::bind_runtime(m);
  eux::python::bind_call_conversion(m);
}
