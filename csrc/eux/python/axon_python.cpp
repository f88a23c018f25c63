#include <execinfo.h>
#include <signal.h>
#include <unistd.h>

#include <cstdlib>

#include "bindings_common.hpp"

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

PYBIND11_MODULE(_axon, m) {
  m.doc() = "Axon tensor RPC runtime (native part)";
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
}
