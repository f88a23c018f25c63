// Hands closures from C++ threads to the asyncio thread: a mutex-protected queue
// plus an eventfd that the event loop watches with loop.add_reader(). The
// closures run on the loop's thread with the GIL held
// (reference: axon/python/src/python_wake_manager.{hpp,cpp}).
#pragma once

#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <sys/eventfd.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <deque>
#include <functional>
#include <mutex>

namespace eux::python {

namespace py = pybind11;

// Closures queued by any manager of this process and not yet taken by its loop. A loop that prefers to
// spin for a while before it sleeps in the selector watches this one word.
inline std::atomic<int64_t>& pending_wakes() {
  static std::atomic<int64_t> n{0};
  return n;
}

// Spins (GIL released by the caller) until a closure is queued or `budget` has passed.
inline bool spin_for_wake(std::chrono::nanoseconds budget) {
  auto& n = pending_wakes();
  const auto end = std::chrono::steady_clock::now() + budget;
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      if (n.load(std::memory_order_acquire) > 0) return true;
#if defined(__x86_64__)
      __builtin_ia32_pause();
#endif
    }
    if (std::chrono::steady_clock::now() >= end) return n.load(std::memory_order_acquire) > 0;
  }
}

class PythonWakeManager {
 public:
  PythonWakeManager() {
    fd_ = ::eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
    if (fd_ < 0) throw std::runtime_error("eventfd failed");
  }
  ~PythonWakeManager() {
    pending_wakes().fetch_sub(static_cast<int64_t>(queue_.size()), std::memory_order_release);
    if (fd_ >= 0) ::close(fd_);
  }
  PythonWakeManager(const PythonWakeManager&) = delete;

  // Register with the loop (must run on the loop's thread, GIL held). Idempotent per loop.
  void attach(py::object loop) {
    if (!loop_.is_none() && loop_.is(loop)) return;
    detach();
    loop_ = loop;
    loop_.attr("add_reader")(fd_, py::cpp_function([this] { process_queue(); }));
  }
  void detach() {
    if (loop_.is_none()) return;
    try {
      if (!loop_.attr("is_closed")().cast<bool>()) loop_.attr("remove_reader")(fd_);
    } catch (py::error_already_set& e) {
      e.discard_as_unraisable("PythonWakeManager.detach");
    }
    loop_ = py::none();
  }
  py::object loop() const { return loop_; }
  bool attached() const { return !loop_.is_none(); }

  // Any thread, no GIL needed.
  void enqueue(std::function<void()> fn) {
    {
      std::lock_guard lk(mu_);
      queue_.push_back(std::move(fn));
    }
    pending_wakes().fetch_add(1, std::memory_order_release);
    uint64_t one = 1;
    (void)!::write(fd_, &one, sizeof(one));
  }

  // Loop thread, GIL held.
  void process_queue() {
    uint64_t n;
    (void)!::read(fd_, &n, sizeof(n));
    // Closures that arrive while a batch runs (the reply to a request that one of them sent, for
    // instance) run in this call too, instead of one trip through the event loop later. Bounded, so
    // that a steady stream of them cannot keep the loop's other work waiting.
    for (int round = 0; round < 4; ++round) {
      std::deque<std::function<void()>> batch;
      {
        std::lock_guard lk(mu_);
        batch.swap(queue_);
      }
      if (batch.empty()) return;
      pending_wakes().fetch_sub(static_cast<int64_t>(batch.size()), std::memory_order_release);
      for (auto& fn : batch) {
        try {
          fn();
        } catch (py::error_already_set& e) {
          e.discard_as_unraisable("axon callback");
        } catch (const std::exception& e) {
          py::print("axon: callback failed:", e.what());
        }
      }
    }
  }

 private:
  int fd_ = -1;
  std::mutex mu_;
  std::deque<std::function<void()>> queue_;
  py::object loop_ = py::none();
};

}  // namespace eux::python
