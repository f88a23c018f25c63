// Fixed-capacity table indexed by `key & (N-1)` with per-slot atomic state:
// emplace succeeds only when the slot is free, find/erase check the full key.
// Used for in-flight RPC bookkeeping: a request id maps to one slot, and two
// live requests whose ids collide modulo N cannot coexist (the second is told
// "resource exhausted") (reference: axon/include/axon/utils/ring_buffer.hpp:44-405).
#pragma once

#include <atomic>
#include <cstddef>
#include <cstdint>
#include <memory>
#include <optional>
#include <utility>

namespace eux::axon::utils {

template <class T, size_t N>
class RingBuffer {
  static_assert(N >= 2 && (N & (N - 1)) == 0, "capacity must be a power of two");
  enum : uint32_t { kEmpty = 0, kBusy = 1, kFull = 2 };
  struct Slot {
    std::atomic<uint32_t> state{kEmpty};
    uint64_t key = 0;
    alignas(T) unsigned char storage[sizeof(T)];
    T* ptr() { return std::launder(reinterpret_cast<T*>(storage)); }
  };

 public:
  static constexpr size_t capacity() { return N; }
  RingBuffer() : slots_(new Slot[N]) {}
  ~RingBuffer() { clear(); }
  RingBuffer(const RingBuffer&) = delete;

  // Construct a value under `key`; false when the slot is occupied.
  template <class... A>
  bool emplace(uint64_t key, A&&... a) {
    Slot& s = slots_[key & (N - 1)];
    uint32_t expected = kEmpty;
    if (!s.state.compare_exchange_strong(expected, kBusy, std::memory_order_acquire)) return false;
    try {
      ::new (static_cast<void*>(s.storage)) T(std::forward<A>(a)...);
    } catch (...) {
      s.state.store(kEmpty, std::memory_order_release);
      throw;
    }
    s.key = key;
    s.state.store(kFull, std::memory_order_release);
    size_.fetch_add(1, std::memory_order_relaxed);
    return true;
  }
  // Remove and return the value stored under exactly this key.
  std::optional<T> take(uint64_t key) {
    Slot& s = slots_[key & (N - 1)];
    uint32_t expected = kFull;
    if (!s.state.compare_exchange_strong(expected, kBusy, std::memory_order_acquire)) return std::nullopt;
    if (s.key != key) {
      s.state.store(kFull, std::memory_order_release);
      return std::nullopt;
    }
    std::optional<T> out(std::move(*s.ptr()));
    s.ptr()->~T();
    s.state.store(kEmpty, std::memory_order_release);
    size_.fetch_sub(1, std::memory_order_relaxed);
    return out;
  }
  bool erase(uint64_t key) { return take(key).has_value(); }
  // Take the value only if `pred(value)` holds (e.g. the session id matches).
  template <class Pred>
  std::optional<T> take_if(uint64_t key, Pred&& pred) {
    Slot& s = slots_[key & (N - 1)];
    uint32_t expected = kFull;
    if (!s.state.compare_exchange_strong(expected, kBusy, std::memory_order_acquire)) return std::nullopt;
    if (s.key != key || !pred(*s.ptr())) {
      s.state.store(kFull, std::memory_order_release);
      return std::nullopt;
    }
    std::optional<T> out(std::move(*s.ptr()));
    s.ptr()->~T();
    s.state.store(kEmpty, std::memory_order_release);
    size_.fetch_sub(1, std::memory_order_relaxed);
    return out;
  }
  bool contains(uint64_t key) const {
    const Slot& s = slots_[key & (N - 1)];
    return s.state.load(std::memory_order_acquire) == kFull && s.key == key;
  }
  // Visit (and remove) everything; used to fail all pending calls at shutdown.
  template <class F>
  size_t drain(F&& f) {
    size_t n = 0;
    for (size_t i = 0; i < N; ++i) {
      Slot& s = slots_[i];
      uint32_t expected = kFull;
      if (!s.state.compare_exchange_strong(expected, kBusy, std::memory_order_acquire)) continue;
      T v(std::move(*s.ptr()));
      s.ptr()->~T();
      uint64_t key = s.key;
      s.state.store(kEmpty, std::memory_order_release);
      size_.fetch_sub(1, std::memory_order_relaxed);
      f(key, std::move(v));
      ++n;
    }
    return n;
  }
  void clear() {
    drain([](uint64_t, T&&) {});
  }
  size_t size() const { return size_.load(std::memory_order_relaxed); }
  bool empty() const { return size() == 0; }

 private:
  std::unique_ptr<Slot[]> slots_;
  std::atomic<size_t> size_{0};
};

}  // namespace eux::axon::utils
