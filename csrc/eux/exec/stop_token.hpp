// Stop tokens for the sender/receiver core: an in-place stop source whose
// callbacks are intrusive nodes (no allocation), and the never-stopping token.
// Same contract as the inplace_stop_source the reference takes from libunifex
// (used by every operation in ucx_context/ucx_am_context/ucx_am_context.hpp).
#pragma once

#include <atomic>
#include <mutex>
#include <thread>
#include <type_traits>
#include <utility>

namespace eux::exec {

class inplace_stop_source;
class inplace_stop_token;
template <class F>
class inplace_stop_callback;

namespace detail {
struct stop_callback_base {
  void (*invoke)(stop_callback_base*) noexcept = nullptr;
  stop_callback_base* next = nullptr;
  stop_callback_base** prev_next = nullptr;  // address of the pointer that points at us
  bool* removed_during_invoke = nullptr;
  std::atomic<bool> finished{false};
  inplace_stop_source* source = nullptr;
};
}  // namespace detail

class inplace_stop_source {
 public:
  inplace_stop_source() = default;
  inplace_stop_source(const inplace_stop_source&) = delete;
  inplace_stop_source& operator=(const inplace_stop_source&) = delete;
  ~inplace_stop_source() = default;

  inplace_stop_token get_token() const noexcept;
  bool stop_requested() const noexcept { return stopped_.load(std::memory_order_acquire); }

  bool request_stop() noexcept {
    std::unique_lock lk(mu_);
    if (stopped_.load(std::memory_order_relaxed)) return false;
    stopped_.store(true, std::memory_order_release);
    notifier_ = std::this_thread::get_id();
    while (head_) {
      detail::stop_callback_base* cb = head_;
      head_ = cb->next;
      if (head_) head_->prev_next = &head_;
      cb->prev_next = nullptr;
      bool removed = false;
      cb->removed_during_invoke = &removed;
      lk.unlock();
      cb->invoke(cb);
      lk.lock();
      if (!removed) {
        cb->removed_during_invoke = nullptr;
        cb->finished.store(true, std::memory_order_release);
      }
    }
    return true;
  }

 private:
  template <class F>
  friend class inplace_stop_callback;

  // returns false when stop was already requested (caller then runs the callback inline)
  bool try_add(detail::stop_callback_base* cb) noexcept {
    std::lock_guard lk(mu_);
    if (stopped_.load(std::memory_order_relaxed)) return false;
    cb->next = head_;
    cb->prev_next = &head_;
    if (head_) head_->prev_next = &cb->next;
    head_ = cb;
    return true;
  }

  void remove(detail::stop_callback_base* cb) noexcept {
    std::unique_lock lk(mu_);
    if (cb->prev_next) {  // still registered
      *cb->prev_next = cb->next;
      if (cb->next) cb->next->prev_next = cb->prev_next;
      cb->prev_next = nullptr;
      return;
    }
    // already taken by request_stop(): running now, or finished
    if (notifier_ == std::this_thread::get_id()) {
      if (cb->removed_during_invoke) *cb->removed_during_invoke = true;
      return;
    }
    lk.unlock();
    while (!cb->finished.load(std::memory_order_acquire)) std::this_thread::yield();
  }

  mutable std::mutex mu_;
  std::atomic<bool> stopped_{false};
  detail::stop_callback_base* head_ = nullptr;
  std::thread::id notifier_{};
};

class inplace_stop_token {
 public:
  template <class F>
  using callback_type = inplace_stop_callback<F>;
  inplace_stop_token() noexcept = default;
  bool stop_requested() const noexcept { return src_ && src_->stop_requested(); }
  bool stop_possible() const noexcept { return src_ != nullptr; }
  friend bool operator==(const inplace_stop_token& a, const inplace_stop_token& b) noexcept { return a.src_ == b.src_; }

 private:
  friend class inplace_stop_source;
  template <class F>
  friend class inplace_stop_callback;
  explicit inplace_stop_token(const inplace_stop_source* s) noexcept : src_(const_cast<inplace_stop_source*>(s)) {}
  inplace_stop_source* src_ = nullptr;
};

inline inplace_stop_token inplace_stop_source::get_token() const noexcept { return inplace_stop_token(this); }

template <class F>
class inplace_stop_callback final : private detail::stop_callback_base {
 public:
  template <class T>
  explicit inplace_stop_callback(inplace_stop_token tok, T&& fn) : fn_(std::forward<T>(fn)) {
    this->invoke = [](detail::stop_callback_base* b) noexcept { static_cast<inplace_stop_callback*>(b)->fn_(); };
    this->source = tok.src_;
    if (this->source && !this->source->try_add(this)) {
      this->source = nullptr;
      fn_();
    }
  }
  inplace_stop_callback(const inplace_stop_callback&) = delete;
  ~inplace_stop_callback() {
    if (this->source) this->source->remove(this);
  }

 private:
  F fn_;
};
template <class F>
inplace_stop_callback(inplace_stop_token, F) -> inplace_stop_callback<F>;

struct unstoppable_token {
  template <class F>
  struct callback_type {
    template <class T>
    callback_type(unstoppable_token, T&&) noexcept {}
  };
  static constexpr bool stop_requested() noexcept { return false; }
  static constexpr bool stop_possible() noexcept { return false; }
};

}  // namespace eux::exec
