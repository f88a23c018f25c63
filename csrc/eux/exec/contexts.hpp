// Execution contexts: static_thread_pool, single_thread_context and
// timed_single_thread_context (schedule / schedule_after / schedule_at / now),
// the three the reference takes from libunifex (axon/src/axon_worker.cpp:85-100
// uses a thread pool for handlers and a timed context for RPC deadlines).
#pragma once

#include <chrono>
#include <condition_variable>
#include <deque>
#include <map>
#include <mutex>
#include <thread>
#include <vector>

#include "eux/exec/exec.hpp"

namespace eux::exec {

namespace detail {
struct task_base {
  void (*execute)(task_base*) noexcept = nullptr;
  task_base* next = nullptr;
};
}  // namespace detail

class static_thread_pool {
 public:
  explicit static_thread_pool(std::size_t n = std::thread::hardware_concurrency()) {
    if (n == 0) n = 1;
    threads_.reserve(n);
    for (std::size_t i = 0; i < n; ++i) threads_.emplace_back([this] { run(); });
  }
  ~static_thread_pool() {
    {
      std::lock_guard lk(mu_);
      stop_ = true;
      stop_hint_.store(true, std::memory_order_relaxed);
    }
    cv_.notify_all();
    for (auto& t : threads_) t.join();
  }
  static_thread_pool(const static_thread_pool&) = delete;

  class scheduler {
   public:
    struct schedule_sender {
      using value_type = void;
      static_thread_pool* pool;
      template <class R>
      struct op : detail::task_base {
        static_thread_pool* pool;
        R r;
        op(static_thread_pool* p, R&& r_) : pool(p), r(std::move(r_)) {
          this->execute = [](detail::task_base* t) noexcept {
            auto* self = static_cast<op*>(t);
            if (exec::get_stop_token(self->r).stop_requested()) self->r.set_done();
            else self->r.set_value();
          };
        }
        op(op&&) = delete;
        void start() noexcept { pool->enqueue(this); }
      };
      template <class R>
      auto connect(R&& r) const {
        return op<std::decay_t<R>>(pool, std::decay_t<R>(std::forward<R>(r)));
      }
    };
    schedule_sender schedule() const noexcept { return {pool_}; }
    friend bool operator==(scheduler a, scheduler b) noexcept { return a.pool_ == b.pool_; }

   private:
    friend class static_thread_pool;
    explicit scheduler(static_thread_pool* p) : pool_(p) {}
    static_thread_pool* pool_;
  };
  scheduler get_scheduler() noexcept { return scheduler(this); }
  std::size_t size() const noexcept { return threads_.size(); }

 private:
  // Submitting never takes the workers' lock: a task is pushed onto a lock-free list, which a worker
  // moves (reversed, so oldest first) into the queue the workers share under their mutex. A futex wake
  // per task would cost the submitting thread a system call and the task a scheduler latency, so one
  // idle worker keeps polling the task count for a short while before it sleeps, and a
  // submitter wakes a sleeper only when nobody polls. A worker that takes a task while more are
  // waiting wakes the next sleeper itself.
  static constexpr int kMaxSpinners = 1;
  static constexpr std::chrono::microseconds kSpinFor{100};
  void enqueue(detail::task_base* t) noexcept {
    detail::task_base* old = incoming_.load(std::memory_order_relaxed);
    do {
      t->next = old;
    } while (!incoming_.compare_exchange_weak(old, t, std::memory_order_seq_cst, std::memory_order_relaxed));
    queued_.fetch_add(1, std::memory_order_seq_cst);
    if (sleepers_.load(std::memory_order_seq_cst) > 0 && spinners_.load(std::memory_order_seq_cst) == 0) {
      { std::lock_guard lk(mu_); }  // a worker between its last check and its wait holds the mutex
      cv_.notify_one();
    }
  }
  // with mu_ held: move what was submitted into the shared queue
  void take_incoming() noexcept {
    detail::task_base* list = incoming_.exchange(nullptr, std::memory_order_seq_cst);
    detail::task_base* rev = nullptr;
    while (list) {
      detail::task_base* n = list->next;
      list->next = rev;
      rev = list;
      list = n;
    }
    if (!rev) return;
    if (tail_) tail_->next = rev;
    else head_ = rev;
    while (rev->next) rev = rev->next;
    tail_ = rev;
  }
  void run() {
    std::unique_lock lk(mu_);
    for (;;) {
      if (!head_) take_incoming();
      if (!head_) {
        if (stop_) return;
        if (spinners_.load(std::memory_order_relaxed) < kMaxSpinners) {
          spinners_.fetch_add(1, std::memory_order_seq_cst);
          lk.unlock();
          const auto until = std::chrono::steady_clock::now() + kSpinFor;
          while (queued_.load(std::memory_order_acquire) == 0 && !stop_hint_.load(std::memory_order_relaxed) &&
                 std::chrono::steady_clock::now() < until) {
#if defined(__x86_64__) || defined(__i386__)
            __builtin_ia32_pause();
#endif
          }
          lk.lock();
          spinners_.fetch_sub(1, std::memory_order_seq_cst);
          if (queued_.load(std::memory_order_seq_cst) > 0 || stop_) continue;
        }
        sleepers_.fetch_add(1, std::memory_order_seq_cst);
        cv_.wait(lk, [&] { return stop_ || queued_.load(std::memory_order_seq_cst) > 0; });
        sleepers_.fetch_sub(1, std::memory_order_seq_cst);
        continue;
      }
      detail::task_base* t = head_;
      head_ = t->next;
      if (!head_) tail_ = nullptr;
      const int left = queued_.fetch_sub(1, std::memory_order_seq_cst) - 1;
      const bool wake_next = left > 0 && sleepers_.load(std::memory_order_relaxed) > 0 && spinners_.load(std::memory_order_relaxed) == 0;
      lk.unlock();
      if (wake_next) cv_.notify_one();
      t->execute(t);
      lk.lock();
    }
  }
  std::mutex mu_;  // the workers' side: head_/tail_, sleeping and waking
  std::condition_variable cv_;
  std::atomic<detail::task_base*> incoming_{nullptr};
  detail::task_base* head_ = nullptr;
  detail::task_base* tail_ = nullptr;
  std::atomic<int> queued_{0};  // submitted and not yet taken by a worker
  std::atomic<bool> stop_hint_{false};
  std::atomic<int> spinners_{0};
  std::atomic<int> sleepers_{0};
  bool stop_ = false;
  std::vector<std::thread> threads_;
};

// One thread with a time-ordered queue. Items can be cancelled through the
// receiver's stop token; a cancelled item completes with set_done().
class timed_single_thread_context {
 public:
  using clock_t = std::chrono::steady_clock;
  using time_point = clock_t::time_point;

  timed_single_thread_context() : thread_([this] { run(); }) {}
  ~timed_single_thread_context() {
    {
      std::lock_guard lk(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    thread_.join();
  }
  timed_single_thread_context(const timed_single_thread_context&) = delete;

  struct item_base {
    void (*fire)(item_base*, bool cancelled) noexcept = nullptr;
    time_point due;
    bool queued = false;
  };

  class scheduler {
   public:
    struct schedule_at_sender {
      using value_type = void;
      timed_single_thread_context* ctx;
      time_point due;
      bool relative = false;
      clock_t::duration delay{};
      template <class R>
      struct op : item_base {
        struct cancel_fn {
          op* o;
          void operator()() const noexcept { o->ctx->cancel(o); }
        };
        using cb_t = typename stop_token_of_t<R>::template callback_type<cancel_fn>;
        timed_single_thread_context* ctx;
        R r;
        bool relative;
        clock_t::duration delay;
        std::optional<cb_t> cb;
        op(timed_single_thread_context* c, time_point d, bool rel, clock_t::duration dl, R&& r_)
            : ctx(c), r(std::move(r_)), relative(rel), delay(dl) {
          this->due = d;
          this->fire = [](item_base* b, bool cancelled) noexcept {
            auto* self = static_cast<op*>(b);
            self->cb.reset();
            if (cancelled) self->r.set_done();
            else self->r.set_value();
          };
        }
        op(op&&) = delete;
        void start() noexcept {
          if (relative) this->due = clock_t::now() + delay;
          // The callback exists before the item is queued (the context thread may fire
          // it at once); a stop request that came first is seen under the queue lock.
          cb.emplace(exec::get_stop_token(r), cancel_fn{this});
          auto tok = exec::get_stop_token(r);
          if (!ctx->enqueue(this, [&] { return tok.stop_requested(); })) this->fire(this, true);
        }
      };
      template <class R>
      auto connect(R&& r) const {
        return op<std::decay_t<R>>(ctx, due, relative, delay, std::decay_t<R>(std::forward<R>(r)));
      }
    };
    schedule_at_sender schedule() const noexcept { return {ctx_, clock_t::now(), false, {}}; }
    schedule_at_sender schedule_at(time_point tp) const noexcept { return {ctx_, tp, false, {}}; }
    template <class Rep, class Period>
    schedule_at_sender schedule_after(std::chrono::duration<Rep, Period> d) const noexcept {
      return {ctx_, {}, true, std::chrono::duration_cast<clock_t::duration>(d)};
    }
    time_point now() const noexcept { return clock_t::now(); }
    friend bool operator==(scheduler a, scheduler b) noexcept { return a.ctx_ == b.ctx_; }

   private:
    friend class timed_single_thread_context;
    explicit scheduler(timed_single_thread_context* c) : ctx_(c) {}
    timed_single_thread_context* ctx_;
  };
  scheduler get_scheduler() noexcept { return scheduler(this); }
  std::thread::id get_thread_id() const noexcept { return thread_.get_id(); }

 private:
  template <class StopCheck>
  bool enqueue(item_base* it, StopCheck stopped) noexcept {
    {
      std::lock_guard lk(mu_);
      if (stopped()) return false;
      it->queued = true;
      queue_.emplace(it->due, it);
    }
    cv_.notify_all();
    return true;
  }
  // Runs on the thread that requested stop. The item is either still queued
  // (we take it and complete it with done) or being fired by the context thread.
  void cancel(item_base* it) noexcept {
    {
      std::lock_guard lk(mu_);
      if (!it->queued) return;
      auto range = queue_.equal_range(it->due);
      for (auto i = range.first; i != range.second; ++i) {
        if (i->second == it) {
          queue_.erase(i);
          break;
        }
      }
      it->queued = false;
      // hand the completion to the context thread: destroying a stop callback from
      // inside its own invocation is fine, but completing inline would re-enter it
      cancelled_.push_back(it);
    }
    cv_.notify_all();
  }
  void run() {
    std::unique_lock lk(mu_);
    for (;;) {
      if (!cancelled_.empty()) {
        item_base* it = cancelled_.front();
        cancelled_.pop_front();
        lk.unlock();
        it->fire(it, true);
        lk.lock();
        continue;
      }
      if (stop_ && queue_.empty()) return;
      if (queue_.empty()) {
        cv_.wait(lk);
        continue;
      }
      auto first = queue_.begin();
      auto nowt = clock_t::now();
      if (first->first <= nowt || stop_) {
        item_base* it = first->second;
        queue_.erase(first);
        it->queued = false;
        bool cancelled = stop_ && it->due > nowt;
        lk.unlock();
        it->fire(it, cancelled);
        lk.lock();
      } else {
        // a copy: the wait re-reads its deadline after the lock is retaken, and the node that
        // holds `first->first` may have been erased by cancel() in the meantime
        const time_point due = first->first;
        cv_.wait_until(lk, due);
      }
    }
  }
  std::mutex mu_;
  std::condition_variable cv_;
  std::multimap<time_point, item_base*> queue_;
  std::deque<item_base*> cancelled_;
  bool stop_ = false;
  std::thread thread_;
};

using single_thread_context = timed_single_thread_context;

}  // namespace eux::exec
