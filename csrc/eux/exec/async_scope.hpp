// async_scope (spawn_detached / spawn_future / join / cleanup), any_sender_of<T>
// and task<T>: the type-erasing and lifetime-managing parts of the executor.
// The reference uses unifex::v2::async_scope for the server loop
// (axon/src/axon_worker.cpp:1293-1359), any_sender_of for dispatcher results
// (rpc_core/async_rpc_dispatcher.hpp:146-768) and unifex::task in its tests.
#pragma once

#include <coroutine>
#include <future>

#include "eux/exec/exec.hpp"

namespace eux::exec {

// ---------------------------------------------------------------------------
// any_sender_of<V>: heap-allocated, type-erased sender. Errors are delivered as
// std::exception_ptr; the stop token is an inplace_stop_token.
// ---------------------------------------------------------------------------
namespace detail {
// Adapts any stop token to an inplace_stop_token.
template <class Tok>
struct stop_token_adapter {
  inplace_stop_source src;
  std::optional<typename Tok::template callback_type<request_stop_fn>> cb;
  inplace_stop_token subscribe(Tok tok) {
    cb.emplace(tok, request_stop_fn{&src});
    return src.get_token();
  }
  void unsubscribe() noexcept { cb.reset(); }
};
template <>
struct stop_token_adapter<inplace_stop_token> {
  inplace_stop_token subscribe(inplace_stop_token tok) noexcept { return tok; }
  void unsubscribe() noexcept {}
};
template <>
struct stop_token_adapter<unstoppable_token> {
  inplace_stop_token subscribe(unstoppable_token) noexcept { return {}; }
  void unsubscribe() noexcept {}
};
}  // namespace detail

template <class V>
class any_sender_of {
 public:
  using value_type = V;

  struct receiver_base {
    virtual void value(non_void_t<V>&&) noexcept = 0;
    virtual void error(std::exception_ptr) noexcept = 0;
    virtual void done() noexcept = 0;
    inplace_stop_token token;
  };
  struct erased_receiver {
    receiver_base* b;
    template <class... A>
    void set_value(A&&... a) noexcept {
      if constexpr (sizeof...(A) == 0) b->value(unit{});
      else b->value(non_void_t<V>(std::forward<A>(a)...));
    }
    template <class E>
    void set_error(E&& e) noexcept {
      b->error(to_exception_ptr(std::forward<E>(e)));
    }
    void set_done() noexcept { b->done(); }
    inplace_stop_token get_stop_token() const noexcept { return b->token; }
  };
  struct op_base {
    virtual ~op_base() = default;
    virtual void start() noexcept = 0;
  };

  struct impl_base {
    virtual ~impl_base() = default;
    virtual std::unique_ptr<op_base> connect(erased_receiver r) = 0;
  };
  template <class S>
  struct model final : impl_base {
    S s;
    explicit model(S&& s_) : s(std::move(s_)) {}
    explicit model(const S& s_) : s(s_) {}
    struct op_model final : op_base {
      connect_result_t<S, erased_receiver> o;
      op_model(S&& s, erased_receiver r) : o(exec::connect(std::move(s), r)) {}
      void start() noexcept override { exec::start(o); }
    };
    std::unique_ptr<op_base> connect(erased_receiver r) override { return std::make_unique<op_model>(std::move(s), r); }
  };

  any_sender_of() = default;
  template <sender S>
    requires(!std::is_same_v<std::decay_t<S>, any_sender_of>)
  any_sender_of(S&& s) : impl_(std::make_unique<model<std::decay_t<S>>>(std::forward<S>(s))) {}
  any_sender_of(any_sender_of&&) noexcept = default;
  any_sender_of& operator=(any_sender_of&&) noexcept = default;
  explicit operator bool() const noexcept { return impl_ != nullptr; }

  template <class R>
  struct op final : receiver_base {
    R r;
    detail::stop_token_adapter<stop_token_of_t<R>> adapter;
    std::unique_ptr<op_base> inner;
    op(std::unique_ptr<typename any_sender_of::impl_base> impl, R&& r_) : r(std::move(r_)) {
      inner = impl->connect(erased_receiver{this});
    }
    op(op&&) = delete;
    void start() noexcept {
      this->token = adapter.subscribe(exec::get_stop_token(r));
      inner->start();
    }
    void value(non_void_t<V>&& v) noexcept override {
      adapter.unsubscribe();
      deliver<V>(r, std::move(v));
    }
    void error(std::exception_ptr e) noexcept override {
      adapter.unsubscribe();
      r.set_error(std::move(e));
    }
    void done() noexcept override {
      adapter.unsubscribe();
      r.set_done();
    }
  };
  template <class R>
  auto connect(R&& r) && {
    return op<std::decay_t<R>>(std::move(impl_), std::decay_t<R>(std::forward<R>(r)));
  }

 private:
  std::unique_ptr<impl_base> impl_;
};

// ---------------------------------------------------------------------------
// async_scope
// ---------------------------------------------------------------------------
class async_scope {
 public:
  async_scope() = default;
  async_scope(const async_scope&) = delete;
  ~async_scope() { assert(outstanding_.load() == 0 && "async_scope destroyed with work in flight"); }

  inplace_stop_token get_stop_token() const noexcept { return stop_.get_token(); }
  void request_stop() noexcept { stop_.request_stop(); }
  std::size_t outstanding() const noexcept { return outstanding_.load(std::memory_order_acquire); }

  // Run the sender to completion in the background; its result is discarded.
  template <sender S>
  void spawn_detached(S&& s);

  // Start now, observe later: the returned sender completes with the spawned result.
  template <sender S>
  auto spawn_future(S&& s) {
    using Sd = std::decay_t<S>;
    using V = value_t<Sd>;
    struct shared {
      std::mutex mu;
      int result = -1;  // -1 pending, 0 value, 1 error, 2 done
      std::optional<non_void_t<V>> val;
      std::exception_ptr err;
      std::function<void()> waiter;
    };
    auto st = std::make_shared<shared>();
    auto finish = [st](int code) {
      std::function<void()> w;
      {
        std::lock_guard lk(st->mu);
        st->result = code;
        w = std::move(st->waiter);
      }
      if (w) w();
    };
    spawn_detached(upon_done(upon_error(then(std::forward<S>(s),
                                             [st, finish](auto&&... v) {
                                               st->val.emplace(std::forward<decltype(v)>(v)...);
                                               finish(0);
                                             }),
                                        [st, finish](std::exception_ptr e) {
                                          st->err = std::move(e);
                                          finish(1);
                                        }),
                             [finish] { finish(2); }));
    return create<V>([st](auto handle) {
      auto complete = [st, handle]() mutable {
        if (st->result == 0) deliver<V>(handle, std::move(*st->val));
        else if (st->result == 1) handle.set_error(st->err);
        else handle.set_done();
      };
      std::unique_lock lk(st->mu);
      if (st->result >= 0) {
        lk.unlock();
        complete();
      } else {
        st->waiter = complete;
      }
    });
  }

  // Completes with a value when nothing spawned is still running, and with done when the receiver asks it to
  // stop first (`stop_when(scope.join(), deadline)` gives the stragglers a deadline): the scope then simply has
  // no waiter any more, and may be joined again later.
  struct join_sender {
    using value_type = void;
    async_scope* scope;
    template <class R>
    struct op {
      // Who completes the operation: the scope's last work item or the stop request, whichever turns `finished`
      // first. The state is shared because the loser may run after the winner's completion has destroyed the
      // operation, and must find that out without touching it. A stop request that arrives while start() is
      // still setting up is only noted; start() acts on it when it is done.
      struct state {
        std::atomic<bool> finished{false};
        std::atomic<bool> starting{true};
        std::atomic<bool> stop_seen{false};
      };
      struct stop_fn {
        op* o;
        void operator()() const noexcept {
          auto s = o->st;  // the callback's registration keeps the operation alive while this runs
          if (s->starting.load(std::memory_order_acquire)) {
            s->stop_seen.store(true, std::memory_order_release);
            if (s->starting.load(std::memory_order_acquire)) return;  // start() will see the note
          }
          cancel(o, s);
        }
      };
      using stop_cb_t = typename stop_token_of_t<R>::template callback_type<stop_fn>;
      async_scope* scope;
      R r;
      std::shared_ptr<state> st;
      std::optional<stop_cb_t> cb;

      op(async_scope* s, R&& r_) : scope(s), r(std::move(r_)) {}
      op(op&&) = delete;

      void start() noexcept {
        auto s = st = std::make_shared<state>();
        cb.emplace(::eux::exec::get_stop_token(r), stop_fn{this});
        {
          std::unique_lock lk(scope->mu_);
          if (scope->outstanding_.load(std::memory_order_acquire) == 0) {
            lk.unlock();
            s->finished.store(true, std::memory_order_release);
            cb.reset();
            r.set_value();
            return;
          }
          scope->waiter_ = [this, s] {
            if (s->finished.exchange(true)) return;  // the stop request completed it: `this` may be gone
            cb.reset();                               // waits for a stop callback that is running right now
            r.set_value();
          };
        }
        // from here on the waiter may complete (and destroy) the operation at any moment: only `s` is touched
        s->starting.store(false, std::memory_order_release);
        if (s->stop_seen.load(std::memory_order_acquire)) cancel(this, s);
      }
      static void cancel(op* o, const std::shared_ptr<state>& s) noexcept {
        if (s->finished.exchange(true)) return;
        {
          std::lock_guard lk(o->scope->mu_);
          o->scope->waiter_ = nullptr;
        }
        o->r.set_done();
      }
    };
    template <class R>
    auto connect(R&& r) const {
      return op<std::decay_t<R>>(scope, std::decay_t<R>(std::forward<R>(r)));
    }
  };
  // completes when nothing spawned is still running
  join_sender join() noexcept { return {this}; }
  join_sender complete() noexcept { return {this}; }
  // request stop, then join
  join_sender cleanup() noexcept {
    request_stop();
    return {this};
  }

 private:
  // The count drops under the mutex that join() checks it under: a joiner that sees zero may
  // destroy the scope at once, so nothing here may touch the scope after the count is zero and
  // the lock is released (the waiter is called from a local copy).
  void done_one() noexcept {
    std::function<void()> w;
    {
      std::lock_guard lk(mu_);
      if (outstanding_.fetch_sub(1, std::memory_order_acq_rel) != 1) return;
      w = std::move(waiter_);
      waiter_ = nullptr;
    }
    if (w) w();
  }
  std::atomic<std::size_t> outstanding_{0};
  inplace_stop_source stop_;
  std::mutex mu_;
  std::function<void()> waiter_;
};

namespace detail {
template <class Sd>
struct detached_holder;
template <class Sd>
struct detached_rcv {
  detached_holder<Sd>* h;
  template <class... A>
  void set_value(A&&...) noexcept {
    finish();
  }
  template <class E>
  void set_error(E&&) noexcept {
    finish();
  }
  void set_done() noexcept { finish(); }
  inplace_stop_token get_stop_token() const noexcept;
  void finish() noexcept;
};
template <class Sd>
struct detached_holder {
  async_scope* scope;
  void (*finished)(async_scope*) noexcept;
  connect_result_t<Sd, detached_rcv<Sd>> op;
  detached_holder(async_scope* sc, void (*fin)(async_scope*) noexcept, Sd&& s)
      : scope(sc), finished(fin), op(exec::connect(std::move(s), detached_rcv<Sd>{this})) {}
};
template <class Sd>
inplace_stop_token detached_rcv<Sd>::get_stop_token() const noexcept {
  return h->scope->get_stop_token();
}
template <class Sd>
void detached_rcv<Sd>::finish() noexcept {
  async_scope* sc = h->scope;
  auto fin = h->finished;
  delete h;
  fin(sc);
}
}  // namespace detail

template <sender S>
void async_scope::spawn_detached(S&& s) {
  using Sd = std::decay_t<S>;
  outstanding_.fetch_add(1, std::memory_order_acq_rel);
  detail::detached_holder<Sd>* h;
  try {
    h = new detail::detached_holder<Sd>(this, [](async_scope* sc) noexcept { sc->done_one(); }, Sd(std::forward<S>(s)));
  } catch (...) {
    done_one();
    throw;
  }
  exec::start(h->op);
}

// ---------------------------------------------------------------------------
// task<T>: a coroutine that can co_await senders and is itself a sender.
// A done signal from an awaited sender unwinds the coroutine and completes the
// task with set_done().
// ---------------------------------------------------------------------------
template <class T>
class task;

namespace detail {
struct task_promise_base {
  struct continuation {
    void* self = nullptr;
    void (*finished)(void*) noexcept = nullptr;   // value or error stored in the promise
    void (*cancelled)(void*) noexcept = nullptr;  // unwinding after a done signal
  } cont;
  inplace_stop_token token;
  std::exception_ptr err;
  std::coroutine_handle<> self_handle;

  std::suspend_always initial_suspend() noexcept { return {}; }
  struct final_awaiter {
    bool await_ready() noexcept { return false; }
    template <class P>
    void await_suspend(std::coroutine_handle<P> h) noexcept {
      auto c = h.promise().cont;
      c.finished(c.self);
    }
    void await_resume() noexcept {}
  };
  final_awaiter final_suspend() noexcept { return {}; }
  void unhandled_exception() noexcept { err = std::current_exception(); }

  // done signal from something we awaited: destroy this frame, tell the continuation
  void unwind_done() noexcept {
    auto c = cont;
    self_handle.destroy();
    c.cancelled(c.self);
  }

  template <sender S>
  auto await_transform(S&& s);
};
}  // namespace detail

namespace detail {
template <class Sd>
struct task_awaiter {
  using V = value_t<Sd>;
  struct rcv {
    task_awaiter* a;
    template <class... A>
    void set_value(A&&... v) noexcept {
      try {
        a->val.emplace(std::forward<A>(v)...);
      } catch (...) {
        a->err = std::current_exception();
      }
      a->h.resume();
    }
    template <class E>
    void set_error(E&& e) noexcept {
      a->err = to_exception_ptr(std::forward<E>(e));
      a->h.resume();
    }
    void set_done() noexcept { a->promise->unwind_done(); }
    inplace_stop_token get_stop_token() const noexcept { return a->promise->token; }
  };
  task_promise_base* promise;
  std::optional<non_void_t<V>> val;
  std::exception_ptr err;
  std::coroutine_handle<> h;
  connect_result_t<Sd, rcv> op;
  task_awaiter(task_promise_base* p, Sd&& s) : promise(p), op(exec::connect(std::move(s), rcv{this})) {}
  task_awaiter(task_awaiter&&) = delete;
  bool await_ready() const noexcept { return false; }
  void await_suspend(std::coroutine_handle<> hh) noexcept {
    h = hh;
    exec::start(op);
  }
  V await_resume() {
    if (err) std::rethrow_exception(err);
    if constexpr (!std::is_void_v<V>) return std::move(*val);
  }
};
template <sender S>
auto task_promise_base::await_transform(S&& s) {
  using Sd = std::decay_t<S>;
  return task_awaiter<Sd>(this, Sd(std::forward<S>(s)));
}

template <class T>
struct task_promise : task_promise_base {
  std::optional<T> result;
  task<T> get_return_object() noexcept;
  template <class U>
  void return_value(U&& u) {
    result.emplace(std::forward<U>(u));
  }
};
template <>
struct task_promise<void> : task_promise_base {
  std::optional<unit> result;
  task<void> get_return_object() noexcept;
  void return_void() { result.emplace(); }
};
}  // namespace detail

template <class T>
class task {
 public:
  using value_type = T;
  using promise_type = detail::task_promise<T>;
  task(task&& o) noexcept : h_(std::exchange(o.h_, {})) {}
  task& operator=(task&& o) noexcept {
    if (h_) h_.destroy();
    h_ = std::exchange(o.h_, {});
    return *this;
  }
  ~task() {
    if (h_) h_.destroy();
  }

  template <class R>
  struct op {
    std::coroutine_handle<promise_type> h;
    R r;
    detail::stop_token_adapter<stop_token_of_t<R>> adapter;
    op(std::coroutine_handle<promise_type> hh, R&& r_) : h(hh), r(std::move(r_)) {}
    op(op&&) = delete;
    ~op() {
      if (h) h.destroy();
    }
    void start() noexcept {
      auto& p = h.promise();
      p.token = adapter.subscribe(exec::get_stop_token(r));
      p.cont.self = this;
      p.cont.finished = [](void* s) noexcept {
        auto* self = static_cast<op*>(s);
        auto& pr = self->h.promise();
        self->adapter.unsubscribe();
        if (pr.err) {
          self->r.set_error(std::move(pr.err));
        } else {
          deliver<T>(self->r, std::move(*pr.result));
        }
      };
      p.cont.cancelled = [](void* s) noexcept {
        auto* self = static_cast<op*>(s);
        self->h = {};  // the frame destroyed itself while unwinding
        self->adapter.unsubscribe();
        self->r.set_done();
      };
      h.resume();
    }
  };
  template <class R>
  auto connect(R&& r) && {
    return op<std::decay_t<R>>(std::exchange(h_, {}), std::decay_t<R>(std::forward<R>(r)));
  }

  explicit task(std::coroutine_handle<promise_type> h) noexcept : h_(h) {}

 private:
  std::coroutine_handle<promise_type> h_;
};

namespace detail {
template <class T>
task<T> task_promise<T>::get_return_object() noexcept {
  auto h = std::coroutine_handle<task_promise<T>>::from_promise(*this);
  this->self_handle = h;
  return task<T>(h);
}
inline task<void> task_promise<void>::get_return_object() noexcept {
  auto h = std::coroutine_handle<task_promise<void>>::from_promise(*this);
  this->self_handle = h;
  return task<void>(h);
}
}  // namespace detail

}  // namespace eux::exec
