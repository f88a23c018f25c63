// Senders of the active-message context: scheduling, timers, connect, accept,
// send, receive (whole message / header first / payload by key) and the
// connection-error handler (reference: ucx_am_context.hpp:1075-4156).
//
// Every operation runs on the context's thread: start() hops there through the
// remote queue when called elsewhere. Cancellation comes through the receiver's
// stop token: the stop callback (any thread) queues a small "cancel node"; the
// node runs on the context's thread, where it can see whether the operation
// has finished, is waiting in a queue, or can be withdrawn. An operation whose
// result is ready while its cancel node is still in flight leaves the delivery
// to the node, so the operation state is never touched after it completes.
//
// Included at the end of ucx_am_context.hpp.
#pragma once

#include <sys/socket.h>

namespace eux::ucxx {

namespace detail {

inline std::error_code status_error(int st) { return make_ucx_error(st); }

template <class Derived, class Receiver>
struct io_op_base : ucx_am_context::parked_op {
  struct cancel_node_t : ucx_am_context::operation_base {
    io_op_base* self = nullptr;
  };
  struct stop_fn {
    io_op_base* o;
    void operator()() const noexcept { o->request_cancel(); }
  };
  using stop_cb_t = typename exec::stop_token_of_t<Receiver>::template callback_type<stop_fn>;

  ucx_am_context& ctx;
  Receiver r;
  cancel_node_t cancel_node;
  std::atomic<bool> cancel_enqueued{false};
  bool cancel_node_ran = false;
  bool cancel_wanted = false;  // cancel arrived while we sat in a run queue
  bool finished = false;
  bool have_result = false;    // a transport callback stored `result_status`
  int result_status = UCS_OK;
  std::function<void()> deferred;
  std::optional<stop_cb_t> stop_cb;

  io_op_base(ucx_am_context& c, Receiver&& rcv) : ctx(c), r(std::move(rcv)) {
    this->execute = [](ucx_am_context::operation_base* b) noexcept {
      auto* self = static_cast<io_op_base*>(static_cast<ucx_am_context::parked_op*>(b));
      static_cast<ucx_am_context::parked_op*>(self)->queued = false;
      self->on_io_thread();
    };
    cancel_node.self = this;
    cancel_node.execute = [](ucx_am_context::operation_base* b) noexcept { static_cast<cancel_node_t*>(b)->self->on_cancel_node(); };
  }
  io_op_base(io_op_base&&) = delete;
  Derived& derived() { return *static_cast<Derived*>(this); }

  void start() noexcept {
    stop_cb.emplace(exec::get_stop_token(r), stop_fn{this});
    if (ctx.is_running_on_io_thread() && !cancel_enqueued.load(std::memory_order_acquire)) {
      on_io_thread();
    } else {
      this->queued = true;
      ctx.schedule_remote(this);
    }
  }
  void request_cancel() noexcept {
    if (!cancel_enqueued.exchange(true, std::memory_order_acq_rel)) ctx.schedule_remote(&cancel_node);
  }
  // queue ourselves to run again on the context's thread (from a transport callback)
  void requeue() noexcept {
    if (!this->queued) {
      this->queued = true;
      ctx.schedule_local(this);
    }
  }
  void on_transport_result(int status) noexcept {
    have_result = true;
    result_status = status;
    requeue();
  }
  void on_io_thread() noexcept {
    if (finished) return;
    if (cancel_wanted && !have_result) {
      if (derived().try_cancel()) {
        finish([this] { r.set_done(); });
        return;
      }
      cancel_wanted = false;
    }
    if (ctx.stopping() && !have_result && derived().try_cancel()) {
      finish([this] { r.set_done(); });
      return;
    }
    derived().step();
  }
  void on_cancel_node() noexcept {
    cancel_node_ran = true;
    if (finished) {
      auto d = std::move(deferred);
      deferred = nullptr;
      if (d) d();
      return;
    }
    if (this->queued) {  // execute() is about to run; let it see the request
      cancel_wanted = true;
      return;
    }
    if (!have_result && derived().try_cancel()) finish([this] { r.set_done(); });
  }
  // Deliver the final signal. Nothing of the operation is touched after `deliver` runs.
  template <class F>
  void finish(F&& deliver) noexcept {
    finished = true;
    stop_cb.reset();
    if (cancel_enqueued.load(std::memory_order_acquire) && !cancel_node_ran) {
      deferred = std::forward<F>(deliver);
      return;
    }
    deliver();
  }
  void finish_error(int status) noexcept {
    if (status == UCS_ERR_CANCELED) finish([this] { r.set_done(); });
    else finish([this, status] { r.set_error(status_error(status)); });
  }
};

// resolve the three ways of naming a connection
inline UcxConnection* resolve_conn(ucx_am_context& ctx, conn_id_t id) { return ctx.connections().get_connection(id); }

}  // namespace detail

// ============================================================================================
// scheduler: schedule / schedule_at / schedule_after / now
// ============================================================================================
class ucx_am_context::scheduler {
 public:
  struct schedule_sender {
    using value_type = void;
    ucx_am_context* ctx;
    template <class R>
    struct op : ucx_am_context::operation_base {
      ucx_am_context* ctx;
      R r;
      op(ucx_am_context* c, R&& r_) : ctx(c), r(std::move(r_)) {
        this->execute = [](ucx_am_context::operation_base* b) noexcept {
          auto* self = static_cast<op*>(b);
          if (exec::get_stop_token(self->r).stop_requested() || self->ctx->stopping()) self->r.set_done();
          else self->r.set_value();
        };
      }
      op(op&&) = delete;
      void start() noexcept {
        if (ctx->is_running_on_io_thread()) ctx->schedule_local(this);
        else ctx->schedule_remote(this);
      }
    };
    template <class R>
    auto connect(R&& r) const {
      return op<std::decay_t<R>>(ctx, std::decay_t<R>(std::forward<R>(r)));
    }
  };

  struct schedule_at_sender {
    using value_type = void;
    ucx_am_context* ctx;
    time_point due;
    bool relative;
    clock_t::duration delay;
    template <class R>
    struct op : detail::io_op_base<op<R>, R> {
      using base = detail::io_op_base<op<R>, R>;
      struct my_timer : ucx_am_context::timer_op {
        op* self = nullptr;
      } timer;
      time_point due;
      bool relative;
      clock_t::duration delay;
      bool armed_once = false;
      op(ucx_am_context* c, time_point d, bool rel, clock_t::duration dl, R&& r_)
          : base(*c, std::move(r_)), due(d), relative(rel), delay(dl) {
        if (relative) due = clock_t::now() + delay;  // measured from creation, refreshed at start
        timer.self = this;
        timer.execute = [](ucx_am_context::operation_base* b) noexcept { static_cast<my_timer*>(b)->self->fired(); };
      }
      void start() noexcept {
        if (relative) due = clock_t::now() + delay;
        base::start();
      }
      void step() noexcept {
        if (armed_once) return;
        armed_once = true;
        timer.due = due;
        this->ctx.schedule_timer(&timer);
      }
      void fired() noexcept {
        if (this->finished) return;
        if (this->ctx.stopping()) this->finish([this] { this->r.set_done(); });
        else this->finish([this] { this->r.set_value(); });
      }
      bool try_cancel() noexcept { return !armed_once || this->ctx.cancel_timer(&timer); }
    };
    template <class R>
    auto connect(R&& r) const {
      return op<std::decay_t<R>>(ctx, due, relative, delay, std::decay_t<R>(std::forward<R>(r)));
    }
  };

  // Completes (with no value) on the context's thread once `*flag >= at_least`. `flag` is host memory that
  // something outside the CPU's threads writes, typically mapped pinned memory into which a kernel
  // release-stores a sequence number after its last store: a handler launches its kernel, returns this
  // sender followed by what builds the reply, and no thread waits for the GPU. Cancellable; completes
  // with done when the context stops. The word must stay valid until the sender has completed.
  struct flag_sender {
    using value_type = void;
    ucx_am_context* ctx;
    const volatile uint64_t* flag;
    uint64_t at_least;
    template <class R>
    struct op : detail::io_op_base<op<R>, R> {
      using base = detail::io_op_base<op<R>, R>;
      struct my_flag : ucx_am_context::flag_op {
        op* self = nullptr;
      } watch;
      bool armed_once = false;
      bool reached() const noexcept { return __atomic_load_n(const_cast<const uint64_t*>(watch.flag), __ATOMIC_ACQUIRE) >= watch.at_least; }
      op(ucx_am_context* c, const volatile uint64_t* f, uint64_t v, R&& r_) : base(*c, std::move(r_)) {
        watch.self = this;
        watch.flag = f;
        watch.at_least = v;
        watch.execute = [](ucx_am_context::operation_base* b) noexcept { static_cast<my_flag*>(b)->self->fired(); };
      }
      void step() noexcept {
        if (armed_once) return;
        armed_once = true;
        if (reached()) {
          fired();
          return;
        }
        this->ctx.watch_flag(&watch);
      }
      void fired() noexcept {
        if (this->finished) return;
        if (this->ctx.stopping() && !reached()) this->finish([this] { this->r.set_done(); });
        else this->finish([this] { this->r.set_value(); });
      }
      bool try_cancel() noexcept { return !armed_once || this->ctx.unwatch_flag(&watch); }
    };
    template <class R>
    auto connect(R&& r) const {
      return op<std::decay_t<R>>(ctx, flag, at_least, std::decay_t<R>(std::forward<R>(r)));
    }
  };
  flag_sender schedule_when_flag(const volatile uint64_t* flag, uint64_t at_least) const noexcept { return {ctx_, flag, at_least}; }

  schedule_sender schedule() const noexcept { return {ctx_}; }
  schedule_at_sender schedule_at(time_point tp) const noexcept { return {ctx_, tp, false, {}}; }
  template <class Rep, class Period>
  schedule_at_sender schedule_after(std::chrono::duration<Rep, Period> d) const noexcept {
    return {ctx_, {}, true, std::chrono::duration_cast<clock_t::duration>(d)};
  }
  time_point now() const noexcept { return clock_t::now(); }
  ucx_am_context& context() const noexcept { return *ctx_; }
  friend bool operator==(const scheduler& a, const scheduler& b) noexcept { return a.ctx_ == b.ctx_; }

 private:
  friend class ucx_am_context;
  explicit scheduler(ucx_am_context* c) noexcept : ctx_(c) {}
  ucx_am_context* ctx_;
};

}  // namespace eux::ucxx

#include "eux/ucxx/ucx_am_context_io_senders.hpp"
