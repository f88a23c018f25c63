// eux::exec -- a small sender/receiver (P2300-style) core.
//
// The reference builds every asynchronous operation on libunifex senders
// (connect/start, set_value/set_error/set_done, stop tokens; e.g.
// ucx_context/ucx_am_context/ucx_am_context.hpp:1075-1509 and
// axon/include/axon/axon_worker.hpp:1052-1208). This header provides the same
// vocabulary with a deliberately small model:
//   * a sender completes with at most one value: `using value_type = T` (or void);
//   * errors are generic (`set_error(E)`), normalised to std::exception_ptr
//     where an algorithm has to store one (std::error_code travels inside
//     std::system_error and is recovered with error_code_of());
//   * cancellation completes with set_done().
// Operation states are immovable and are started with start().
#pragma once

#include <atomic>
#include <cassert>
#include <condition_variable>
#include <exception>
#include <functional>
#include <memory>
#include <mutex>
#include <optional>
#include <system_error>
#include <tuple>
#include <type_traits>
#include <utility>
#include <variant>

#include "eux/exec/stop_token.hpp"

namespace eux::exec {

struct unit {
  friend bool operator==(unit, unit) { return true; }
};
template <class T>
using non_void_t = std::conditional_t<std::is_void_v<T>, unit, T>;

template <class T>
class manual_lifetime {
 public:
  manual_lifetime() noexcept {}
  ~manual_lifetime() {}
  manual_lifetime(const manual_lifetime&) = delete;
  template <class F>
  T& construct_with(F&& f) {
    return *::new (static_cast<void*>(&buf_)) T(std::forward<F>(f)());
  }
  template <class... A>
  T& construct(A&&... a) {
    return *::new (static_cast<void*>(&buf_)) T(std::forward<A>(a)...);
  }
  void destruct() noexcept { get().~T(); }
  T& get() noexcept { return *std::launder(reinterpret_cast<T*>(&buf_)); }

 private:
  alignas(T) unsigned char buf_[sizeof(T)];
};

// ---- errors -----------------------------------------------------------------
template <class E>
std::exception_ptr to_exception_ptr(E&& e) noexcept {
  using D = std::remove_cvref_t<E>;
  if constexpr (std::is_same_v<D, std::exception_ptr>) {
    return std::forward<E>(e);
  } else if constexpr (std::is_same_v<D, std::error_code>) {
    return std::make_exception_ptr(std::system_error(e));
  } else {
    return std::make_exception_ptr(std::forward<E>(e));
  }
}
inline std::error_code error_code_of(const std::exception_ptr& ep) noexcept {
  if (!ep) return {};
  try {
    std::rethrow_exception(ep);
  } catch (const std::system_error& se) {
    return se.code();
  } catch (...) {
    return std::make_error_code(std::errc::io_error);
  }
}
inline std::string what_of(const std::exception_ptr& ep) noexcept {
  if (!ep) return {};
  try {
    std::rethrow_exception(ep);
  } catch (const std::exception& e) {
    return e.what();
  } catch (...) {
    return "unknown error";
  }
}

// ---- queries ------------------------------------------------------------------
inline constexpr struct get_stop_token_t {
  template <class R>
  auto operator()(const R& r) const noexcept {
    if constexpr (requires { r.get_stop_token(); }) {
      return r.get_stop_token();
    } else {
      return unstoppable_token{};
    }
  }
} get_stop_token{};
template <class R>
using stop_token_of_t = decltype(get_stop_token(std::declval<const R&>()));

// ---- sender basics --------------------------------------------------------------
template <class S>
concept sender = requires { typename std::remove_cvref_t<S>::value_type; };
template <class S>
using value_t = typename std::remove_cvref_t<S>::value_type;

template <class S, class R>
auto connect(S&& s, R&& r) {
  return std::forward<S>(s).connect(std::forward<R>(r));
}
template <class S, class R>
using connect_result_t = decltype(exec::connect(std::declval<S>(), std::declval<R>()));
template <class O>
void start(O& o) noexcept {
  o.start();
}

// deliver a non_void_t<V> to a receiver expecting V
template <class V, class R, class T>
void deliver(R& r, T&& v) noexcept {
  if constexpr (std::is_void_v<V>) {
    r.set_value();
  } else {
    r.set_value(std::forward<T>(v));
  }
}

// forwards everything to a receiver held elsewhere
template <class R>
struct ref_receiver {
  R* r;
  template <class... A>
  void set_value(A&&... a) noexcept {
    r->set_value(std::forward<A>(a)...);
  }
  template <class E>
  void set_error(E&& e) noexcept {
    r->set_error(std::forward<E>(e));
  }
  void set_done() noexcept { r->set_done(); }
  auto get_stop_token() const noexcept { return exec::get_stop_token(*r); }
};

// ---- pipe syntax -------------------------------------------------------------
template <class F>
struct closure {
  F f;
  template <sender S>
  friend auto operator|(S&& s, closure&& c) {
    return std::move(c.f)(std::forward<S>(s));
  }
  template <sender S>
  friend auto operator|(S&& s, const closure& c) {
    return c.f(std::forward<S>(s));
  }
};
template <class F>
closure(F) -> closure<F>;

// ---- just / just_from / just_error / just_done --------------------------------
template <class V>
struct just_sender {
  using value_type = V;
  [[no_unique_address]] non_void_t<V> v;
  template <class R>
  struct op {
    [[no_unique_address]] non_void_t<V> v;
    R r;
    void start() noexcept { deliver<V>(r, std::move(v)); }
  };
  template <class R>
  auto connect(R&& r) && {
    return op<std::decay_t<R>>{std::move(v), std::forward<R>(r)};
  }
  template <class R>
  auto connect(R&& r) const& {
    return op<std::decay_t<R>>{v, std::forward<R>(r)};
  }
};
inline auto just() { return just_sender<void>{}; }
template <class V>
auto just(V&& v) {
  return just_sender<std::decay_t<V>>{std::forward<V>(v)};
}

template <class F>
struct just_from_sender {
  using value_type = std::invoke_result_t<F&>;
  F f;
  template <class R>
  struct op {
    F f;
    R r;
    void start() noexcept {
      try {
        if constexpr (std::is_void_v<value_type>) {
          f();
          r.set_value();
        } else {
          r.set_value(f());
        }
      } catch (...) {
        r.set_error(std::current_exception());
      }
    }
  };
  template <class R>
  auto connect(R&& r) && {
    return op<std::decay_t<R>>{std::move(f), std::forward<R>(r)};
  }
  template <class R>
  auto connect(R&& r) const& {
    return op<std::decay_t<R>>{f, std::forward<R>(r)};
  }
};
template <class F>
auto just_from(F&& f) {
  return just_from_sender<std::decay_t<F>>{std::forward<F>(f)};
}

template <class E, class V = void>
struct just_error_sender {
  using value_type = V;
  E e;
  template <class R>
  struct op {
    E e;
    R r;
    void start() noexcept { r.set_error(std::move(e)); }
  };
  template <class R>
  auto connect(R&& r) && {
    return op<std::decay_t<R>>{std::move(e), std::forward<R>(r)};
  }
  template <class R>
  auto connect(R&& r) const& {
    return op<std::decay_t<R>>{e, std::forward<R>(r)};
  }
};
template <class V = void, class E>
auto just_error(E&& e) {
  return just_error_sender<std::decay_t<E>, V>{std::forward<E>(e)};
}

template <class V = void>
struct just_done_sender {
  using value_type = V;
  template <class R>
  struct op {
    R r;
    void start() noexcept { r.set_done(); }
  };
  template <class R>
  auto connect(R&& r) const {
    return op<std::decay_t<R>>{std::forward<R>(r)};
  }
};
template <class V = void>
auto just_done() {
  return just_done_sender<V>{};
}

// ---- then / upon_error / upon_done --------------------------------------------
namespace detail {
template <class F, class V>
struct invoke_with {
  using type = std::invoke_result_t<F, V>;
};
template <class F>
struct invoke_with<F, void> {
  using type = std::invoke_result_t<F>;
};
template <class F, class V>
using invoke_with_t = typename invoke_with<F, V>::type;
}  // namespace detail

template <class S, class F>
struct then_sender {
  using value_type = detail::invoke_with_t<F, value_t<S>>;
  S s;
  F f;
  template <class R>
  struct rcv {
    R r;
    F f;
    template <class... A>
    void set_value(A&&... a) noexcept {
      try {
        if constexpr (std::is_void_v<value_type>) {
          std::invoke(std::move(f), std::forward<A>(a)...);
          r.set_value();
        } else {
          r.set_value(std::invoke(std::move(f), std::forward<A>(a)...));
        }
      } catch (...) {
        r.set_error(std::current_exception());
      }
    }
    template <class E>
    void set_error(E&& e) noexcept {
      r.set_error(std::forward<E>(e));
    }
    void set_done() noexcept { r.set_done(); }
    auto get_stop_token() const noexcept { return exec::get_stop_token(r); }
  };
  template <class R>
  auto connect(R&& r) && {
    return exec::connect(std::move(s), rcv<std::decay_t<R>>{std::forward<R>(r), std::move(f)});
  }
  template <class R>
  auto connect(R&& r) const& {
    return exec::connect(s, rcv<std::decay_t<R>>{std::forward<R>(r), f});
  }
};
template <sender S, class F>
auto then(S&& s, F&& f) {
  return then_sender<std::decay_t<S>, std::decay_t<F>>{std::forward<S>(s), std::forward<F>(f)};
}
template <class F>
auto then(F&& f) {
  return closure{[f = std::forward<F>(f)](auto&& s) mutable { return exec::then(std::forward<decltype(s)>(s), std::move(f)); }};
}

// upon_error: f(std::exception_ptr) -> value_type of the source (or void)
template <class S, class F>
struct upon_error_sender {
  using value_type = value_t<S>;
  S s;
  F f;
  template <class R>
  struct rcv {
    R r;
    F f;
    template <class... A>
    void set_value(A&&... a) noexcept {
      r.set_value(std::forward<A>(a)...);
    }
    template <class E>
    void set_error(E&& e) noexcept {
      try {
        if constexpr (std::is_void_v<value_type>) {
          std::invoke(std::move(f), to_exception_ptr(std::forward<E>(e)));
          r.set_value();
        } else {
          r.set_value(std::invoke(std::move(f), to_exception_ptr(std::forward<E>(e))));
        }
      } catch (...) {
        r.set_error(std::current_exception());
      }
    }
    void set_done() noexcept { r.set_done(); }
    auto get_stop_token() const noexcept { return exec::get_stop_token(r); }
  };
  template <class R>
  auto connect(R&& r) && {
    return exec::connect(std::move(s), rcv<std::decay_t<R>>{std::forward<R>(r), std::move(f)});
  }
};
template <sender S, class F>
auto upon_error(S&& s, F&& f) {
  return upon_error_sender<std::decay_t<S>, std::decay_t<F>>{std::forward<S>(s), std::forward<F>(f)};
}
template <class F>
auto upon_error(F&& f) {
  return closure{[f = std::forward<F>(f)](auto&& s) mutable { return exec::upon_error(std::forward<decltype(s)>(s), std::move(f)); }};
}

template <class S, class F>
struct upon_done_sender {
  using value_type = value_t<S>;
  S s;
  F f;
  template <class R>
  struct rcv {
    R r;
    F f;
    template <class... A>
    void set_value(A&&... a) noexcept {
      r.set_value(std::forward<A>(a)...);
    }
    template <class E>
    void set_error(E&& e) noexcept {
      r.set_error(std::forward<E>(e));
    }
    void set_done() noexcept {
      try {
        if constexpr (std::is_void_v<value_type>) {
          std::invoke(std::move(f));
          r.set_value();
        } else {
          r.set_value(std::invoke(std::move(f)));
        }
      } catch (...) {
        r.set_error(std::current_exception());
      }
    }
    auto get_stop_token() const noexcept { return exec::get_stop_token(r); }
  };
  template <class R>
  auto connect(R&& r) && {
    return exec::connect(std::move(s), rcv<std::decay_t<R>>{std::forward<R>(r), std::move(f)});
  }
};
template <sender S, class F>
auto upon_done(S&& s, F&& f) {
  return upon_done_sender<std::decay_t<S>, std::decay_t<F>>{std::forward<S>(s), std::forward<F>(f)};
}
template <class F>
auto upon_done(F&& f) {
  return closure{[f = std::forward<F>(f)](auto&& s) mutable { return exec::upon_done(std::forward<decltype(s)>(s), std::move(f)); }};
}

// ---- let_value / let_error / let_done / defer ---------------------------------
namespace detail {
template <class F, class V>
struct let_succ {
  using type = std::invoke_result_t<F&, V&>;
};
template <class F>
struct let_succ<F, void> {
  using type = std::invoke_result_t<F&>;
};
}  // namespace detail

template <class S, class F>
struct let_value_sender {
  using in_t = value_t<S>;
  using succ_t = typename detail::let_succ<F, in_t>::type;
  using value_type = value_t<succ_t>;
  S s;
  F f;
  template <class R>
  struct op {
    struct pred_rcv {
      op* o;
      template <class... A>
      void set_value(A&&... a) noexcept {
        o->on_value(std::forward<A>(a)...);
      }
      template <class E>
      void set_error(E&& e) noexcept {
        o->r.set_error(std::forward<E>(e));
      }
      void set_done() noexcept { o->r.set_done(); }
      auto get_stop_token() const noexcept { return exec::get_stop_token(o->r); }
    };
    using succ_op_t = connect_result_t<succ_t, ref_receiver<R>>;
    R r;
    F f;
    std::optional<non_void_t<in_t>> val;
    connect_result_t<S, pred_rcv> pred;
    manual_lifetime<succ_op_t> succ;
    bool succ_live = false;
    op(S&& s_, F&& f_, R&& r_) : r(std::move(r_)), f(std::move(f_)), pred(exec::connect(std::move(s_), pred_rcv{this})) {}
    op(op&&) = delete;
    ~op() {
      if (succ_live) succ.destruct();
    }
    void start() noexcept { exec::start(pred); }
    template <class... A>
    void on_value(A&&... a) noexcept {
      try {
        val.emplace(std::forward<A>(a)...);
        succ.construct_with([&] {
          if constexpr (std::is_void_v<in_t>) {
            return exec::connect(f(), ref_receiver<R>{&r});
          } else {
            return exec::connect(f(*val), ref_receiver<R>{&r});
          }
        });
        succ_live = true;
      } catch (...) {
        r.set_error(std::current_exception());
        return;
      }
      exec::start(succ.get());
    }
  };
  template <class R>
  auto connect(R&& r) && {
    return op<std::decay_t<R>>(std::move(s), std::move(f), std::decay_t<R>(std::forward<R>(r)));
  }
  template <class R>
  auto connect(R&& r) const& {
    return op<std::decay_t<R>>(S(s), F(f), std::decay_t<R>(std::forward<R>(r)));
  }
};
template <sender S, class F>
auto let_value(S&& s, F&& f) {
  return let_value_sender<std::decay_t<S>, std::decay_t<F>>{std::forward<S>(s), std::forward<F>(f)};
}
template <class F>
auto let_value(F&& f) {
  return closure{[f = std::forward<F>(f)](auto&& s) mutable { return exec::let_value(std::forward<decltype(s)>(s), std::move(f)); }};
}

// let_error: f(std::exception_ptr) -> sender with the same value_type; let_done: f() -> sender
template <class S, class F, bool OnError>
struct let_alt_sender {
  using value_type = value_t<S>;
  using succ_t = std::conditional_t<OnError, std::invoke_result<F&, std::exception_ptr>, std::invoke_result<F&>>::type;
  S s;
  F f;
  template <class R>
  struct op {
    struct pred_rcv {
      op* o;
      template <class... A>
      void set_value(A&&... a) noexcept {
        o->r.set_value(std::forward<A>(a)...);
      }
      template <class E>
      void set_error(E&& e) noexcept {
        if constexpr (OnError) {
          o->divert(to_exception_ptr(std::forward<E>(e)));
        } else {
          o->r.set_error(std::forward<E>(e));
        }
      }
      void set_done() noexcept {
        if constexpr (OnError) {
          o->r.set_done();
        } else {
          o->divert(nullptr);
        }
      }
      auto get_stop_token() const noexcept { return exec::get_stop_token(o->r); }
    };
    using succ_op_t = connect_result_t<succ_t, ref_receiver<R>>;
    R r;
    F f;
    connect_result_t<S, pred_rcv> pred;
    manual_lifetime<succ_op_t> succ;
    bool succ_live = false;
    op(S&& s_, F&& f_, R&& r_) : r(std::move(r_)), f(std::move(f_)), pred(exec::connect(std::move(s_), pred_rcv{this})) {}
    op(op&&) = delete;
    ~op() {
      if (succ_live) succ.destruct();
    }
    void start() noexcept { exec::start(pred); }
    void divert(std::exception_ptr ep) noexcept {
      try {
        succ.construct_with([&] {
          if constexpr (OnError) {
            return exec::connect(f(std::move(ep)), ref_receiver<R>{&r});
          } else {
            return exec::connect(f(), ref_receiver<R>{&r});
          }
        });
        succ_live = true;
      } catch (...) {
        r.set_error(std::current_exception());
        return;
      }
      exec::start(succ.get());
    }
  };
  template <class R>
  auto connect(R&& r) && {
    return op<std::decay_t<R>>(std::move(s), std::move(f), std::decay_t<R>(std::forward<R>(r)));
  }
};
template <sender S, class F>
auto let_error(S&& s, F&& f) {
  return let_alt_sender<std::decay_t<S>, std::decay_t<F>, true>{std::forward<S>(s), std::forward<F>(f)};
}
template <class F>
auto let_error(F&& f) {
  return closure{[f = std::forward<F>(f)](auto&& s) mutable { return exec::let_error(std::forward<decltype(s)>(s), std::move(f)); }};
}
template <sender S, class F>
auto let_done(S&& s, F&& f) {
  return let_alt_sender<std::decay_t<S>, std::decay_t<F>, false>{std::forward<S>(s), std::forward<F>(f)};
}
template <class F>
auto let_done(F&& f) {
  return closure{[f = std::forward<F>(f)](auto&& s) mutable { return exec::let_done(std::forward<decltype(s)>(s), std::move(f)); }};
}

template <class F>
auto defer(F&& f) {
  return let_value(just(), std::forward<F>(f));
}

// let_value_with(state_factory, f): keeps a state object alive for the successor
template <class SF, class F>
auto let_value_with(SF&& sf, F&& f) {
  return let_value(just_from(std::forward<SF>(sf)), std::forward<F>(f));
}

// sequence(a, b, ...): run in order; the result is the last one's
template <sender A>
auto sequence(A&& a) {
  return std::forward<A>(a);
}
template <sender A, sender B, sender... Rest>
auto sequence(A&& a, B&& b, Rest&&... rest) {
  static_assert(std::is_void_v<value_t<A>>, "sequence() predecessors must complete with no value");
  return sequence(let_value(std::forward<A>(a), [b = std::decay_t<B>(std::forward<B>(b))]() mutable { return std::move(b); }),
                  std::forward<Rest>(rest)...);
}

// ---- with_query_value(sender, get_stop_token, token) ---------------------------
template <class S, class Tok>
struct with_stop_token_sender {
  using value_type = value_t<S>;
  S s;
  Tok tok;
  template <class R>
  struct rcv {
    R r;
    Tok tok;
    template <class... A>
    void set_value(A&&... a) noexcept {
      r.set_value(std::forward<A>(a)...);
    }
    template <class E>
    void set_error(E&& e) noexcept {
      r.set_error(std::forward<E>(e));
    }
    void set_done() noexcept { r.set_done(); }
    Tok get_stop_token() const noexcept { return tok; }
  };
  template <class R>
  auto connect(R&& r) && {
    return exec::connect(std::move(s), rcv<std::decay_t<R>>{std::forward<R>(r), tok});
  }
  template <class R>
  auto connect(R&& r) const& {
    return exec::connect(s, rcv<std::decay_t<R>>{std::forward<R>(r), tok});
  }
};
template <sender S, class Tok>
auto with_query_value(S&& s, get_stop_token_t, Tok tok) {
  return with_stop_token_sender<std::decay_t<S>, Tok>{std::forward<S>(s), tok};
}

// ---- when_all ---------------------------------------------------------------------
namespace detail {
template <class Op>
struct op_holder {
  Op op;
  template <class F>
  explicit op_holder(F&& f) : op(std::forward<F>(f)()) {}
};
struct request_stop_fn {
  inplace_stop_source* src;
  void operator()() const noexcept { src->request_stop(); }
};
}  // namespace detail

template <class... S>
struct when_all_sender {
  using value_type = std::tuple<non_void_t<value_t<S>>...>;
  std::tuple<S...> ss;

  template <class R, class Idx>
  struct op;
  template <class R, std::size_t... I>
  struct op<R, std::index_sequence<I...>> {
    template <std::size_t K>
    struct child_rcv {
      op* o;
      template <class... A>
      void set_value(A&&... a) noexcept {
        try {
          std::get<K>(o->vals).emplace(std::forward<A>(a)...);
        } catch (...) {
          o->fail(std::current_exception());
          return;
        }
        o->arrive();
      }
      template <class E>
      void set_error(E&& e) noexcept {
        o->fail(to_exception_ptr(std::forward<E>(e)));
      }
      void set_done() noexcept {
        int expected = 0;
        o->state.compare_exchange_strong(expected, 2);
        o->stop.request_stop();
        o->arrive();
      }
      inplace_stop_token get_stop_token() const noexcept { return o->stop.get_token(); }
    };
    using parent_cb = typename stop_token_of_t<R>::template callback_type<detail::request_stop_fn>;
    R r;
    std::atomic<std::size_t> remaining{sizeof...(S)};
    std::atomic<int> state{0};  // 0 values, 1 error, 2 done
    std::exception_ptr err;
    inplace_stop_source stop;
    std::optional<parent_cb> on_stop;
    std::tuple<std::optional<non_void_t<value_t<S>>>...> vals;
    std::tuple<detail::op_holder<connect_result_t<S, child_rcv<I>>>...> ops;

    op(std::tuple<S...>&& ss, R&& r_)
        : r(std::move(r_)), ops([&] { return exec::connect(std::get<I>(std::move(ss)), child_rcv<I>{this}); }...) {}
    op(op&&) = delete;
    void start() noexcept {
      on_stop.emplace(exec::get_stop_token(r), detail::request_stop_fn{&stop});
      (exec::start(std::get<I>(ops).op), ...);
    }
    void fail(std::exception_ptr ep) noexcept {
      int expected = 0;
      if (state.compare_exchange_strong(expected, 1)) err = std::move(ep);
      stop.request_stop();
      arrive();
    }
    void arrive() noexcept {
      if (remaining.fetch_sub(1, std::memory_order_acq_rel) != 1) return;
      on_stop.reset();
      switch (state.load()) {
        case 0: r.set_value(value_type{std::move(*std::get<I>(vals))...}); break;
        case 1: r.set_error(std::move(err)); break;
        default: r.set_done(); break;
      }
    }
  };
  template <class R>
  auto connect(R&& r) && {
    return op<std::decay_t<R>, std::index_sequence_for<S...>>(std::move(ss), std::decay_t<R>(std::forward<R>(r)));
  }
};
template <sender... S>
auto when_all(S&&... s) {
  return when_all_sender<std::decay_t<S>...>{std::tuple<std::decay_t<S>...>(std::forward<S>(s)...)};
}

// ---- stop_when(source, trigger) -----------------------------------------------------
// Runs both; the first to finish requests stop on the other. The result is the source's.
template <class S, class T>
struct stop_when_sender {
  using value_type = value_t<S>;
  S s;
  T t;
  template <class R>
  struct op {
    struct src_rcv {
      op* o;
      template <class... A>
      void set_value(A&&... a) noexcept {
        try {
          o->val.emplace(std::forward<A>(a)...);
          o->result = 0;
        } catch (...) {
          o->err = std::current_exception();
          o->result = 1;
        }
        o->stop.request_stop();
        o->arrive();
      }
      template <class E>
      void set_error(E&& e) noexcept {
        o->err = to_exception_ptr(std::forward<E>(e));
        o->result = 1;
        o->stop.request_stop();
        o->arrive();
      }
      void set_done() noexcept {
        o->result = 2;
        o->stop.request_stop();
        o->arrive();
      }
      inplace_stop_token get_stop_token() const noexcept { return o->stop.get_token(); }
    };
    struct trig_rcv {
      op* o;
      template <class... A>
      void set_value(A&&...) noexcept {
        o->stop.request_stop();
        o->arrive();
      }
      template <class E>
      void set_error(E&&) noexcept {
        o->stop.request_stop();
        o->arrive();
      }
      void set_done() noexcept {
        o->stop.request_stop();
        o->arrive();
      }
      inplace_stop_token get_stop_token() const noexcept { return o->stop.get_token(); }
    };
    using parent_cb = typename stop_token_of_t<R>::template callback_type<detail::request_stop_fn>;
    R r;
    std::atomic<int> remaining{2};
    int result = 2;
    std::exception_ptr err;
    std::optional<non_void_t<value_type>> val;
    inplace_stop_source stop;
    std::optional<parent_cb> on_stop;
    connect_result_t<S, src_rcv> sop;
    connect_result_t<T, trig_rcv> top;
    op(S&& s_, T&& t_, R&& r_)
        : r(std::move(r_)), sop(exec::connect(std::move(s_), src_rcv{this})), top(exec::connect(std::move(t_), trig_rcv{this})) {}
    op(op&&) = delete;
    void start() noexcept {
      on_stop.emplace(exec::get_stop_token(r), detail::request_stop_fn{&stop});
      exec::start(sop);
      exec::start(top);
    }
    void arrive() noexcept {
      if (remaining.fetch_sub(1, std::memory_order_acq_rel) != 1) return;
      on_stop.reset();
      if (result == 0) deliver<value_type>(r, std::move(*val));
      else if (result == 1) r.set_error(std::move(err));
      else r.set_done();
    }
  };
  template <class R>
  auto connect(R&& r) && {
    return op<std::decay_t<R>>(std::move(s), std::move(t), std::decay_t<R>(std::forward<R>(r)));
  }
};
template <sender S, sender T>
auto stop_when(S&& s, T&& t) {
  return stop_when_sender<std::decay_t<S>, std::decay_t<T>>{std::forward<S>(s), std::forward<T>(t)};
}
template <sender T>
auto stop_when(T&& t) {
  return closure{[t = std::decay_t<T>(std::forward<T>(t))](auto&& s) mutable {
    return exec::stop_when(std::forward<decltype(s)>(s), std::move(t));
  }};
}

// ---- schedulers ---------------------------------------------------------------------
template <class Sch>
auto schedule(Sch&& sch) {
  return sch.schedule();
}
template <class Sch, class D>
auto schedule_after(Sch&& sch, D d) {
  return sch.schedule_after(d);
}
template <class Sch, class TP>
auto schedule_at(Sch&& sch, TP tp) {
  return sch.schedule_at(tp);
}
template <class Sch>
auto now(Sch&& sch) {
  return sch.now();
}

// on(scheduler, sender): start the sender on the scheduler's context
template <class Sch, sender S>
auto on(Sch&& sch, S&& s) {
  return let_value(exec::schedule(sch), [s = std::decay_t<S>(std::forward<S>(s))]() mutable { return std::move(s); });
}
// via(scheduler): continue on the scheduler's context after the source completes with a value
template <class Sch, sender S>
auto via(Sch sch, S&& s) {
  using V = value_t<S>;
  if constexpr (std::is_void_v<V>) {
    return let_value(std::forward<S>(s), [sch]() mutable { return exec::schedule(sch); });
  } else {
    return let_value(std::forward<S>(s), [sch](V& v) mutable {
      return then(exec::schedule(sch), [&v]() mutable { return std::move(v); });
    });
  }
}

// ---- repeat_effect_until / repeat_effect ------------------------------------------------
template <class S, class P>
struct repeat_until_sender {
  static_assert(std::is_void_v<value_t<S>>, "repeat_effect_until needs a sender of no value");
  using value_type = void;
  S s;
  P pred;
  template <class R>
  struct op {
    struct rcv {
      op* o;
      void set_value() noexcept { o->iteration_finished(kValue, nullptr); }
      template <class E>
      void set_error(E&& e) noexcept {
        o->iteration_finished(kError, to_exception_ptr(std::forward<E>(e)));
      }
      void set_done() noexcept { o->iteration_finished(kDone, nullptr); }
      auto get_stop_token() const noexcept { return exec::get_stop_token(o->r); }
    };
    // st: kStarting while start() of the current iteration is on the stack; an
    // iteration that finishes meanwhile leaves its outcome for run() to pick up.
    enum : int { kStarting = 0, kSuspended = 1, kValue = 2, kError = 3, kDone = 4 };
    S s;
    P pred;
    R r;
    manual_lifetime<connect_result_t<const S&, rcv>> inner;
    bool live = false;
    std::atomic<int> st{kStarting};
    std::exception_ptr pending_err;
    op(S&& s_, P&& p_, R&& r_) : s(std::move(s_)), pred(std::move(p_)), r(std::move(r_)) {}
    op(op&&) = delete;
    ~op() {
      if (live) inner.destruct();
    }
    void start() noexcept { run(); }
    // returns true when another iteration should run
    bool after_iteration(int code) noexcept {
      inner.destruct();
      live = false;
      if (code == kError) {
        r.set_error(std::move(pending_err));
        return false;
      }
      if (code == kDone) {
        r.set_done();
        return false;
      }
      bool stop_now;
      try {
        stop_now = pred();
      } catch (...) {
        r.set_error(std::current_exception());
        return false;
      }
      if (stop_now) {
        r.set_value();
        return false;
      }
      return true;
    }
    void run() noexcept {
      for (;;) {
        try {
          inner.construct_with([&] { return exec::connect(std::as_const(s), rcv{this}); });
          live = true;
        } catch (...) {
          r.set_error(std::current_exception());
          return;
        }
        st.store(kStarting, std::memory_order_relaxed);
        exec::start(inner.get());
        int expected = kStarting;
        if (st.compare_exchange_strong(expected, kSuspended, std::memory_order_acq_rel)) return;  // completes later
        if (!after_iteration(expected)) return;
      }
    }
    void iteration_finished(int code, std::exception_ptr ep) noexcept {
      pending_err = std::move(ep);
      int expected = kStarting;
      if (st.compare_exchange_strong(expected, code, std::memory_order_acq_rel)) return;  // run() continues
      if (after_iteration(code)) run();
    }
  };
  template <class R>
  auto connect(R&& r) && {
    return op<std::decay_t<R>>(std::move(s), std::move(pred), std::decay_t<R>(std::forward<R>(r)));
  }
};
template <sender S, class P>
auto repeat_effect_until(S&& s, P&& p) {
  return repeat_until_sender<std::decay_t<S>, std::decay_t<P>>{std::forward<S>(s), std::forward<P>(p)};
}
template <sender S>
auto repeat_effect(S&& s) {
  return repeat_effect_until(std::forward<S>(s), [] { return false; });
}

// ---- create<V>(fn): adapt a callback-style API ----------------------------------------
template <class V, class Fn>
struct create_sender {
  using value_type = V;
  Fn fn;
  template <class R>
  struct op {
    R r;
    Fn fn;
    // the handle handed to fn; it may be kept and completed later from any thread
    struct handle {
      op* o;
      template <class... A>
      void set_value(A&&... a) noexcept {
        o->r.set_value(std::forward<A>(a)...);
      }
      template <class E>
      void set_error(E&& e) noexcept {
        o->r.set_error(std::forward<E>(e));
      }
      void set_done() noexcept { o->r.set_done(); }
      auto get_stop_token() const noexcept { return exec::get_stop_token(o->r); }
    };
    void start() noexcept {
      try {
        fn(handle{this});
      } catch (...) {
        r.set_error(std::current_exception());
      }
    }
  };
  template <class R>
  auto connect(R&& r) && {
    return op<std::decay_t<R>>{std::forward<R>(r), std::move(fn)};
  }
};
template <class V = void, class Fn>
auto create(Fn&& fn) {
  return create_sender<V, std::decay_t<Fn>>{std::forward<Fn>(fn)};
}

// ---- sync_wait ------------------------------------------------------------------------
namespace detail {
template <class V>
struct sync_wait_state {
  std::mutex mu;
  std::condition_variable cv;
  bool finished = false;
  std::optional<non_void_t<V>> val;
  std::exception_ptr err;
  inplace_stop_token tok;
  void finish() {
    std::lock_guard lk(mu);
    finished = true;
    cv.notify_one();
  }
};
template <class V>
struct sync_wait_rcv {
  sync_wait_state<V>* st;
  template <class... A>
  void set_value(A&&... a) noexcept {
    try {
      st->val.emplace(std::forward<A>(a)...);
    } catch (...) {
      st->err = std::current_exception();
    }
    st->finish();
  }
  template <class E>
  void set_error(E&& e) noexcept {
    st->err = to_exception_ptr(std::forward<E>(e));
    st->finish();
  }
  void set_done() noexcept { st->finish(); }
  inplace_stop_token get_stop_token() const noexcept { return st->tok; }
};
}  // namespace detail

// Blocks the calling thread. nullopt = the sender completed with done; errors are rethrown.
template <sender S>
std::optional<non_void_t<value_t<S>>> sync_wait(S&& s, inplace_stop_token tok = {}) {
  using V = value_t<S>;
  detail::sync_wait_state<V> st;
  st.tok = tok;
  auto op = exec::connect(std::forward<S>(s), detail::sync_wait_rcv<V>{&st});
  exec::start(op);
  {
    std::unique_lock lk(st.mu);
    st.cv.wait(lk, [&] { return st.finished; });
  }
  if (st.err) std::rethrow_exception(st.err);
  return std::move(st.val);
}

}  // namespace eux::exec
