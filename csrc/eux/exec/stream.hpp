// Streams and the few stream algorithms the active-message context's users rely on
// (the reference takes them from libunifex: for_each, take_until, single, stop_on_request,
// stop_if_requested, variant_sender; see ucx_context/ucx_am_context/ucx_am_context_test.cpp:349-372).
//
// A stream is an object with `next()` -> sender of the next element (completing with done when
// the stream has ended) and `cleanup()` -> sender<void> to run once after the last `next()`.
// `accept_endpoint(...)` is such a stream.
#pragma once

#include <atomic>
#include <memory>
#include <optional>
#include <variant>

#include "eux/exec/async_scope.hpp"
#include "eux/exec/exec.hpp"

namespace eux::exec {

template <class S>
concept stream = requires(S& s) {
  s.next();
  s.cleanup();
};
template <class S>
using next_sender_t = decltype(std::declval<S&>().next());

// ---- variant_sender: one of several senders with the same value type ---------------------------
template <class... S>
struct variant_sender {
  using first_t = std::tuple_element_t<0, std::tuple<S...>>;
  using value_type = value_t<first_t>;
  static_assert((std::is_same_v<value_type, value_t<S>> && ...), "variant_sender needs one value type");
  std::variant<S...> alt;
  template <class T>
    requires(std::is_same_v<std::decay_t<T>, S> || ...)
  variant_sender(T&& t) : alt(std::forward<T>(t)) {}  // NOLINT: implicit on purpose
  template <class R>
  struct op {
    std::variant<std::monostate, detail::op_holder<connect_result_t<S, R>>...> inner;
    op(variant_sender&& vs, R&& r) {
      std::visit(
          [&](auto& s) {
            using Sd = std::decay_t<decltype(s)>;
            inner.template emplace<detail::op_holder<connect_result_t<Sd, R>>>([&] { return exec::connect(std::move(s), std::move(r)); });
          },
          vs.alt);
    }
    op(op&&) = delete;
    void start() noexcept {
      std::visit(
          [](auto& b) {
            if constexpr (!std::is_same_v<std::decay_t<decltype(b)>, std::monostate>) exec::start(b.op);
          },
          inner);
    }
  };
  template <class R>
  auto connect(R&& r) && {
    return op<std::decay_t<R>>(std::move(*this), std::decay_t<R>(std::forward<R>(r)));
  }
};

// ---- stop_if_requested: done when the receiver's stop token is set, a value otherwise ----------
struct stop_if_requested_sender {
  using value_type = void;
  template <class R>
  struct op {
    R r;
    void start() noexcept {
      if (exec::get_stop_token(r).stop_requested()) r.set_done();
      else r.set_value();
    }
  };
  template <class R>
  auto connect(R&& r) const {
    return op<std::decay_t<R>>{std::forward<R>(r)};
  }
};
inline stop_if_requested_sender stop_if_requested() { return {}; }

// ---- stop_on_request(token): completes with done when the token (or the receiver's) is set -----
template <class Tok>
struct stop_on_request_sender {
  using value_type = void;
  Tok tok;
  template <class R>
  struct op {
    struct on_stop {
      op* self;
      void operator()() const noexcept { self->fire(); }
    };
    Tok tok;
    R r;
    std::atomic<int> phase{0};  // 0 starting, 1 armed, 2 fired
    std::optional<typename Tok::template callback_type<on_stop>> cb_token;
    std::optional<typename stop_token_of_t<R>::template callback_type<on_stop>> cb_receiver;
    op(Tok t, R&& rr) : tok(t), r(std::move(rr)) {}
    op(op&&) = delete;
    void start() noexcept {
      cb_token.emplace(tok, on_stop{this});
      cb_receiver.emplace(exec::get_stop_token(r), on_stop{this});
      int expected = 0;
      if (!phase.compare_exchange_strong(expected, 1, std::memory_order_acq_rel)) complete();  // fired while arming
    }
    void fire() noexcept {
      if (phase.exchange(2, std::memory_order_acq_rel) == 1) complete();
    }
    void complete() noexcept {
      cb_token.reset();
      cb_receiver.reset();
      r.set_done();
    }
  };
  template <class R>
  auto connect(R&& r) const {
    return op<std::decay_t<R>>(tok, std::decay_t<R>(std::forward<R>(r)));
  }
};
template <class Tok>
auto stop_on_request(Tok tok) {
  return stop_on_request_sender<Tok>{tok};
}

// ---- single(sender): a stream of exactly one element -------------------------------------------
template <class S>
struct single_stream {
  std::optional<S> s;
  auto next() {
    using V = value_t<S>;
    using out = variant_sender<S, just_done_sender<V>>;
    if (s) {
      S taken = std::move(*s);
      s.reset();
      return out(std::move(taken));
    }
    return out(just_done<V>());
  }
  auto cleanup() { return just(); }
};
template <sender S>
auto single(S&& s) {
  return single_stream<std::decay_t<S>>{std::decay_t<S>(std::forward<S>(s))};
}

// ---- take_until(source, trigger): the source's elements until the trigger produces one or ends --
template <class Source, class Trigger>
class take_until_stream {
  struct state {
    Source source;
    Trigger trigger;
    inplace_stop_source stop_source_next;  // set when the trigger fires: ends a pending next()
    inplace_stop_source stop_trigger;      // set by cleanup(): ends the trigger's pending next()
    async_scope scope;
    std::atomic<bool> fired{false};
    bool watching = false;
    state(Source&& s, Trigger&& t) : source(std::move(s)), trigger(std::move(t)) {}
  };
  std::unique_ptr<state> st_;

 public:
  take_until_stream(Source&& s, Trigger&& t) : st_(std::make_unique<state>(std::move(s), std::move(t))) {}
  auto next() {
    state* st = st_.get();
    if (!st->watching) {
      st->watching = true;
      auto fire = [st] {
        st->fired.store(true, std::memory_order_release);
        st->stop_source_next.request_stop();
      };
      // value, error or done of the trigger all end the stream
      st->scope.spawn_detached(with_query_value(
          upon_done(upon_error(then(st->trigger.next(), [fire](auto&&...) { fire(); }), [fire](std::exception_ptr) { fire(); }), fire),
          get_stop_token, st->stop_trigger.get_token()));
    }
    using inner = with_stop_token_sender<next_sender_t<Source>, inplace_stop_token>;
    using out = variant_sender<inner, just_done_sender<value_t<inner>>>;
    if (st->fired.load(std::memory_order_acquire)) return out(just_done<value_t<inner>>());
    return out(with_query_value(st->source.next(), get_stop_token, st->stop_source_next.get_token()));
  }
  auto cleanup() {
    state* st = st_.get();
    return sequence(just_from([st] { st->stop_trigger.request_stop(); }), st->scope.join(), st->source.cleanup(), st->trigger.cleanup());
  }
};
template <stream Source, stream Trigger>
auto take_until(Source&& s, Trigger&& t) {
  return take_until_stream<std::decay_t<Source>, std::decay_t<Trigger>>(std::decay_t<Source>(std::forward<Source>(s)),
                                                                          std::decay_t<Trigger>(std::forward<Trigger>(t)));
}

// ---- for_each(stream, fn): fn on every element; completes when the stream ends, after cleanup() --
template <stream S, class F>
auto for_each(S&& s, F&& f) {
  struct box {
    std::decay_t<S> s;
    std::decay_t<F> f;
    bool ended = false;
  };
  auto st = std::make_shared<box>(box{std::decay_t<S>(std::forward<S>(s)), std::decay_t<F>(std::forward<F>(f)), false});
  auto body = repeat_effect_until(defer([st] {
                                    return upon_done(then(st->s.next(), [st](auto&&... v) { st->f(std::forward<decltype(v)>(v)...); }),
                                                     [st] { st->ended = true; });
                                  }),
                                  [st] { return st->ended; });
  // cleanup runs on both ways out; an error of the loop is delivered after it
  return let_error(sequence(std::move(body), defer([st] { return st->s.cleanup(); })), [st](std::exception_ptr e) {
    return sequence(upon_error(defer([st] { return st->s.cleanup(); }), [](std::exception_ptr) {}), just_error<void>(e));
  });
}

}  // namespace eux::exec
