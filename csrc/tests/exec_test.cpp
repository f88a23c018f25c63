// Unit tests of the sender/receiver core (CPU only).
#include <chrono>
#include <string>
#include <thread>

#include "check.hpp"
#include "eux/exec/async_scope.hpp"
#include "eux/exec/contexts.hpp"
#include "eux/exec/exec.hpp"
#include "eux/exec/stream.hpp"

using namespace eux::exec;
namespace ex = eux::exec;
using namespace std::chrono_literals;

EUX_TEST(just_then_pipe) {
  auto r = sync_wait(just(20) | then([](int x) { return x + 1; }) | then([](int x) { return x * 2; }));
  CHECK(r.has_value() && *r == 42);
  auto v = sync_wait(just() | then([] {}));
  CHECK(v.has_value());
}

EUX_TEST(errors_and_done) {
  CHECK_THROWS(sync_wait(just(1) | then([](int) -> int { throw std::runtime_error("boom"); })));
  auto r = sync_wait(just_error<int>(std::make_error_code(std::errc::timed_out)) |
                     upon_error([](std::exception_ptr e) { return error_code_of(e) == std::errc::timed_out ? 7 : 0; }));
  CHECK(r && *r == 7);
  auto d = sync_wait(just_done<int>());
  CHECK(!d.has_value());
  auto d2 = sync_wait(just_done<int>() | upon_done([] { return 5; }));
  CHECK(d2 && *d2 == 5);
  auto e2 = sync_wait(just_error<int>(std::make_error_code(std::errc::io_error)) | let_error([](std::exception_ptr) { return just(9); }));
  CHECK(e2 && *e2 == 9);
  auto d3 = sync_wait(just_done<int>() | let_done([] { return just(11); }));
  CHECK(d3 && *d3 == 11);
}

EUX_TEST(let_value_keeps_state) {
  auto r = sync_wait(let_value(just(std::string("abc")), [](std::string& s) { return just(s.size()) | then([&s](size_t n) { return s + std::to_string(n); }); }));
  CHECK(r && *r == "abc3");
  int order = 0;
  auto s = sequence(just_from([&] { CHECK_EQ(order++, 0); }), just_from([&] { CHECK_EQ(order++, 1); }), just_from([&] { return order; }));
  auto o = sync_wait(std::move(s));
  CHECK(o && *o == 2);
  auto df = sync_wait(defer([] { return just(3); }));
  CHECK(df && *df == 3);
}

EUX_TEST(when_all_values_and_failure) {
  static_thread_pool pool(3);
  auto sch = pool.get_scheduler();
  auto r = sync_wait(when_all(on(sch, just(1)), on(sch, just(std::string("x"))), on(sch, just())));
  CHECK(r.has_value());
  CHECK_EQ(std::get<0>(*r), 1);
  CHECK_EQ(std::get<1>(*r), "x");
  timed_single_thread_context timer;
  // one branch fails: the long timer is cancelled promptly
  auto t0 = std::chrono::steady_clock::now();
  CHECK_THROWS(sync_wait(when_all(schedule_after(timer.get_scheduler(), 5s), just_error(std::make_error_code(std::errc::io_error)))));
  CHECK(std::chrono::steady_clock::now() - t0 < 2s);
}

EUX_TEST(stop_when_timeout_and_completion) {
  timed_single_thread_context timer;
  auto sch = timer.get_scheduler();
  auto t0 = std::chrono::steady_clock::now();
  // trigger fires first: source (5 s timer) is cancelled -> done
  auto r = sync_wait(stop_when(schedule_after(sch, 5s) | then([] { return 1; }), schedule_after(sch, 20ms)));
  CHECK(!r.has_value());
  // source first: the trigger is cancelled, value comes through
  auto r2 = sync_wait(stop_when(schedule_after(sch, 10ms) | then([] { return 2; }), schedule_after(sch, 5s)));
  CHECK(r2 && *r2 == 2);
  CHECK(std::chrono::steady_clock::now() - t0 < 2s);
}

EUX_TEST(repeat_effect_until_inline_and_async) {
  int n = 0;
  auto r = sync_wait(repeat_effect_until(just_from([&] { ++n; }), [&] { return n >= 100000; }));
  CHECK(r.has_value());
  CHECK_EQ(n, 100000);
  static_thread_pool pool(2);
  int m = 0;
  auto r2 = sync_wait(repeat_effect_until(on(pool.get_scheduler(), just_from([&] { ++m; })), [&] { return m >= 2000; }));
  CHECK(r2.has_value());
  CHECK_EQ(m, 2000);
  // error ends the loop
  int k = 0;
  CHECK_THROWS(sync_wait(repeat_effect_until(just_from([&] { if (++k == 5) throw std::runtime_error("x"); }), [] { return false; })));
  CHECK_EQ(k, 5);
}

EUX_TEST(stop_token_callbacks) {
  inplace_stop_source src;
  int hits = 0;
  {
    inplace_stop_callback cb(src.get_token(), [&] { ++hits; });
    inplace_stop_callback cb2(src.get_token(), [&] { ++hits; });
    CHECK(src.request_stop());
    CHECK(!src.request_stop());
  }
  CHECK_EQ(hits, 2);
  inplace_stop_callback late(src.get_token(), [&] { ++hits; });
  CHECK_EQ(hits, 3);
  // with_query_value injects a token
  inplace_stop_source s2;
  s2.request_stop();
  static_thread_pool pool(1);
  auto r = sync_wait(with_query_value(schedule(pool.get_scheduler()), get_stop_token, s2.get_token()));
  CHECK(!r.has_value());
}

EUX_TEST(async_scope_spawn_and_join) {
  static_thread_pool pool(4);
  async_scope scope;
  std::atomic<int> n{0};
  for (int i = 0; i < 200; ++i) scope.spawn_detached(on(pool.get_scheduler(), just_from([&] { n.fetch_add(1); })));
  auto fut = scope.spawn_future(on(pool.get_scheduler(), just(41) | then([](int x) { return x + 1; })));
  auto v = sync_wait(std::move(fut));
  CHECK(v && *v == 42);
  sync_wait(scope.join());
  CHECK_EQ(n.load(), 200);
  // cleanup cancels a long timer
  timed_single_thread_context timer;
  scope.spawn_detached(schedule_after(timer.get_scheduler(), 10s));
  auto t0 = std::chrono::steady_clock::now();
  sync_wait(scope.cleanup());
  CHECK(std::chrono::steady_clock::now() - t0 < 2s);
}

// join() under a deadline: work that ignores its stop request does not hold the joiner for ever; once the work
// has finished, the same scope joins as usual. Many rounds, so that the work's end and the deadline also meet.
EUX_TEST(async_scope_join_gives_up_at_a_deadline) {
  timed_single_thread_context timer;
  auto sch = timer.get_scheduler();
  {
    async_scope scope;
    std::thread worker;
    std::atomic<bool> release{false};
    scope.spawn_detached(create<int>([&](auto h) {
                           worker = std::thread([h, &release]() mutable {
                             while (!release.load()) std::this_thread::sleep_for(1ms);
                             h.set_value(1);
                           });
                         }) |
                         then([](int) {}));
    auto t0 = std::chrono::steady_clock::now();
    auto r = sync_wait(stop_when(scope.join(), schedule_after(sch, 30ms)));
    CHECK(!r.has_value());  // done: the deadline came first
    CHECK(std::chrono::steady_clock::now() - t0 < 2s);
    release.store(true);
    CHECK(sync_wait(scope.join()).has_value());
    worker.join();
  }
  static_thread_pool pool(2);
  int joined = 0, gave_up = 0;
  for (int round = 0; round < 300; ++round) {
    async_scope scope;
    scope.spawn_detached(on(pool.get_scheduler(), just_from([round] { std::this_thread::sleep_for(std::chrono::microseconds(50 + (round * 37) % 400)); })));
    auto r = sync_wait(stop_when(scope.join(), schedule_after(sch, std::chrono::microseconds(50 + (round * 53) % 400))));
    r.has_value() ? ++joined : ++gave_up;
    CHECK(sync_wait(scope.join()).has_value());
  }
  CHECK_EQ(joined + gave_up, 300);
}

EUX_TEST(any_sender_type_erasure) {
  any_sender_of<int> a = just(5) | then([](int x) { return x * 3; });
  auto r = sync_wait(std::move(a));
  CHECK(r && *r == 15);
  any_sender_of<void> b = just();
  CHECK(sync_wait(std::move(b)).has_value());
  any_sender_of<int> c = just_error<int>(std::make_error_code(std::errc::io_error));
  CHECK_THROWS(sync_wait(std::move(c)));
  timed_single_thread_context timer;
  any_sender_of<void> d = schedule_after(timer.get_scheduler(), 10s);
  auto t0 = std::chrono::steady_clock::now();
  auto rr = sync_wait(stop_when(std::move(d), schedule_after(timer.get_scheduler(), 10ms)));
  CHECK(!rr.has_value());
  CHECK(std::chrono::steady_clock::now() - t0 < 2s);
}

EUX_TEST(create_callback_adapter) {
  std::thread th;
  auto s = create<int>([&](auto h) { th = std::thread([h]() mutable { std::this_thread::sleep_for(5ms); h.set_value(77); }); });
  auto r = sync_wait(std::move(s));
  th.join();
  CHECK(r && *r == 77);
}

static task<int> add_later(static_thread_pool::scheduler sch, int a, int b) {
  co_await schedule(sch);
  int x = co_await (just(a) | then([](int v) { return v * 2; }));
  co_return x + b;
}
static task<void> outer(static_thread_pool::scheduler sch, int& out) {
  out = co_await add_later(sch, 10, 1);
  try {
    co_await just_error(std::make_error_code(std::errc::timed_out));
  } catch (const std::system_error& e) {
    if (e.code() == std::errc::timed_out) out += 100;
  }
}
static task<int> cancelled_inside() {
  co_await just_done();
  co_return 1;
}

EUX_TEST(coroutine_task) {
  static_thread_pool pool(2);
  int out = 0;
  auto r = sync_wait(outer(pool.get_scheduler(), out));
  CHECK(r.has_value());
  CHECK_EQ(out, 121);
  auto d = sync_wait(cancelled_inside());
  CHECK(!d.has_value());
}

// A stream that counts: next() yields 0, 1, 2, ... (after a short timer each when `ctx` is given),
// ends after `limit` elements when limit >= 0.
struct return_int {
  int v;
  int operator()() const { return v; }
};
struct counting_stream {
  ex::timed_single_thread_context* ctx = nullptr;
  int limit = -1;
  int next_value = 0;
  int* cleanups = nullptr;
  auto next() {
    using timed = decltype(ex::then(ex::schedule_after(ctx->get_scheduler(), 1ms), return_int{0}));
    using out = ex::variant_sender<timed, ex::just_sender<int>, ex::just_done_sender<int>>;
    if (limit >= 0 && next_value >= limit) return out(ex::just_done<int>());
    const int v = next_value++;
    if (ctx) return out(ex::then(ex::schedule_after(ctx->get_scheduler(), 1ms), return_int{v}));
    return out(ex::just(v));
  }
  auto cleanup() {
    return ex::just_from([c = cleanups] {
      if (c) ++*c;
    });
  }
};

EUX_TEST(streams_for_each_take_until_single) {
  // for_each over a finite stream, cleanup exactly once
  int cleanups = 0, sum = 0;
  ex::sync_wait(ex::for_each(counting_stream{nullptr, 5, 0, &cleanups}, [&](int v) { sum += v; }));
  CHECK_EQ(sum, 0 + 1 + 2 + 3 + 4);
  CHECK_EQ(cleanups, 1);
  // an endless timed stream, ended from another thread through take_until(single(stop_on_request))
  ex::timed_single_thread_context ctx;
  ex::inplace_stop_source stop;
  std::atomic<int> seen{0};
  int cleanups2 = 0;
  std::thread stopper([&] {
    while (seen.load() < 5) std::this_thread::sleep_for(1ms);
    stop.request_stop();
  });
  auto t0 = std::chrono::steady_clock::now();
  ex::sync_wait(ex::for_each(ex::take_until(counting_stream{&ctx, -1, 0, &cleanups2}, ex::single(ex::stop_on_request(stop.get_token()))),
                             [&](int) { seen.fetch_add(1); }));
  stopper.join();
  CHECK(seen.load() >= 5);
  CHECK_EQ(cleanups2, 1);
  CHECK(std::chrono::steady_clock::now() - t0 < 5s);
  // a trigger that is already set ends the stream before its first element
  ex::inplace_stop_source set;
  set.request_stop();
  int n = 0;
  ex::sync_wait(ex::for_each(ex::take_until(counting_stream{&ctx, -1, 0, nullptr}, ex::single(ex::stop_on_request(set.get_token()))),
                             [&](int) { ++n; }));
  CHECK(n <= 1);
  // an error thrown by the callback reaches the caller, after cleanup
  int cleanups3 = 0;
  CHECK_THROWS(ex::sync_wait(ex::for_each(counting_stream{nullptr, 3, 0, &cleanups3}, [&](int v) {
    if (v == 1) throw std::runtime_error("boom");
  })));
  CHECK_EQ(cleanups3, 1);
  // stop_if_requested and variant_sender on their own
  CHECK(ex::sync_wait(ex::stop_if_requested()).has_value());
  CHECK(!ex::sync_wait(ex::with_query_value(ex::stop_if_requested(), ex::get_stop_token, set.get_token())).has_value());
  ex::variant_sender<ex::just_sender<int>, ex::just_done_sender<int>> vs(ex::just(7));
  CHECK_EQ(*ex::sync_wait(std::move(vs)), 7);
}

EUX_TEST_MAIN()
