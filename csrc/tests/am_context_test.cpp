// Two ucx_am_context instances in one process, each on its own thread, talking over
// TCP loopback (the arrangement of the reference's ucx_am_context_test.cpp:169-187).
#include <arpa/inet.h>

#include <cstring>
#include <random>
#include <thread>

#include "check.hpp"
#include "eux/exec/async_scope.hpp"
#include "eux/exec/stream.hpp"
#include "eux/exec/contexts.hpp"
#include "eux/ucxx/ucx_am_context.hpp"

using namespace eux::ucxx;
namespace ex = eux::exec;
using namespace std::chrono_literals;

struct Runner {
  DefaultUcxMemoryResourceManager mr;
  ucx_am_context ctx;
  ex::inplace_stop_source stop;
  std::thread th;
  explicit Runner(const char* name, bool handle_err = false, std::chrono::milliseconds to = 300ms) : ctx(mr, name, to, handle_err) {
    th = std::thread([this] { ctx.run(stop.get_token()); });
    while (!ctx_running()) std::this_thread::yield();
  }
  bool ctx_running() {
    // the loop publishes its thread id when it starts
    return ex::sync_wait(ex::then(ctx.get_scheduler().schedule(), [] { return true; })).has_value();
  }
  ~Runner() {
    stop.request_stop();
    th.join();
  }
};

static uint16_t free_port() {
  int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  sockaddr_in in{};
  in.sin_family = AF_INET;
  in.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  in.sin_port = 0;
  ::bind(fd, (sockaddr*)&in, sizeof(in));
  socklen_t len = sizeof(in);
  getsockname(fd, (sockaddr*)&in, &len);
  uint16_t p = ntohs(in.sin_port);
  ::close(fd);
  return p;
}
static std::unique_ptr<sockaddr> loopback(uint16_t port) {
  auto* in = new sockaddr_in{};
  in->sin_family = AF_INET;
  in->sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  in->sin_port = htons(port);
  return std::unique_ptr<sockaddr>(reinterpret_cast<sockaddr*>(in));
}

EUX_TEST(schedule_and_timers) {
  Runner a("a");
  auto sch = a.ctx.get_scheduler();
  auto t0 = std::chrono::steady_clock::now();
  CHECK(ex::sync_wait(sch.schedule_after(20ms)).has_value());
  auto dt = std::chrono::steady_clock::now() - t0;
  CHECK(dt >= 19ms && dt < 500ms);
  CHECK(ex::sync_wait(sch.schedule_at(sch.now() + 5ms)).has_value());
  // a long timer is cancelled by stop_when
  t0 = std::chrono::steady_clock::now();
  auto r = ex::sync_wait(ex::stop_when(sch.schedule_after(10s), sch.schedule_after(10ms)));
  CHECK(!r.has_value());
  CHECK(std::chrono::steady_clock::now() - t0 < 2s);
}

// A word in host memory that somebody else writes (a kernel, through mapped pinned memory; here a thread).
EUX_TEST(wait_for_a_flag_word) {
  Runner a("a");
  auto sch = a.ctx.get_scheduler();
  alignas(64) static uint64_t word = 0;
  static int published = 0;
  word = 0;
  published = 0;
  const volatile uint64_t* flag = &word;
  std::thread writer([] {
    std::this_thread::sleep_for(15ms);
    published = 42;
    __atomic_store_n(&word, uint64_t(7), __ATOMIC_RELEASE);
  });
  auto t0 = std::chrono::steady_clock::now();
  CHECK(ex::sync_wait(sch.schedule_when_flag(flag, 7)).has_value());
  CHECK(std::chrono::steady_clock::now() - t0 >= 14ms);
  CHECK_EQ(published, 42);  // what was written before the word is visible after it
  writer.join();
  // already there: completes at once, also for a smaller value
  CHECK(ex::sync_wait(sch.schedule_when_flag(flag, 7)).has_value());
  CHECK(ex::sync_wait(sch.schedule_when_flag(flag, 3)).has_value());
  // never reached: the wait can be cancelled, and the context still serves afterwards
  t0 = std::chrono::steady_clock::now();
  CHECK(!ex::sync_wait(ex::stop_when(sch.schedule_when_flag(flag, 1000), sch.schedule_after(10ms))).has_value());
  CHECK(std::chrono::steady_clock::now() - t0 < 2s);
  // several waiters on a counter that grows: each completes once its value is reached
  std::atomic<int> done8{0}, done9{0};
  ex::async_scope scope;
  scope.spawn_detached(ex::then(sch.schedule_when_flag(flag, 8), [&] { done8 = 1; }));
  scope.spawn_detached(ex::then(sch.schedule_when_flag(flag, 9), [&] { done9 = 1; }));
  std::this_thread::sleep_for(5ms);
  CHECK(done8 == 0 && done9 == 0);
  __atomic_store_n(&word, uint64_t(8), __ATOMIC_RELEASE);
  for (int i = 0; i < 200 && !done8; ++i) std::this_thread::sleep_for(1ms);
  CHECK(done8 == 1 && done9 == 0);
  __atomic_store_n(&word, uint64_t(9), __ATOMIC_RELEASE);
  ex::sync_wait(scope.join());
  CHECK(done9 == 1);
}

EUX_TEST(accept_cancelled_by_stop_token) {
  Runner srv("srv", true);
  auto acc = accept_endpoint(srv.ctx.get_scheduler(), free_port());
  ex::timed_single_thread_context timer;
  auto r = ex::sync_wait(ex::stop_when(acc.next(), ex::schedule_after(timer.get_scheduler(), 30ms)));
  CHECK(!r.has_value());
  ex::sync_wait(acc.cleanup());
}

// The accept stream with the stream algorithms, as a server loop is usually written:
// for_each(take_until(accept_endpoint(...), single(stop_on_request(token))), on_batch).
EUX_TEST(accept_stream_with_for_each_and_take_until) {
  Runner srv("srv", true), cli("cli", true);
  const uint16_t port = free_port();
  ex::inplace_stop_source stop;
  std::atomic<int> accepted{0};
  ex::async_scope scope;
  scope.spawn_detached(ex::upon_error(
      ex::for_each(ex::take_until(accept_endpoint(srv.ctx.get_scheduler(), port), ex::single(ex::stop_on_request(stop.get_token()))),
                   [&](std::vector<std::pair<uint64_t, std::error_code>>&& batch) {
                     for (auto& [id, ec] : batch)
                       if (id != 0 && !ec) accepted.fetch_add(1);
                   }),
      [](std::exception_ptr) {}));
  int connected = 0;
  for (int attempt = 0; attempt < 200 && connected < 2; ++attempt) {
    try {
      auto c = ex::sync_wait(connect_endpoint(cli.ctx.get_scheduler(), nullptr, loopback(port), sizeof(sockaddr_in)));
      if (c) ++connected;
    } catch (...) {
      std::this_thread::sleep_for(5ms);
    }
  }
  CHECK_EQ(connected, 2);
  for (int i = 0; i < 400 && accepted.load() < 2; ++i) std::this_thread::sleep_for(5ms);
  CHECK_EQ(accepted.load(), 2);
  stop.request_stop();  // ends the pending next(), then the stream is cleaned up
  ex::sync_wait(scope.join());
}

struct Pair {
  Runner srv{"server", true}, cli{"client", true};
  conn_id_t cli_conn = 0, srv_conn = 0;
  std::optional<accept_connection> acc;
  Pair() {
    uint16_t port = free_port();
    acc.emplace(accept_endpoint(srv.ctx.get_scheduler(), port));
    ex::async_scope scope;
    auto fut = scope.spawn_future(acc->next());
    // the listener is opened by next() on the server thread; retry until it is there
    for (int i = 0; i < 100 && !cli_conn; ++i) {
      try {
        auto c = ex::sync_wait(connect_endpoint(cli.ctx.get_scheduler(), nullptr, loopback(port), sizeof(sockaddr_in)));
        if (c) cli_conn = *c;
      } catch (...) {
        std::this_thread::sleep_for(5ms);
      }
    }
    auto batch = ex::sync_wait(std::move(fut));
    ex::sync_wait(scope.join());
    if (batch && !batch->empty()) srv_conn = (*batch)[0].first;
  }
};

EUX_TEST(connect_accept_small_and_large_messages) {
  Pair p;
  CHECK(p.cli_conn != 0 && p.srv_conn != 0);
  auto csch = p.cli.ctx.get_scheduler();
  auto ssch = p.srv.ctx.get_scheduler();
  for (size_t size : {size_t(0), size_t(8), size_t(4096), size_t(65536), size_t(3 << 20)}) {
    std::vector<char> payload(size);
    for (size_t i = 0; i < size; ++i) payload[i] = char(i * 7 + size);
    uint64_t hdr[2] = {size, 0xabcdef};
    ucx_am_data d{};
    d.header = {hdr, sizeof(hdr)};
    d.buffer = {payload.data(), size};
    d.buffer_type = ucx_memory_type::HOST;
    ex::async_scope scope;
    auto rfut = scope.spawn_future(connection_recv(ssch, ucx_memory_type::HOST));
    CHECK(ex::sync_wait(connection_send(csch, p.cli_conn, d)).has_value());
    auto got = ex::sync_wait(std::move(rfut));
    ex::sync_wait(scope.join());
    CHECK(got.has_value());
    auto& raw = got->get_raw_data();
    CHECK_EQ(raw.header.size, sizeof(hdr));
    CHECK(std::memcmp(raw.header.data, hdr, sizeof(hdr)) == 0);
    CHECK_EQ(raw.buffer.size, size);
    CHECK(size == 0 || std::memcmp(raw.buffer.data, payload.data(), size) == 0);
    CHECK_EQ(got->conn_id(), p.srv_conn);
  }
}

EUX_TEST(header_first_then_buffer_and_iovec) {
  Pair p;
  auto csch = p.cli.ctx.get_scheduler();
  auto ssch = p.srv.ctx.get_scheduler();
  // scatter-gather send: three segments, sizes carried in the application header
  std::vector<std::vector<char>> segs = {std::vector<char>(100, 'a'), std::vector<char>(50000, 'b'), std::vector<char>(7, 'c')};
  uint64_t hdr[3] = {100, 50000, 7};
  ucx_buffer_t iov[3] = {{segs[0].data(), 100}, {segs[1].data(), 50000}, {segs[2].data(), 7}};
  ucx_am_iovec v{};
  v.header = {hdr, sizeof(hdr)};
  v.buffer_vec = iov;
  v.buffer_count = 3;
  v.buffer_type = ucx_memory_type::HOST;
  for (int mode = 0; mode < 2; ++mode) {
    ex::async_scope scope;
    auto hfut = scope.spawn_future(connection_recv_header(ssch));
    auto sfut = scope.spawn_future(connection_send(csch, p.cli_conn, v));
    auto h = ex::sync_wait(std::move(hfut));
    CHECK(h.has_value() && h->index() == 0);
    auto& [key, header] = std::get<0>(*h);
    CHECK_EQ(header.size(), sizeof(hdr));
    const uint64_t* sz = static_cast<const uint64_t*>(header.data());
    CHECK(p.srv.ctx.view_pending_am_desc(key) != nullptr);
    if (mode == 0) {  // receive as iov
      UcxBufferVec dst(p.srv.mr, ucx_memory_type::HOST, std::vector<size_t>{sz[0], sz[1], sz[2]});
      auto b = ex::sync_wait(connection_recv_buffer(ssch, key, std::move(dst)));
      CHECK(b.has_value());
      auto& bv = b->buffer();
      CHECK_EQ(bv.size(), 3u);
      for (int i = 0; i < 3; ++i) CHECK(std::memcmp(bv[i].data, segs[i].data(), segs[i].size()) == 0);
    } else {  // receive contiguous, then split without copying
      auto b = ex::sync_wait(connection_recv_buffer(ssch, key, ucx_memory_type::HOST));
      CHECK(b.has_value());
      CHECK_EQ(b->buffer().size(), 50107u);
      auto split = std::move(b->buffer()).to_buffer_vec({100, 50000, 7});
      CHECK(split.has_backing_buffer());
      CHECK(std::memcmp(split[1].data, segs[1].data(), 50000) == 0);
      CHECK(static_cast<char*>(split[2].data)[6] == 'c');
    }
    CHECK(ex::sync_wait(std::move(sfut)).has_value());
    ex::sync_wait(scope.join());
  }
  // eager message through recv_header arrives whole
  ucx_am_data d{};
  uint64_t h2 = 42;
  char small[16] = "hello";
  d.header = {&h2, 8};
  d.buffer = {small, 16};
  ex::async_scope scope;
  auto hfut = scope.spawn_future(connection_recv_header(ssch));
  ex::sync_wait(connection_send(csch, p.cli_conn, d));
  auto h = ex::sync_wait(std::move(hfut));
  ex::sync_wait(scope.join());
  CHECK(h && h->index() == 1);
  CHECK(std::memcmp(std::get<1>(*h).buffer().data(), "hello", 6) == 0);
}

EUX_TEST(connect_by_worker_address_and_echo) {
  Runner a("alpha"), b("beta");
  std::vector<std::byte> addr;
  CHECK_EQ(b.ctx.get_ucp_address(addr), UCS_OK);
  auto c = ex::sync_wait(connect_endpoint(a.ctx.get_scheduler(), addr));
  CHECK(c.has_value());
  // echo: b receives, divides every float by two on a thread pool, sends back on the same connection
  ex::static_thread_pool pool(2);
  std::vector<float> v(1 << 16);
  for (size_t i = 0; i < v.size(); ++i) v[i] = float(i);
  uint32_t hdr = 7;
  ucx_am_data d{};
  d.header = {&hdr, 4};
  d.buffer = {v.data(), v.size() * 4};
  ex::async_scope scope;
  scope.spawn_detached(ex::let_value(connection_recv(b.ctx.get_scheduler(), ucx_memory_type::HOST), [&](active_message_bundle& m) {
    return ex::let_value(ex::on(pool.get_scheduler(), ex::just_from([&m] {
                           auto& raw = m.get_raw_data();
                           float* f = static_cast<float*>(raw.buffer.data);
                           for (size_t i = 0; i < raw.buffer.size / 4; ++i) f[i] /= 2.0f;
                         })),
                         [&] { return connection_send(b.ctx.get_scheduler(), m.conn_id(), m.get_raw_data()); });
  }));
  CHECK(ex::sync_wait(connection_send(a.ctx.get_scheduler(), *c, d)).has_value());
  auto back = ex::sync_wait(connection_recv(a.ctx.get_scheduler(), ucx_memory_type::HOST));
  ex::sync_wait(scope.join());
  CHECK(back.has_value());
  const float* f = static_cast<const float*>(back->get_raw_data().buffer.data);
  CHECK_EQ(back->get_raw_data().buffer.size, v.size() * 4);
  for (size_t i = 0; i < v.size(); i += 997) CHECK_EQ(f[i], float(i) / 2.0f);
}

// Two contexts built on one shared transport context: its eager limit applies to both
// (a 256-byte payload goes by rendezvous when the limit is 64).
EUX_TEST(shared_transport_context) {
  ucp_context_h shared = nullptr;
  setenv("EUX_EAGER_LIMIT", "64", 1);
  CHECK_EQ(ucx_am_context::init_ucp_context("shared", shared, true, false), UCS_OK);
  unsetenv("EUX_EAGER_LIMIT");
  CHECK(shared != nullptr && shared->eager_limit == 64 && shared->mt_workers_shared);
  {
    DefaultUcxMemoryResourceManager mr;
    ucx_am_context a(mr, shared, "shared_a", 300ms, true), b(mr, shared, "shared_b", 300ms, true);
    ex::inplace_stop_source stop;
    std::thread ta([&] { a.run(stop.get_token()); }), tb([&] { b.run(stop.get_token()); });
    ex::sync_wait(a.get_scheduler().schedule());
    ex::sync_wait(b.get_scheduler().schedule());
    std::vector<std::byte> addr;
    b.get_ucp_address(addr);
    auto c = ex::sync_wait(connect_endpoint(a.get_scheduler(), addr));
    CHECK(c.has_value());
    uint32_t h = 7;
    std::vector<char> body(256, 'x');
    ucx_am_data d{};
    d.header = {&h, 4};
    d.buffer = {body.data(), body.size()};
    d.buffer_type = ucx_memory_type::HOST;
    ex::async_scope scope;
    scope.spawn_detached(ex::upon_error(connection_send(a.get_scheduler(), *c, d), [](std::exception_ptr) {}));
    auto got = ex::sync_wait(connection_recv_header(b.get_scheduler()));
    CHECK(got.has_value());
    // above the limit the header arrives first and the payload waits for a buffer
    CHECK(got->index() == 0);
    if (got->index() == 0) {
      auto& [key, hdr] = std::get<0>(*got);
      auto buf = ex::sync_wait(connection_recv_buffer(b.get_scheduler(), key, ucx_memory_type::HOST));
      CHECK(buf.has_value() && buf->buffer().size() == 256);
    }
    ex::sync_wait(scope.cleanup());
    stop.request_stop();
    ta.join();
    tb.join();
  }
  ucx_am_context::destroy_ucp_context(shared);
}

EUX_TEST(unroutable_address_reports_error) {
  Runner cli("cli", true, 100ms);
  auto* in = new sockaddr_in{};
  in->sin_family = AF_INET;
  inet_pton(AF_INET, "192.0.2.1", &in->sin_addr);  // TEST-NET-1: never routable
  in->sin_port = htons(9);
  auto t0 = std::chrono::steady_clock::now();
  bool failed = false;
  try {
    auto r = ex::sync_wait(connect_endpoint(cli.ctx.get_scheduler(), nullptr, std::unique_ptr<sockaddr>((sockaddr*)in), sizeof(sockaddr_in)));
    failed = !r.has_value();
  } catch (const std::system_error& e) {
    failed = std::string(e.code().category().name()) == "UCX";
  }
  CHECK(failed);
  CHECK(std::chrono::steady_clock::now() - t0 < 3s);
}

EUX_TEST(peer_failure_reaches_error_handler) {
  auto srv = std::make_unique<Runner>("srv", true);
  Runner cli("cli", true);
  std::vector<std::byte> addr;
  srv->ctx.get_ucp_address(addr);
  auto c = ex::sync_wait(connect_endpoint(cli.ctx.get_scheduler(), addr));
  CHECK(c.has_value());
  std::atomic<uint64_t> seen{0};
  ex::async_scope scope;
  scope.spawn_detached(handle_error_connection(cli.ctx.get_scheduler(), [&](conn_id_t id, std::error_code ec) {
    seen = id;
    return false;  // no reconnect
  }));
  srv.reset();  // the peer goes away on the host side
  for (int i = 0; i < 400 && !seen; ++i) std::this_thread::sleep_for(5ms);
  ex::sync_wait(scope.cleanup());
  CHECK_EQ(seen.load(), *c);
  // sending on the failed connection is an error, not a hang
  uint32_t h = 1;
  ucx_am_data d{};
  d.header = {&h, 4};
  CHECK_THROWS(ex::sync_wait(connection_send(cli.ctx.get_scheduler(), *c, d)));
}

// 10 000 active messages, 16-byte header {seq, tag}, payload size drawn from
// {8 B, 256 B, 4 KiB, 64 KiB}, seeded random bytes, every byte verified.
EUX_TEST(ten_thousand_messages_verified) {
  Pair p;
  CHECK(p.cli_conn != 0);
  const int N = 10000;
  const size_t sizes[4] = {8, 256, 4096, 65536};
  auto gen_payload = [&](uint64_t seq, std::vector<unsigned char>& out) {
    std::mt19937_64 rng(seq * 1315423911u + 17);
    out.resize(sizes[rng() % 4]);
    for (size_t i = 0; i + 8 <= out.size(); i += 8) {
      uint64_t w = rng();
      std::memcpy(out.data() + i, &w, 8);
    }
  };
  std::atomic<int> verified{0};
  std::atomic<bool> bad{false};
  ex::async_scope scope;
  int received = 0;
  auto ssch = p.srv.ctx.get_scheduler();
  scope.spawn_detached(ex::repeat_effect_until(
      ex::defer([&] {
        return ex::then(connection_recv(ssch, ucx_memory_type::HOST), [&](active_message_bundle m) {
          auto& raw = m.get_raw_data();
          uint64_t hdr[2];
          if (raw.header.size != 16) { bad = true; return; }
          std::memcpy(hdr, raw.header.data, 16);
          std::vector<unsigned char> want;
          gen_payload(hdr[0], want);
          if (hdr[0] != uint64_t(received) || hdr[1] != (hdr[0] ^ 0x5555) || raw.buffer.size != want.size() ||
              std::memcmp(raw.buffer.data, want.data(), want.size()) != 0)
            bad = true;
          ++received;
          verified.fetch_add(1);
        });
      }),
      [&] { return received >= N; }));
  auto csch = p.cli.ctx.get_scheduler();
  std::vector<unsigned char> payload;
  for (int i = 0; i < N; ++i) {
    gen_payload(i, payload);
    uint64_t hdr[2] = {uint64_t(i), uint64_t(i) ^ 0x5555};
    ucx_am_data d{};
    d.header = {hdr, 16};
    d.buffer = {payload.data(), payload.size()};
    CHECK(ex::sync_wait(connection_send(csch, p.cli_conn, d)).has_value());
  }
  ex::sync_wait(scope.join());
  CHECK_EQ(verified.load(), N);
  CHECK(!bad.load());
}

EUX_TEST_MAIN()
