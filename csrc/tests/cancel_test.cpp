// Cancellation of every kind of operation of ucx_am_context by a stop token: the operation ends with
// "done" (no value, no error) promptly, leaves nothing behind, and the context and the connection keep
// working afterwards. One case per cancel node: connect, send (rendezvous, before the receiver asked for the
// bytes), recv, recv_header, recv_buffer (host rendezvous whose data never comes), accept, timers, flag
// waits. (The reference tests connect and accept under a stop token, ucx_am_context_test.cpp:1108-1190;
// its per-operation cancel protocol is ucx_am_context.hpp:1297-1361.) A device pull in flight is the one
// thing that cannot be withdrawn (a kernel is writing the buffer); that case needs a GPU and lives in the
// GPU tests.
#include <arpa/inet.h>

#include <atomic>
#include <cstring>
#include <thread>

#include "check.hpp"
#include "eux/exec/async_scope.hpp"
#include "eux/exec/contexts.hpp"
#include "eux/ucxx/ucx_am_context.hpp"

using namespace eux::ucxx;
namespace ex = eux::exec;
namespace tr = eux::ucxx::transport;
using namespace std::chrono_literals;

namespace {

struct Runner {
  DefaultUcxMemoryResourceManager mr;
  ucx_am_context ctx;
  ex::inplace_stop_source stop;
  std::thread th;
  explicit Runner(const char* name) : ctx(mr, name, 300ms, true) {
    th = std::thread([this] { ctx.run(stop.get_token()); });
    ex::sync_wait(ctx.get_scheduler().schedule());
  }
  ~Runner() {
    stop.request_stop();
    th.join();
  }
};

uint16_t free_port() {
  int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  sockaddr_in in{};
  in.sin_family = AF_INET;
  in.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  ::bind(fd, (sockaddr*)&in, sizeof(in));
  socklen_t len = sizeof(in);
  getsockname(fd, (sockaddr*)&in, &len);
  uint16_t p = ntohs(in.sin_port);
  ::close(fd);
  return p;
}
std::unique_ptr<sockaddr> addr_of(uint32_t ip_host_order, uint16_t port) {
  auto* in = new sockaddr_in{};
  in->sin_family = AF_INET;
  in->sin_addr.s_addr = htonl(ip_host_order);
  in->sin_port = htons(port);
  return std::unique_ptr<sockaddr>(reinterpret_cast<sockaddr*>(in));
}

// Two connected contexts (client -> server through the server's worker address).
struct Pair {
  Runner srv{"server"}, cli{"client"};
  conn_id_t conn = 0;
  Pair() {
    std::vector<std::byte> addr;
    srv.ctx.get_ucp_address(addr);
    auto c = ex::sync_wait(connect_endpoint(cli.ctx.get_scheduler(), addr));
    conn = c ? *c : 0;
  }
};

// Runs `op` under a timer of `after`: true when the operation ended as "done" (cancelled), and within a
// second (a cancel that had to wait for the operation's own completion would take as long as the operation).
template <class Sender>
bool cancelled_promptly(Sender&& op, std::chrono::milliseconds after = 30ms) {
  ex::timed_single_thread_context timer;
  const auto t0 = std::chrono::steady_clock::now();
  auto r = ex::sync_wait(ex::stop_when(std::forward<Sender>(op), ex::schedule_after(timer.get_scheduler(), after)));
  return !r.has_value() && std::chrono::steady_clock::now() - t0 < 1s;
}

// One small message client -> server, received whole: what must still work after every cancellation.
bool still_works(Pair& p, uint64_t tag) {
  char body[32] = "still here";
  ucx_am_data d{};
  d.header = {&tag, 8};
  d.buffer = {body, sizeof(body)};
  ex::async_scope scope;
  auto rf = scope.spawn_future(connection_recv(p.srv.ctx.get_scheduler(), ucx_memory_type::HOST));
  const bool sent = ex::sync_wait(connection_send(p.cli.ctx.get_scheduler(), p.conn, d)).has_value();
  auto got = ex::sync_wait(std::move(rf));
  ex::sync_wait(scope.join());
  if (!sent || !got) return false;
  uint64_t seen = 0;
  std::memcpy(&seen, got->get_raw_data().header.data, 8);
  return seen == tag && std::memcmp(got->get_raw_data().buffer.data, body, sizeof(body)) == 0;
}

}  // namespace

EUX_TEST(connect_is_cancellable_while_the_peer_does_not_answer) {
  Runner cli("client");
  // A listener that completes the TCP handshake (from its backlog) but never speaks the worker protocol:
  // the connection attempt stays pending until it is withdrawn.
  int lfd = ::socket(AF_INET, SOCK_STREAM, 0);
  sockaddr_in in{};
  in.sin_family = AF_INET;
  in.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  CHECK(::bind(lfd, (sockaddr*)&in, sizeof(in)) == 0 && ::listen(lfd, 4) == 0);
  socklen_t len = sizeof(in);
  getsockname(lfd, (sockaddr*)&in, &len);
  CHECK(cancelled_promptly(connect_endpoint(cli.ctx.get_scheduler(), nullptr, addr_of(0x7F000001u, ntohs(in.sin_port)), sizeof(sockaddr_in))));
  ::close(lfd);
  // the context is as usable as before
  Runner srv("server");
  std::vector<std::byte> addr;
  srv.ctx.get_ucp_address(addr);
  CHECK(ex::sync_wait(connect_endpoint(cli.ctx.get_scheduler(), addr)).has_value());
}

EUX_TEST(accept_is_cancellable_while_nobody_connects) {
  Runner srv("server");
  auto acc = accept_endpoint(srv.ctx.get_scheduler(), free_port());
  CHECK(cancelled_promptly(acc.next()));
  ex::sync_wait(acc.cleanup());
}

EUX_TEST(recv_is_cancellable_while_no_message_is_pending) {
  Pair p;
  CHECK(p.conn != 0);
  CHECK(cancelled_promptly(connection_recv(p.srv.ctx.get_scheduler(), ucx_memory_type::HOST)));
  CHECK(still_works(p, 1));  // the withdrawn receive did not swallow the next message
}

EUX_TEST(recv_header_is_cancellable_while_no_message_is_pending) {
  Pair p;
  CHECK(cancelled_promptly(connection_recv_header(p.srv.ctx.get_scheduler())));
  CHECK_EQ(p.srv.ctx.pending_message_count(), 0u);
  CHECK(still_works(p, 2));
}

EUX_TEST(rendezvous_send_is_cancellable_before_the_receiver_asks_for_the_bytes) {
  Pair p;
  std::vector<char> big(1 << 20, 'x');  // far beyond the eager limit: announced, then held until asked for
  uint64_t tag = 77;
  ucx_am_data d{};
  d.header = {&tag, 8};
  d.buffer = {big.data(), big.size()};
  CHECK(cancelled_promptly(connection_send(p.cli.ctx.get_scheduler(), p.conn, d)));
  // The announcement had already reached the server. Its header can still be read there, but the bytes are
  // gone: asking for them fails instead of waiting for data that will never be sent.
  auto h = ex::sync_wait(connection_recv_header(p.srv.ctx.get_scheduler()));
  CHECK(h.has_value() && h->index() == 0);
  const size_t key = std::get<0>(*h).first;
  bool failed = false;
  try {
    ex::timed_single_thread_context timer;
    auto r = ex::sync_wait(ex::stop_when(connection_recv_buffer(p.srv.ctx.get_scheduler(), key, ucx_memory_type::HOST),
                                         ex::schedule_after(timer.get_scheduler(), 500ms)));
    failed = !r.has_value();
  } catch (...) {
    failed = true;
  }
  CHECK(failed);
  CHECK(still_works(p, 3));  // the user's memory was released by the cancellation: `big` may go now
}

EUX_TEST(recv_buffer_is_cancellable_while_the_data_does_not_come) {
  Pair p;
  // the clear-to-send of the server gets lost on the wire, so the client never sends the bytes
  tr::set_fault_hook([](const std::string& worker, uint8_t type, uint64_t) { return worker == "server" && type == tr::kRndvCts; });
  std::vector<char> big(1 << 20, 'y');
  uint64_t tag = 5;
  ucx_am_data d{};
  d.header = {&tag, 8};
  d.buffer = {big.data(), big.size()};
  ex::async_scope scope;
  std::atomic<int> send_state{0};  // 1 value, 2 error, 3 done
  scope.spawn_detached(ex::upon_done(ex::upon_error(ex::then(connection_send(p.cli.ctx.get_scheduler(), p.conn, d), [&] { send_state = 1; }),
                                                    [&](std::exception_ptr) { send_state = 2; }),
                                     [&] { send_state = 3; }));
  auto h = ex::sync_wait(connection_recv_header(p.srv.ctx.get_scheduler()));
  CHECK(h.has_value() && h->index() == 0);
  CHECK(cancelled_promptly(connection_recv_buffer(p.srv.ctx.get_scheduler(), std::get<0>(*h).first, ucx_memory_type::HOST), 50ms));
  tr::set_fault_hook({});
  // the sender is told that its message will not be read, and its operation ends (not with a value)
  scope.request_stop();
  ex::sync_wait(scope.join());
  CHECK(send_state.load() != 1);
  CHECK(still_works(p, 4));
}

EUX_TEST(timers_are_cancellable) {
  Runner r("ctx");
  auto sch = r.ctx.get_scheduler();
  CHECK(cancelled_promptly(sch.schedule_after(10s)));
  CHECK(cancelled_promptly(sch.schedule_at(sch.now() + 10s)));
  // a timer that is not cancelled still fires
  const auto t0 = std::chrono::steady_clock::now();
  CHECK(ex::sync_wait(sch.schedule_after(20ms)).has_value());
  CHECK(std::chrono::steady_clock::now() - t0 >= 19ms);
}

EUX_TEST(flag_waits_are_cancellable) {
  Runner r("ctx");
  alignas(8) static uint64_t word = 0;
  CHECK(cancelled_promptly(r.ctx.get_scheduler().schedule_when_flag(&word, 1)));
  __atomic_store_n(&word, uint64_t(1), __ATOMIC_RELEASE);
  CHECK(ex::sync_wait(r.ctx.get_scheduler().schedule_when_flag(&word, 1)).has_value());
}

EUX_TEST(stopping_the_context_ends_parked_operations) {
  auto r = std::make_unique<Runner>("ctx");
  ex::async_scope scope;
  std::atomic<int> ended{0};
  scope.spawn_detached(ex::upon_done(ex::upon_error(ex::then(connection_recv(r->ctx.get_scheduler(), ucx_memory_type::HOST), [&](auto&&) { ended = 1; }),
                                                    [&](std::exception_ptr) { ended = 2; }),
                                     [&] { ended = 3; }));
  std::this_thread::sleep_for(10ms);
  r->stop.request_stop();
  ex::sync_wait(scope.join());
  CHECK(ended.load() == 3 || ended.load() == 2);  // not a value: nothing ever arrived
  r.reset();
}

EUX_TEST_MAIN()
