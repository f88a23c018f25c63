// Latency and throughput of the active-message context (the counterpart of the
// reference's ucx_context/ucx_am_context/ucx_am_context_perf.cpp:119-439), with a
// device-payload mode in which the payload lives in GPU memory and moves through
// the transfer kernel.
//
//   eux_ucx_am_context_perf [-t latency|throughput] [-H header_bytes] [-M message_bytes]
//                           [-w warmup] [-i iterations] [-m host|cuda] [-d device]
//                           [--server | --client <address-hex>]
//
// Without --server/--client both ends run in this process on two threads and
// connect over TCP loopback through the worker address. Latency is half the
// ping-pong round trip (min / mean / p50 / p99 / p99.9); throughput is messages
// and megabytes per second of a one-way stream with a final acknowledgement.
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <iostream>
#include <numeric>
#include <string>
#include <thread>
#include <vector>

#include "eux/exec/async_scope.hpp"
#include "eux/ucxx/cuda/ucx_cuda_context.hpp"
#include "eux/ucxx/cuda/ucx_cuda_memory_manager.hpp"
#include "eux/ucxx/ucx_am_context.hpp"

using namespace eux::ucxx;
namespace ex = eux::exec;
using clk = std::chrono::steady_clock;

struct Options {
  std::string test = "latency";
  size_t header = 8, message = 64;
  int warmup = 10, iters = 100;
  bool cuda = false;
  int device = 0;
  bool server = false;
  std::string client_addr;
};

struct Node {
  std::unique_ptr<UcxMemoryResourceManager> mr;
  std::unique_ptr<ucx_am_context> ctx;
  ex::inplace_stop_source stop;
  std::thread th;
  Node(const char* name, const Options& o) {
    std::unique_ptr<UcxAutoDeviceContext> dev;
    if (o.cuda) {
      UcxCudaMemoryResourceManager::Options mo;
      mo.device = o.device;
      mr = std::make_unique<UcxCudaMemoryResourceManager>(mo);
      dev = std::make_unique<UcxAutoCudaDeviceContext>(o.device);
    } else {
      mr = std::make_unique<DefaultUcxMemoryResourceManager>();
    }
    ctx = std::make_unique<ucx_am_context>(*mr, name, std::chrono::milliseconds(5000), true, 0, std::move(dev));
    th = std::thread([this] { ctx->run(stop.get_token()); });
    ex::sync_wait(ctx->get_scheduler().schedule());
  }
  ~Node() {
    stop.request_stop();
    th.join();
  }
};

static std::vector<std::byte> from_hex(const std::string& h) {
  std::vector<std::byte> out(h.size() / 2);
  for (size_t i = 0; i < out.size(); ++i) out[i] = std::byte(std::stoi(h.substr(2 * i, 2), nullptr, 16));
  return out;
}
static std::string to_hex(const std::vector<std::byte>& b) {
  static const char* d = "0123456789abcdef";
  std::string s;
  for (auto x : b) {
    s += d[(int(x) >> 4) & 15];
    s += d[int(x) & 15];
  }
  return s;
}

// echo `count` messages back to where they came from
static void serve(Node& n, const Options& o, int count, bool echo_payload) {
  auto sched = n.ctx->get_scheduler();
  const auto type = o.cuda ? ucx_memory_type::CUDA : ucx_memory_type::HOST;
  for (int i = 0; i < count; ++i) {
    auto m = ex::sync_wait(connection_recv(sched, type));
    if (!m) return;
    if (echo_payload) {
      ex::sync_wait(connection_send(sched, m->conn_id(), m->get_raw_data()));
    } else if (i + 1 == count) {  // throughput: acknowledge the last message only
      ucx_am_data ack{};
      uint64_t h = 1;
      ack.header = {&h, sizeof(h)};
      ex::sync_wait(connection_send(sched, m->conn_id(), ack));
    }
  }
}

static void run_client(Node& n, conn_id_t conn, const Options& o) {
  auto sched = n.ctx->get_scheduler();
  const auto type = o.cuda ? ucx_memory_type::CUDA : ucx_memory_type::HOST;
  std::vector<char> header(std::max<size_t>(o.header, 1), 'h');
  UcxBuffer payload(*n.mr, type, o.message);
  ucx_am_data d{};
  d.header = {header.data(), header.size()};
  d.buffer = {payload.data(), payload.size()};
  d.buffer_type = type;
  if (o.test == "latency") {
    std::vector<double> us;
    for (int i = 0; i < o.warmup + o.iters; ++i) {
      auto t0 = clk::now();
      ex::sync_wait(connection_send(sched, conn, d));
      auto back = ex::sync_wait(connection_recv(sched, type));
      auto t1 = clk::now();
      if (!back) {
        std::fprintf(stderr, "receive cancelled\n");
        return;
      }
      if (i >= o.warmup) us.push_back(std::chrono::duration<double, std::micro>(t1 - t0).count() / 2.0);
    }
    std::sort(us.begin(), us.end());
    auto pct = [&](double q) { return us[std::min(us.size() - 1, size_t(q * (us.size() - 1) + 0.5))]; };
    double mean = std::accumulate(us.begin(), us.end(), 0.0) / us.size();
    std::printf("latency(us) memory=%s header=%zu message=%zu iters=%d min=%.2f mean=%.2f p50=%.2f p99=%.2f p999=%.2f\n",
                o.cuda ? "cuda" : "host", o.header, o.message, o.iters, us.front(), mean, pct(0.5), pct(0.99), pct(0.999));
  } else {
    for (int i = 0; i < o.warmup; ++i) ex::sync_wait(connection_send(sched, conn, d));
    // the warm-up messages are acknowledged once, then the timed stream starts
    (void)ex::sync_wait(connection_recv(sched, ucx_memory_type::HOST));
    auto t0 = clk::now();
    ex::async_scope scope;
    std::atomic<int> inflight{0};
    for (int i = 0; i < o.iters; ++i) {
      while (inflight.load() >= 64) std::this_thread::yield();  // bounded window
      inflight.fetch_add(1);
      scope.spawn_detached(ex::upon_error(ex::then(connection_send(sched, conn, d), [&] { inflight.fetch_sub(1); }),
                                          [&](std::exception_ptr) { inflight.fetch_sub(1); }));
    }
    (void)ex::sync_wait(connection_recv(sched, ucx_memory_type::HOST));
    auto t1 = clk::now();
    ex::sync_wait(scope.join());
    double s = std::chrono::duration<double>(t1 - t0).count();
    std::printf("throughput memory=%s header=%zu message=%zu iters=%d qps=%.0f MBps=%.1f\n", o.cuda ? "cuda" : "host", o.header, o.message,
                o.iters, o.iters / s, o.iters * double(o.message) / s / 1e6);
  }
}

int main(int argc, char** argv) {
  Options o;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    auto next = [&] { return i + 1 < argc ? std::string(argv[++i]) : std::string(); };
    if (a == "-t") o.test = next();
    else if (a == "-H") o.header = std::stoul(next());
    else if (a == "-M") o.message = std::stoul(next());
    else if (a == "-w") o.warmup = std::stoi(next());
    else if (a == "-i") o.iters = std::stoi(next());
    else if (a == "-m") o.cuda = next() == "cuda";
    else if (a == "-d") o.device = std::stoi(next());
    else if (a == "--server") o.server = true;
    else if (a == "--client") o.client_addr = next();
    else {
      std::fprintf(stderr, "usage: %s [-t latency|throughput] [-H bytes] [-M bytes] [-w n] [-i n] [-m host|cuda] [-d dev] [--server|--client hex]\n", argv[0]);
      return 2;
    }
  }
  const bool latency = o.test == "latency";
  const int served = latency ? o.warmup + o.iters : o.iters;
  try {
    if (o.server) {
      Node srv("perf_server", o);
      std::vector<std::byte> addr;
      srv.ctx->get_ucp_address(addr);
      std::cout << "ADDRESS " << to_hex(addr) << std::endl;
      if (!latency) serve(srv, o, o.warmup, false);
      serve(srv, o, served, latency);
      return 0;
    }
    if (!o.client_addr.empty()) {
      Node cli("perf_client", o);
      auto conn = ex::sync_wait(connect_endpoint(cli.ctx->get_scheduler(), from_hex(o.client_addr)));
      if (!conn) return 1;
      run_client(cli, *conn, o);
      return 0;
    }
    Node srv("perf_server", o), cli("perf_client", o);
    std::vector<std::byte> addr;
    srv.ctx->get_ucp_address(addr);
    auto conn = ex::sync_wait(connect_endpoint(cli.ctx->get_scheduler(), addr));
    if (!conn) return 1;
    std::thread server_thread([&] {
      if (!latency && o.warmup > 0) serve(srv, o, o.warmup, false);
      serve(srv, o, served, latency);
    });
    run_client(cli, *conn, o);
    server_thread.join();
  } catch (const std::exception& e) {
    std::fprintf(stderr, "perf failed: %s\n", e.what());
    return 1;
  }
  return 0;
}
