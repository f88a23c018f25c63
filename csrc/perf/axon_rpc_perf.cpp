// RPC storm: latency and throughput of Axon RPCs that carry one fp32 tensor and get it back
// with 1.0 added (the counterpart of the reference's axon/benchmark/axon_benchmark.cpp), for
// host and for device payloads.
//
//   eux_axon_rpc_perf [-m host|cuda] [-d device] [-s bytes[,bytes...]] [-n requests] [-o outstanding]
//                     [-w warmup] [--server | --client <address-hex>]
//   eux_axon_rpc_perf --mesh --rank R --world N --dir DIR [-m host|cuda] [-d device] [-n requests-per-peer]
//                     [-o outstanding-per-peer]
//
// --mesh is the all-to-all storm: N processes (one per GPU), each serving `plus_one` and calling it on
// every other rank with `outstanding` requests in flight per peer; tensor sizes are log-uniform in
// 256 B - 64 KiB. The ranks find each other through files in DIR (address, ready and done markers).
//
// Without --server/--client both runtimes live in this process. For every size it prints the
// round-trip latency with one request in flight (p50 / p99) and the request rate and payload
// bandwidth with `outstanding` requests in flight. Device payloads stay on the device: the
// receiver pulls them with the transfer kernel and the handler adds 1.0 with the same kernel.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <iostream>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include <cuda_runtime_api.h>

#include "eux/axon/axon_runtime.hpp"
#include "eux/ucxx/cuda/ucx_cuda_context.hpp"
#include "eux/ucxx/cuda/ucx_cuda_memory_manager.hpp"
#include "kernels/eux_kernels.h"

using namespace eux::axon;
using namespace eux::rpc;
using eux::ucxx::UcxBuffer;
namespace ex = eux::exec;
using clk = std::chrono::steady_clock;

struct Options {
  bool cuda = false;
  int device = 0;
  std::vector<size_t> sizes{256, 1024, 4096, 16384, 65536};
  int requests = 2000, outstanding = 64, warmup = 50;
  bool server = false;
  std::string client_addr;
  bool mesh = false;
  int rank = 0, world = 1;
  std::string dir;
};

static TensorMeta f32_meta(size_t bytes) {
  TensorMeta m;
  m.ndim = 1;
  m.dtype = {kDLFloat, 32, 1};
  m.shape = {static_cast<int64_t>(bytes / 4)};
  m.strides = {1};
  return m;
}

static std::shared_ptr<eux::ucxx::UcxMemoryResourceManager> make_mr(const Options& o) {
  if (!o.cuda) return std::make_shared<eux::ucxx::DefaultUcxMemoryResourceManager>();
  eux::ucxx::UcxCudaMemoryResourceManager::Options mo;
  mo.device = o.device;
  if (o.mesh) mo.arena_bytes = size_t(256) << 20;  // hundreds of 64 KiB tensors in flight
  return std::make_shared<eux::ucxx::UcxCudaMemoryResourceManager>(mo);
}

static std::unique_ptr<eux::ucxx::UcxAutoDeviceContext> make_dev(const Options& o) {
  if (!o.cuda) return nullptr;
  return std::make_unique<eux::ucxx::UcxAutoCudaDeviceContext>(o.device);
}

// y = x + 1 on the device, on a stream of the calling thread. The kernel publishes a sequence number in
// mapped pinned host memory when its stores are done; the caller gets the word and the number to wait for.
// Nobody calls into the driver to wait, so handlers on other threads and the transport's launches are
// not held up. Kernels of one thread run in order on its stream, so its numbers are reached in order.
struct DeviceDone {
  const volatile uint64_t* flag;
  uint64_t seq;
};
static DeviceDone device_plus_one_start(const void* x, void* y, size_t bytes, int device) {
  thread_local cudaStream_t st = nullptr;
  thread_local uint32_t* counter = nullptr;
  thread_local uint64_t* flag_host = nullptr;
  thread_local uint64_t* flag_dev = nullptr;
  thread_local uint64_t seq = 0;
  if (!st) {
    cudaSetDevice(device);
    cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
    cudaMalloc(reinterpret_cast<void**>(&counter), 256);
    cudaMemsetAsync(counter, 0, 256, st);
    void *h = nullptr, *d = nullptr;
    if (eux_host_alloc_mapped(&h, &d, 64) != 0) throw std::runtime_error("handler: no mapped host memory");
    flag_host = static_cast<uint64_t*>(h);
    flag_dev = static_cast<uint64_t*>(d);
  }
  eux_xfer_desc d{};
  d.src = x;
  d.dst = y;
  d.n_elems = bytes / 4;
  d.src_dtype = d.dst_dtype = EUX_DT_F32;
  d.op = EUX_OP_ADD;
  d.op_arg = 1.0f;
  d.flag = flag_dev;
  d.flag_value = ++seq;
  int rc = eux_xfer_launch(&d, counter, 0, st);
  if (rc != 0) throw std::runtime_error(std::string("handler kernel: ") + eux_error_string(rc));
  return {flag_host, seq};
}

static void register_plus_one(AxonRuntime& rt, const Options& o) {
  auto mr = rt.memory_resource();
  if (!o.cuda) {
    auto handler = [mr](const TensorMeta& m, UcxBuffer& buf) {
      UcxBuffer out(*mr, buf.type(), buf.size());
      const float* f = static_cast<const float*>(buf.data());
      float* g = static_cast<float*>(out.data());
      // the element count comes from the bytes that arrived, not from the caller's description of them
      const size_t count = buf.size() / sizeof(float);
      for (size_t i = 0; i < count; ++i) g[i] = f[i] + 1.0f;
      return std::tuple<TensorMeta, UcxBuffer>(m, std::move(out));
    };
    rt.RegisterFunction(function_id_t{1}, handler, "plus_one");
    return;
  }
  // Device tensors: the handler launches its kernel and returns a sender that the server's loop completes
  // when the kernel's flag shows up; the reply is built there. No thread waits for the GPU.
  const int dev = o.device;
  auto* worker = &rt.worker();
  auto handler = [mr, dev, worker](const TensorMeta& m, UcxBuffer& buf) {
    UcxBuffer out(*mr, buf.type(), buf.size());
    const DeviceDone done = device_plus_one_start(buf.data(), out.data(), buf.size(), dev);
    auto sched = worker->server_context()->get_scheduler();
    return ex::then(sched.schedule_when_flag(done.flag, done.seq),
                    [m, out = std::move(out)]() mutable { return std::tuple<TensorMeta, UcxBuffer>(m, std::move(out)); });
  };
  CustomMemoryPolicy<UcxBuffer> provider = [mr](eux::rpc::utils::TensorMetaSpan metas) {
    return UcxBuffer(*mr, ucx_memory_type::CUDA, eux::rpc::utils::CalculateTensorSize(metas[0]));
  };
  eux::axon::ServerMemoryPolicy mp;
  mp.on_host = false;
  mp.buffer_provider = provider;
  mp.provider_inline = true;  // a block from the memory manager's pool: nothing that could hold up the context's thread
  rt.worker().RegisterFunction(function_id_t{1}, handler, "plus_one", std::move(mp), MessageLifecyclePolicy{});
}

static ClientMemoryPolicy client_policy(AxonRuntime& rt, const Options& o) {
  ClientMemoryPolicy p;
  if (o.cuda) {
    auto mr = rt.memory_resource();
    p.on_host = false;
    p.provider_inline = true;
    p.buffer_provider = [mr](eux::rpc::utils::TensorMetaSpan metas) {
      return UcxBuffer(*mr, ucx_memory_type::CUDA, eux::rpc::utils::CalculateTensorSize(metas[0]));
    };
  }
  return p;
}

static double pct(std::vector<double>& v, double q) {
  if (v.empty()) return 0;
  std::sort(v.begin(), v.end());
  return v[std::min(v.size() - 1, size_t(q * (v.size() - 1) + 0.5))];
}

static int run_client(AxonRuntime& cli, const std::string& server_name, const Options& o) {
  auto mr = cli.memory_resource();
  const auto type = o.cuda ? ucx_memory_type::CUDA : ucx_memory_type::HOST;
  std::printf("%-6s %10s %12s %12s %12s %14s %12s\n", "memory", "bytes", "rtt_p50_us", "rtt_p99_us", "outstanding", "requests/s", "GB/s");
  for (size_t bytes : o.sizes) {
    std::vector<float> host(bytes / 4);
    for (size_t i = 0; i < host.size(); ++i) host[i] = float(i % 1000);
    // every request sends the same resident tensor: a view that does not own the bytes
    UcxBuffer resident(*mr, type, bytes);
    mr->memcpy(type, resident.data(), ucx_memory_type::HOST, host.data(), bytes);
    auto make_payload = [&] { return UcxBuffer(*mr, type, resident.data(), bytes, nullptr, false); };
    auto call = [&] {
      return cli.InvokeRpc(server_name, session_id_t{1}, function_id_t{1}, workflow_id_t{}, client_policy(cli, o), f32_meta(bytes), make_payload());
    };
    // correctness once per size
    {
      auto r = ex::sync_wait(call());
      if (!r || !r->header.status.ok()) {
        std::fprintf(stderr, "rpc failed at %zu bytes\n", bytes);
        return 1;
      }
      auto& out = std::get<UcxBuffer>(r->payload);
      std::vector<float> back(bytes / 4);
      mr->memcpy(ucx_memory_type::HOST, back.data(), out.type(), out.data(), bytes);
      for (size_t i = 0; i < back.size(); i += 17)
        if (back[i] != host[i] + 1.0f) {
          std::fprintf(stderr, "wrong result at %zu bytes, element %zu\n", bytes, i);
          return 1;
        }
    }
    // latency: one in flight
    std::vector<double> us;
    const int lat_iters = std::max(50, o.requests / 10);
    for (int i = 0; i < o.warmup + lat_iters; ++i) {
      auto t0 = clk::now();
      auto r = ex::sync_wait(call());
      auto t1 = clk::now();
      if (!r || !r->header.status.ok()) return 1;
      if (i >= o.warmup) us.push_back(std::chrono::duration<double, std::micro>(t1 - t0).count());
    }
    const double p50 = pct(us, 0.5), p99 = pct(us, 0.99);
    // throughput: a window of requests in flight
    std::atomic<int> inflight{0}, done{0}, failed{0};
    ex::async_scope scope;
    auto t0 = clk::now();
    for (int i = 0; i < o.requests; ++i) {
      while (inflight.load(std::memory_order_acquire) >= o.outstanding) std::this_thread::yield();
      inflight.fetch_add(1);
      scope.spawn_detached(ex::upon_error(ex::then(call(),
                                                   [&](InvokeResult r) {
                                                     if (!r.header.status.ok()) failed.fetch_add(1);
                                                     done.fetch_add(1);
                                                     inflight.fetch_sub(1, std::memory_order_release);
                                                   }),
                                          [&](std::exception_ptr) {
                                            failed.fetch_add(1);
                                            done.fetch_add(1);
                                            inflight.fetch_sub(1, std::memory_order_release);
                                          }));
    }
    ex::sync_wait(scope.join());
    const double s = std::chrono::duration<double>(clk::now() - t0).count();
    if (failed.load()) std::fprintf(stderr, "%d of %d requests failed at %zu bytes\n", failed.load(), o.requests, bytes);
    std::printf("%-6s %10zu %12.1f %12.1f %12d %14.0f %12.3f\n", o.cuda ? "cuda" : "host", bytes, p50, p99, o.outstanding, o.requests / s,
                2.0 * o.requests * double(bytes) / s / 1e9);
    std::fflush(stdout);
  }
  return 0;
}

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

// ---- all-to-all storm -------------------------------------------------------------------------
#include <fstream>
#include <random>
#include <sys/stat.h>

static bool file_exists(const std::string& p) {
  struct stat st{};
  return ::stat(p.c_str(), &st) == 0;
}
static void write_file(const std::string& p, const std::string& text) {
  const std::string tmp = p + ".tmp";
  {
    std::ofstream f(tmp);
    f << text;
  }
  ::rename(tmp.c_str(), p.c_str());
}
static bool wait_for_all(const std::string& dir, const std::string& stem, int world, int seconds) {
  const auto limit = clk::now() + std::chrono::seconds(seconds);
  for (;;) {
    int have = 0;
    for (int r = 0; r < world; ++r) have += file_exists(dir + "/" + stem + "." + std::to_string(r));
    if (have == world) return true;
    if (clk::now() > limit) return false;
    std::this_thread::sleep_for(std::chrono::milliseconds(2));
  }
}

static int run_mesh(const Options& o) {
  using namespace std::chrono_literals;
  const std::string me = "mesh" + std::to_string(o.rank);
  AxonRuntime rt(me, 8, 30000ms, make_dev(o), make_mr(o));
  register_plus_one(rt, o);
  if (auto ec = rt.Start()) throw std::runtime_error(ec.message());
  write_file(o.dir + "/addr." + std::to_string(o.rank), to_hex(rt.GetLocalAddress()));
  if (!wait_for_all(o.dir, "addr", o.world, 120)) throw std::runtime_error("not every rank published its address");
  std::vector<std::string> peers;
  for (int r = 0; r < o.world; ++r) {
    if (r == o.rank) continue;
    std::ifstream f(o.dir + "/addr." + std::to_string(r));
    std::string hex;
    f >> hex;
    const std::string name = "mesh" + std::to_string(r);
    rt.ConnectEndpoint(from_hex(hex), name);
    peers.push_back(name);
  }
  write_file(o.dir + "/ready." + std::to_string(o.rank), "1");
  if (!wait_for_all(o.dir, "ready", o.world, 120)) throw std::runtime_error("not every rank got ready");

  auto mr = rt.memory_resource();
  const auto type = o.cuda ? ucx_memory_type::CUDA : ucx_memory_type::HOST;
  const size_t max_bytes = 65536;
  UcxBuffer resident(*mr, type, max_bytes);
  {
    std::vector<float> host(max_bytes / 4);
    std::mt19937 rng(1234 + o.rank);
    std::uniform_real_distribution<float> u(-1.f, 1.f);
    for (auto& v : host) v = u(rng);
    mr->memcpy(type, resident.data(), ucx_memory_type::HOST, host.data(), max_bytes);
  }
  std::mt19937_64 rng(99 + o.rank);
  std::uniform_real_distribution<double> logu(std::log(256.0), std::log(65536.0));
  const int P = static_cast<int>(peers.size());
  // untimed warm-up: the first transfers between two processes map each other's memory and
  // switch on peer access, which takes a good fraction of a second
  {
    ex::async_scope warm;
    for (int i = 0; i < std::max(1, o.warmup); ++i)
      for (int p = 0; p < P; ++p)
        warm.spawn_detached(ex::upon_error(ex::then(rt.InvokeRpc(peers[p], session_id_t{1}, function_id_t{1}, workflow_id_t{}, client_policy(rt, o),
                                                                 f32_meta(max_bytes), UcxBuffer(*mr, type, resident.data(), max_bytes, nullptr, false)),
                                                    [](InvokeResult) {}),
                                           [](std::exception_ptr) {}));
    ex::sync_wait(warm.join());
  }
  write_file(o.dir + "/warm." + std::to_string(o.rank), "1");
  if (!wait_for_all(o.dir, "warm", o.world, 120)) throw std::runtime_error("not every rank finished its warm-up");
  std::vector<std::atomic<int>> inflight(P);
  for (auto& a : inflight) a.store(0);
  std::atomic<int> failed{0};
  std::mutex lat_mu;
  std::vector<double> lat_us;
  lat_us.reserve(size_t(P) * o.requests);
  uint64_t bytes_total = 0;
  ex::async_scope scope;
  std::vector<int> issued(P, 0);
  int remaining = P * o.requests;
  const auto t0 = clk::now();
  while (remaining > 0) {
    bool any = false;
    for (int p = 0; p < P; ++p) {
      if (issued[p] >= o.requests || inflight[p].load(std::memory_order_acquire) >= o.outstanding) continue;
      const size_t bytes = std::min<size_t>(max_bytes, (static_cast<size_t>(std::exp(logu(rng))) + 3) / 4 * 4);
      bytes_total += 2 * bytes;
      ++issued[p];
      --remaining;
      any = true;
      inflight[p].fetch_add(1);
      const auto start = clk::now();
      auto fin = [&, p, start](bool ok) {
        const double us = std::chrono::duration<double, std::micro>(clk::now() - start).count();
        {
          std::lock_guard lk(lat_mu);
          lat_us.push_back(us);
        }
        if (!ok) failed.fetch_add(1);
        inflight[p].fetch_sub(1, std::memory_order_release);
      };
      scope.spawn_detached(ex::upon_error(
          ex::then(rt.InvokeRpc(peers[p], session_id_t{1}, function_id_t{1}, workflow_id_t{}, client_policy(rt, o), f32_meta(bytes),
                                UcxBuffer(*mr, type, resident.data(), bytes, nullptr, false)),
                   [fin](InvokeResult r) mutable { fin(r.header.status.ok()); }),
          [fin](std::exception_ptr) mutable { fin(false); }));
    }
    // every window is full: sleep for a moment instead of spinning (with one process per GPU the issuing
    // threads would otherwise take a core each away from the context threads that do the work)
    if (!any) std::this_thread::sleep_for(std::chrono::microseconds(20));
  }
  ex::sync_wait(scope.join());
  const double secs = std::chrono::duration<double>(clk::now() - t0).count();
  write_file(o.dir + "/done." + std::to_string(o.rank), "1");
  // keep serving until every rank has finished its own calls
  wait_for_all(o.dir, "done", o.world, 120);
  const size_t calls = lat_us.size();
  std::printf("mesh rank=%d world=%d memory=%s outstanding_per_peer=%d calls=%zu failed=%d seconds=%.4f calls_per_s=%.0f "
              "payload_GBps=%.3f p50_us=%.1f p99_us=%.1f\n",
              o.rank, o.world, o.cuda ? "cuda" : "host", o.outstanding, calls, failed.load(), secs, calls / secs,
              bytes_total / secs / 1e9, pct(lat_us, 0.5), pct(lat_us, 0.99));
  std::fflush(stdout);
  std::this_thread::sleep_for(50ms);
  rt.Stop();
  return failed.load() ? 1 : 0;
}

int main(int argc, char** argv) {
  Options o;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    auto next = [&] { return i + 1 < argc ? std::string(argv[++i]) : std::string(); };
    if (a == "-m") o.cuda = next() == "cuda";
    else if (a == "-d") o.device = std::stoi(next());
    else if (a == "-n") o.requests = std::stoi(next());
    else if (a == "-o") o.outstanding = std::stoi(next());
    else if (a == "-w") o.warmup = std::stoi(next());
    else if (a == "-s") {
      o.sizes.clear();
      std::string list = next();
      size_t pos = 0;
      while (pos < list.size()) {
        size_t comma = list.find(',', pos);
        if (comma == std::string::npos) comma = list.size();
        o.sizes.push_back(std::stoul(list.substr(pos, comma - pos)) / 4 * 4);
        pos = comma + 1;
      }
    } else if (a == "--mesh") o.mesh = true;
    else if (a == "--rank") o.rank = std::stoi(next());
    else if (a == "--world") o.world = std::stoi(next());
    else if (a == "--dir") o.dir = next();
    else if (a == "--server") o.server = true;
    else if (a == "--client") o.client_addr = next();
    else {
      std::fprintf(stderr, "usage: %s [-m host|cuda] [-d dev] [-s bytes,...] [-n requests] [-o outstanding] [-w warmup] [--server|--client hex]\n", argv[0]);
      return 2;
    }
  }
  using namespace std::chrono_literals;
  try {
    if (o.cuda) cudaSetDevice(o.device);
    if (o.mesh) {
      if (o.dir.empty() || o.world < 2 || o.rank < 0 || o.rank >= o.world) {
        std::fprintf(stderr, "--mesh needs --rank R --world N (N >= 2) --dir DIR\n");
        return 2;
      }
      return run_mesh(o);
    }
    if (o.server) {
      AxonRuntime srv("perf_server", 4, 30000ms, make_dev(o), make_mr(o));
      register_plus_one(srv, o);
      if (auto ec = srv.StartServer()) throw std::runtime_error(ec.message());
      std::cout << "ADDRESS " << to_hex(srv.GetLocalAddress()) << std::endl;
      std::string line;
      while (std::getline(std::cin, line) && line != "quit") {
      }
      srv.Stop();
      return 0;
    }
    if (!o.client_addr.empty()) {
      AxonRuntime cli("perf_client", 4, 30000ms, make_dev(o), make_mr(o));
      if (auto ec = cli.StartClient()) throw std::runtime_error(ec.message());
      cli.ConnectEndpoint(from_hex(o.client_addr), "perf_server");
      int rc = run_client(cli, "perf_server", o);
      cli.Stop();
      return rc;
    }
    AxonRuntime srv("perf_server", 4, 30000ms, make_dev(o), make_mr(o));
    AxonRuntime cli("perf_client", 4, 30000ms, make_dev(o), make_mr(o));
    register_plus_one(srv, o);
    if (auto ec = srv.StartServer()) throw std::runtime_error(ec.message());
    if (auto ec = cli.StartClient()) throw std::runtime_error(ec.message());
    cli.ConnectEndpoint(srv.GetLocalAddress(), "perf_server");
    int rc = run_client(cli, "perf_server", o);
    cli.Stop();
    srv.Stop();
    return rc;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "axon_rpc_perf failed: %s\n", e.what());
    return 1;
  }
}
