// RPC storm: latency and throughput of Axon RPCs that carry one fp32 tensor and get it back
// with 1.0 added (the counterpart of the reference's axon/benchmark/axon_benchmark.cpp), for
// host and for device payloads.
//
//   eux_axon_rpc_perf [-m host|cuda] [-d device] [-s bytes[,bytes...]] [-n requests] [-o outstanding]
//                     [-w warmup] [--server | --client <address-hex>]
//
// Without --server/--client both runtimes live in this process. For every size it prints the
// round-trip latency with one request in flight (p50 / p99) and the request rate and payload
// bandwidth with `outstanding` requests in flight. Device payloads stay on the device: the
// receiver pulls them with the transfer kernel and the handler adds 1.0 with the same kernel.
#include <algorithm>
#include <atomic>
#include <chrono>
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
  return std::make_shared<eux::ucxx::UcxCudaMemoryResourceManager>(mo);
}

static std::unique_ptr<eux::ucxx::UcxAutoDeviceContext> make_dev(const Options& o) {
  if (!o.cuda) return nullptr;
  return std::make_unique<eux::ucxx::UcxAutoCudaDeviceContext>(o.device);
}

// y = x + 1 on the device, on a stream of the calling thread
static void device_plus_one(const void* x, void* y, size_t bytes, int device) {
  thread_local cudaStream_t st = nullptr;
  thread_local uint32_t* counter = nullptr;
  if (!st) {
    cudaSetDevice(device);
    cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
    cudaMalloc(reinterpret_cast<void**>(&counter), 256);
    cudaMemsetAsync(counter, 0, 256, st);
  }
  eux_xfer_desc d{};
  d.src = x;
  d.dst = y;
  d.n_elems = bytes / 4;
  d.src_dtype = d.dst_dtype = EUX_DT_F32;
  d.op = EUX_OP_ADD;
  d.op_arg = 1.0f;
  int rc = eux_xfer_launch(&d, counter, 0, st);
  if (rc != 0) throw std::runtime_error(std::string("handler kernel: ") + eux_error_string(rc));
  cudaStreamSynchronize(st);
}

static void register_plus_one(AxonRuntime& rt, const Options& o) {
  auto mr = rt.memory_resource();
  const bool cuda = o.cuda;
  const int dev = o.device;
  auto handler = [mr, cuda, dev](const TensorMeta& m, UcxBuffer& buf) {
    UcxBuffer out(*mr, buf.type(), buf.size());
    if (cuda) {
      device_plus_one(buf.data(), out.data(), buf.size(), dev);
    } else {
      const float* f = static_cast<const float*>(buf.data());
      float* g = static_cast<float*>(out.data());
      for (int64_t i = 0; i < m.shape[0]; ++i) g[i] = f[i] + 1.0f;
    }
    return std::tuple<TensorMeta, UcxBuffer>(m, std::move(out));
  };
  if (cuda) {
    CustomMemoryPolicy<UcxBuffer> provider = [mr](eux::rpc::utils::TensorMetaSpan metas) {
      return UcxBuffer(*mr, ucx_memory_type::CUDA, eux::rpc::utils::CalculateTensorSize(metas[0]));
    };
    rt.worker().RegisterFunction<UcxBuffer>(function_id_t{1}, handler, "plus_one", provider, MessageLifecyclePolicy{});
  } else {
    rt.RegisterFunction(function_id_t{1}, handler, "plus_one");
  }
}

static ClientMemoryPolicy client_policy(AxonRuntime& rt, const Options& o) {
  ClientMemoryPolicy p;
  if (o.cuda) {
    auto mr = rt.memory_resource();
    p.on_host = false;
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
    } else if (a == "--server") o.server = true;
    else if (a == "--client") o.client_addr = next();
    else {
      std::fprintf(stderr, "usage: %s [-m host|cuda] [-d dev] [-s bytes,...] [-n requests] [-o outstanding] [-w warmup] [--server|--client hex]\n", argv[0]);
      return 2;
    }
  }
  using namespace std::chrono_literals;
  try {
    if (o.cuda) cudaSetDevice(o.device);
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
