// ucx_am_context with device memory on a real GPU: the CUDA forms of the context tests (the reference runs each
// of its context tests with host and with CUDA buffers, ucx_am_context_test.cpp:1377-1945). Two contexts in one
// process on GPU 0. Run by tests/test_native_gpu.py; needs a GPU, so it is not among the CPU test binaries.
#include <cuda_runtime_api.h>

#include <cstdlib>
#include <cstring>
#include <thread>

#include "check.hpp"
#include "eux/exec/async_scope.hpp"
#include "eux/exec/contexts.hpp"
#include "eux/ucxx/cuda/ucx_cuda_context.hpp"
#include "eux/ucxx/cuda/ucx_cuda_memory_manager.hpp"
#include "eux/ucxx/ucx_am_context.hpp"

using namespace eux::ucxx;
namespace ex = eux::exec;
using namespace std::chrono_literals;

namespace {

struct Node {
  UcxCudaMemoryResourceManager mr;
  ucx_am_context ctx;
  ex::inplace_stop_source stop;
  std::thread th;
  explicit Node(const char* name) : mr(options()), ctx(mr, name, 5000ms, true, 0, std::make_unique<UcxAutoCudaDeviceContext>(0)) {
    th = std::thread([this] { ctx.run(stop.get_token()); });
    ex::sync_wait(ctx.get_scheduler().schedule());
  }
  static UcxCudaMemoryResourceManager::Options options() {
    UcxCudaMemoryResourceManager::Options o;
    o.device = 0;
    return o;
  }
  ~Node() {
    stop.request_stop();
    th.join();
  }
};

struct Pair {
  Node srv{"cuda_server"}, cli{"cuda_client"};
  conn_id_t conn = 0;
  Pair() {
    std::vector<std::byte> addr;
    srv.ctx.get_ucp_address(addr);
    auto c = ex::sync_wait(connect_endpoint(cli.ctx.get_scheduler(), addr));
    conn = c ? *c : 0;
  }
};

// environment for the transport of the contexts made while this object lives
struct Env {
  std::vector<std::string> names;
  Env(std::initializer_list<std::pair<const char*, const char*>> kv) {
    for (auto& [k, v] : kv) {
      setenv(k, v, 1);
      names.push_back(k);
    }
  }
  ~Env() {
    for (auto& n : names) unsetenv(n.c_str());
  }
};

std::vector<unsigned char> pattern(size_t n, unsigned seed) {
  std::vector<unsigned char> v(n);
  uint32_t x = seed * 2654435761u + 1;
  for (size_t i = 0; i < n; ++i) {
    x = x * 1664525u + 1013904223u;
    v[i] = static_cast<unsigned char>(x >> 24);
  }
  return v;
}
UcxBuffer device_copy(UcxCudaMemoryResourceManager& mr, const std::vector<unsigned char>& host) {
  UcxBuffer b(mr, ucx_memory_type::CUDA, host.size());
  cudaMemcpy(b.data(), host.data(), host.size(), cudaMemcpyHostToDevice);
  return b;
}
std::vector<unsigned char> to_host(const void* dev, size_t n) {
  std::vector<unsigned char> v(n);
  cudaMemcpy(v.data(), dev, n, cudaMemcpyDeviceToHost);
  return v;
}

// one message client -> server with a device payload, received into device memory; returns what arrived
std::vector<unsigned char> round(Pair& p, UcxBuffer& payload, uint64_t tag, std::shared_ptr<const UcxSendAttr> attr = nullptr) {
  ucx_am_data d{};
  d.header = {&tag, 8};
  d.buffer = {payload.data(), payload.size()};
  d.buffer_type = ucx_memory_type::CUDA;
  if (attr) p.cli.ctx.attach_send_attr(&tag, attr);
  ex::async_scope scope;
  auto rf = scope.spawn_future(connection_recv(p.srv.ctx.get_scheduler(), ucx_memory_type::CUDA));
  const bool sent = ex::sync_wait(connection_send(p.cli.ctx.get_scheduler(), p.conn, d)).has_value();
  auto got = ex::sync_wait(std::move(rf));
  ex::sync_wait(scope.join());
  if (!sent || !got) return {};
  uint64_t seen = 0;
  std::memcpy(&seen, got->get_raw_data().header.data, 8);
  if (seen != tag) return {};
  return to_host(got->get_raw_data().buffer.data, got->get_raw_data().buffer.size);
}

uint16_t bf16_of(float f) {  // round to nearest even, as the kernel's conversion does
  uint32_t u;
  std::memcpy(&u, &f, 4);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

}  // namespace

EUX_TEST(device_payloads_eager_and_pushed) {
  Pair p;
  CHECK(p.conn != 0);
  // 4 KiB: one ring slot, one CTA of a batched launch; 2 MiB: a run of slots, a launch of its own; 24 MiB: pushed
  size_t sizes[] = {4096, 2u << 20, 24u << 20, 4096 + 3};
  for (size_t i = 0; i < 4; ++i) {
    auto host = pattern(sizes[i], unsigned(i));
    UcxBuffer dev = device_copy(p.cli.mr, host);
    CHECK(round(p, dev, 100 + i) == host);
  }
  auto cs = p.cli.ctx.worker().stats(), ss = p.srv.ctx.worker().stats();
  CHECK_EQ(cs.device_eager_sent, uint64_t(3));
  CHECK_EQ(ss.device_eager_recv, uint64_t(3));
  CHECK_EQ(cs.device_pushes, uint64_t(1));
  CHECK_EQ(ss.device_push_recv, uint64_t(1));
  CHECK_EQ(cs.device_staged + ss.device_staged, uint64_t(0));
}

EUX_TEST(device_payloads_pulled_when_neither_eager_nor_pushed) {
  Env env{{"EUX_DEV_EAGER_LIMIT", "65536"}, {"EUX_PUSH_THRESH", "0"}};
  Pair p;
  for (size_t n : {size_t(100) << 10, size_t(16) << 20}) {  // a small pull (batched launch) and a large one
    auto host = pattern(n, unsigned(n));
    UcxBuffer dev = device_copy(p.cli.mr, host);
    CHECK(round(p, dev, n) == host);
  }
  auto ss = p.srv.ctx.worker().stats();
  CHECK_EQ(ss.device_pulls, uint64_t(2));
  CHECK_EQ(ss.device_staged, uint64_t(0));
}

EUX_TEST(device_scatter_gather_send_into_separate_device_buffers) {
  Pair p;
  std::vector<std::vector<unsigned char>> host = {pattern(1000, 1), pattern(3u << 20, 2), pattern(17, 3)};
  std::vector<UcxBuffer> dev;
  for (auto& h : host) dev.push_back(device_copy(p.cli.mr, h));
  ucx_buffer_t iov[3] = {{dev[0].data(), dev[0].size()}, {dev[1].data(), dev[1].size()}, {dev[2].data(), dev[2].size()}};
  uint64_t hdr = 9;
  ucx_am_iovec v{};
  v.header = {&hdr, 8};
  v.buffer_vec = iov;
  v.buffer_count = 3;
  v.buffer_type = ucx_memory_type::CUDA;
  ex::async_scope scope;
  auto hf = scope.spawn_future(connection_recv_header(p.srv.ctx.get_scheduler()));
  auto sf = scope.spawn_future(connection_send(p.cli.ctx.get_scheduler(), p.conn, v));
  auto h = ex::sync_wait(std::move(hf));
  CHECK(h.has_value() && h->index() == 0);
  UcxBufferVec dst(p.srv.mr, ucx_memory_type::CUDA, std::vector<size_t>{host[0].size(), host[1].size(), host[2].size()});
  auto b = ex::sync_wait(connection_recv_buffer(p.srv.ctx.get_scheduler(), std::get<0>(*h).first, std::move(dst)));
  CHECK(b.has_value());
  CHECK(ex::sync_wait(std::move(sf)).has_value());
  ex::sync_wait(scope.join());
  for (int i = 0; i < 3; ++i) CHECK(to_host(b->buffer()[i].data, host[i].size()) == host[i]);
  CHECK_EQ(p.srv.ctx.worker().stats().device_staged, uint64_t(0));
}

EUX_TEST(device_payload_received_into_host_memory_is_staged_and_counted) {
  Env env{{"EUX_DEV_EAGER_LIMIT", "0"}};
  Pair p;
  auto host = pattern(1u << 20, 5);
  UcxBuffer dev = device_copy(p.cli.mr, host);
  uint64_t tag = 5;
  ucx_am_data d{};
  d.header = {&tag, 8};
  d.buffer = {dev.data(), dev.size()};
  d.buffer_type = ucx_memory_type::CUDA;
  ex::async_scope scope;
  auto rf = scope.spawn_future(connection_recv(p.srv.ctx.get_scheduler(), ucx_memory_type::HOST));
  CHECK(ex::sync_wait(connection_send(p.cli.ctx.get_scheduler(), p.conn, d)).has_value());
  auto got = ex::sync_wait(std::move(rf));
  ex::sync_wait(scope.join());
  CHECK(got.has_value());
  CHECK(std::memcmp(got->get_raw_data().buffer.data, host.data(), host.size()) == 0);
}

EUX_TEST(strided_and_converted_payloads_are_gathered_on_the_way) {
  Pair p;
  const int64_t rows = 300, cols = 70;  // the matrix lies row-major as rows x cols; its transpose is sent
  std::vector<float> m(size_t(rows * cols));
  for (size_t i = 0; i < m.size(); ++i) m[i] = float(i) * 0.25f - 1000.0f;
  std::vector<unsigned char> raw(m.size() * 4);
  std::memcpy(raw.data(), m.data(), raw.size());
  UcxBuffer dev = device_copy(p.cli.mr, raw);
  auto attr = std::make_shared<UcxSendAttr>();
  attr->ndim = 2;
  attr->elem_size = 4;
  attr->shape[0] = cols, attr->shape[1] = rows;
  attr->stride[0] = 1, attr->stride[1] = cols;
  attr->span_bytes = raw.size();
  attr->dense_bytes = raw.size();
  auto got = round(p, dev, 1, attr);  // 82 KiB: gathered into the ring slot
  CHECK_EQ(got.size(), raw.size());
  const float* g = reinterpret_cast<const float*>(got.data());
  bool same = got.size() == raw.size();
  for (int64_t c = 0; same && c < cols; ++c)
    for (int64_t r = 0; same && r < rows; ++r) same = g[c * rows + r] == m[size_t(r * cols + c)];
  CHECK(same);
  // the same view, converted to bf16 on the way: half the bytes arrive
  auto cast = std::make_shared<UcxSendAttr>(*attr);
  cast->src_dtype = 1;
  cast->dst_dtype = 3;
  cast->dense_bytes = raw.size() / 2;
  UcxBuffer half_view(p.cli.mr, ucx_memory_type::CUDA, dev.data(), raw.size() / 2, nullptr, false);  // the message's size is the converted one
  auto got16 = round(p, half_view, 2, cast);
  CHECK_EQ(got16.size(), raw.size() / 2);
  const uint16_t* h = reinterpret_cast<const uint16_t*>(got16.data());
  same = got16.size() == raw.size() / 2;
  for (int64_t c = 0; same && c < cols; ++c)
    for (int64_t r = 0; same && r < rows; ++r) same = h[c * rows + r] == bf16_of(m[size_t(r * cols + c)]);
  CHECK(same);
  CHECK_EQ(p.cli.ctx.worker().stats().device_gathers, uint64_t(2));
  CHECK_EQ(p.cli.ctx.worker().stats().device_packs, uint64_t(0));
  // a layout that reaches outside its span is refused at the sender, before any kernel sees it
  auto bad = std::make_shared<UcxSendAttr>(*attr);
  bad->stride[1] = cols + 1;
  ucx_am_data d{};
  uint64_t tag = 3;
  d.header = {&tag, 8};
  d.buffer = {dev.data(), dev.size()};
  d.buffer_type = ucx_memory_type::CUDA;
  p.cli.ctx.attach_send_attr(&tag, bad);
  CHECK_THROWS(ex::sync_wait(connection_send(p.cli.ctx.get_scheduler(), p.conn, d)));
}

EUX_TEST(a_payload_whose_producer_is_still_running_is_sent_when_it_is_done) {
  Pair p;
  cudaStream_t st;
  CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) == cudaSuccess);
  for (size_t n : {size_t(8) << 10, size_t(8) << 20}) {  // a small and a large one: either is announced once its producer is done
    UcxBuffer dev(p.cli.mr, ucx_memory_type::CUDA, n);
    cudaMemset(dev.data(), 0, n);
    cudaDeviceSynchronize();
    // the producer: 60 ms of nothing (a host function holds the stream), then the bytes
    cudaLaunchHostFunc(st, [](void*) { std::this_thread::sleep_for(60ms); }, nullptr);
    cudaMemsetAsync(dev.data(), 0x5b, n, st);
    cudaEvent_t ev;
    cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    cudaEventRecord(ev, st);
    auto attr = std::make_shared<UcxSendAttr>();
    attr->ready_event = ev;
    attr->device = 0;
    attr->keep = std::shared_ptr<void>(ev, [](void* e) { cudaEventDestroy(static_cast<cudaEvent_t>(e)); });
    const auto t0 = std::chrono::steady_clock::now();
    auto got = round(p, dev, n, attr);
    CHECK(std::chrono::steady_clock::now() - t0 >= 55ms);
    CHECK_EQ(got.size(), n);
    bool all = !got.empty();
    for (unsigned char c : got) all = all && c == 0x5b;
    CHECK(all);
  }
  CHECK(p.cli.ctx.worker().stats().sends_held >= 1);
  cudaStreamDestroy(st);
}

EUX_TEST(a_device_transfer_in_flight_is_not_torn_by_a_stop_request) {
  // A pull that has been launched cannot be withdrawn (a kernel is writing the buffer): the operation either
  // was stopped before the launch, or completes with the whole payload. Either way the next message works.
  Env env{{"EUX_DEV_EAGER_LIMIT", "65536"}, {"EUX_PUSH_THRESH", "0"}};
  Pair p;
  auto host = pattern(size_t(64) << 20, 77);
  UcxBuffer dev = device_copy(p.cli.mr, host);
  uint64_t tag = 1;
  ucx_am_data d{};
  d.header = {&tag, 8};
  d.buffer = {dev.data(), dev.size()};
  d.buffer_type = ucx_memory_type::CUDA;
  ex::async_scope scope;
  ex::timed_single_thread_context timer;
  scope.spawn_detached(ex::upon_error(ex::upon_done(connection_send(p.cli.ctx.get_scheduler(), p.conn, d), [] {}), [](std::exception_ptr) {}));
  auto h = ex::sync_wait(connection_recv_header(p.srv.ctx.get_scheduler()));
  CHECK(h.has_value() && h->index() == 0);
  auto r = ex::sync_wait(ex::stop_when(connection_recv_buffer(p.srv.ctx.get_scheduler(), std::get<0>(*h).first, ucx_memory_type::CUDA),
                                       ex::schedule_after(timer.get_scheduler(), 20us)));
  if (r.has_value()) CHECK(to_host(r->buffer().data(), host.size()) == host);
  scope.request_stop();
  ex::sync_wait(scope.join());
  auto again = pattern(4096, 3);
  UcxBuffer small = device_copy(p.cli.mr, again);
  CHECK(round(p, small, 2) == again);
}

EUX_TEST_MAIN()
