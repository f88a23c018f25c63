// AxonWorker end to end: two workers over loopback in one process, and a
// client/server pair in forked processes (address through a pipe).
#include <sys/wait.h>
#include <unistd.h>

#include <cstring>
#include <mutex>
#include <numeric>
#include <set>
#include <thread>

#include "check.hpp"
#include "eux/ucxx/transport.hpp"
#include "eux/axon/axon_runtime.hpp"

using namespace eux::axon;
using namespace eux::rpc;
using eux::ucxx::DefaultUcxMemoryResourceManager;
using eux::ucxx::UcxBuffer;
using eux::ucxx::UcxBufferVec;
namespace ex = eux::exec;
namespace autils = eux::axon::utils;
using namespace std::chrono_literals;

static TensorMeta f32_meta(int64_t n) {
  TensorMeta m;
  m.ndim = 1;
  m.dtype = {kDLFloat, 32, 1};
  m.shape = {n};
  m.strides = {1};
  return m;
}

struct Pair {
  std::shared_ptr<DefaultUcxMemoryResourceManager> mr = std::make_shared<DefaultUcxMemoryResourceManager>();
  AxonWorker server{mr, "server", 4, 2000ms};
  AxonWorker client{mr, "client", 2, 2000ms};
  void connect() {
    CHECK(!server.StartServer());
    CHECK(!client.StartClient());
    client.ConnectEndpoint(server.GetLocalAddress(), "server");
    auto sigs = server.GetLocalSignatures();
    CHECK(client.RegisterEndpointSignatures("server", sigs.data(), sigs.size()));
  }
};

EUX_TEST(hash_contract) {
  // same inputs, same ids on both ends; different names, different ids
  uint32_t a = autils::FunctionIdFromName("echo", "server"), b = autils::FunctionIdFromName("echo", "server");
  CHECK_EQ(a, b);
  CHECK(a != autils::FunctionIdFromName("echo", "other"));
  CHECK(a != autils::FunctionIdFromName("echp", "server"));
  CHECK(autils::StringHash("abc") == autils::DataHash("abc", 3));
  CHECK(!(autils::StringHash("abc") == autils::StringHash("abd")));
}

EUX_TEST(ring_buffer_and_slot_map) {
  autils::RingBuffer<int, 8> rb;
  CHECK(rb.emplace(3, 30));
  CHECK(!rb.emplace(11, 110));  // 11 & 7 == 3: slot taken
  CHECK(!rb.take(11).has_value());
  CHECK(!rb.take_if(3, [](int v) { return v == 0; }).has_value());
  CHECK_EQ(*rb.take(3), 30);
  CHECK(rb.emplace(11, 110));
  CHECK_EQ(rb.size(), 1u);
  autils::SlotMap<std::string> sm;
  auto k1 = sm.insert("one");
  CHECK(*sm.find(k1) == "one");
  CHECK(sm.erase(k1));
  auto k2 = sm.insert("two");
  CHECK_EQ(k2.index, k1.index);
  CHECK(sm.find(k1) == nullptr);  // stale generation
  CHECK(*sm.find(k2) == "two");
}

EUX_TEST(echo_primitives_and_small_tensor) {
  Pair p;
  p.server.RegisterFunction(function_id_t{1}, [](int32_t a, int32_t b) { return a + b; }, "add");
  p.server.RegisterFunction(function_id_t{2}, [](const TensorMeta& m, UcxBuffer& buf) {
    float* f = static_cast<float*>(buf.data());
    for (int64_t i = 0; i < m.shape[0]; ++i) f[i] += 1.0f;
    UcxBuffer out(buf.mr(), buf.type(), buf.size());
    std::memcpy(out.data(), buf.data(), buf.size());
    return std::tuple<TensorMeta, UcxBuffer>(m, std::move(out));
  }, "plus_one");
  p.connect();
  auto r = ex::sync_wait(p.client.InvokeRpc("server", session_id_t{1}, function_id_t{1}, workflow_id_t{5}, ClientMemoryPolicy{}, int32_t(2), int32_t(40)));
  CHECK(r.has_value());
  CHECK(r->header.status.ok());
  CHECK_EQ(r->header.GetPrimitive<int32_t>(0), 42);
  CHECK_EQ(r->header.workflow_id.v_, 5u);
  CHECK(r->header.hlc.Raw() > 0);
  // eager tensor (256 floats) and rendezvous tensor (64 Ki floats)
  for (int64_t n : {int64_t(256), int64_t(65536)}) {
    UcxBuffer buf(*p.mr, ucx_memory_type::HOST, size_t(n) * 4);
    float* f = static_cast<float*>(buf.data());
    for (int64_t i = 0; i < n; ++i) f[i] = float(i);
    auto t = ex::sync_wait(p.client.InvokeRpc("server", session_id_t{1}, function_id_t{2}, workflow_id_t{}, ClientMemoryPolicy{}, f32_meta(n), std::move(buf)));
    CHECK(t.has_value() && t->header.status.ok());
    auto& out = std::get<UcxBuffer>(t->payload);
    CHECK_EQ(out.size(), size_t(n) * 4);
    const float* g = static_cast<const float*>(out.data());
    for (int64_t i = 0; i < n; i += 37) CHECK_EQ(g[i], float(i) + 1.0f);
    CHECK(t->header.GetTensor(0).shape[0] == n);
  }
  // the signature the client learned from the server
  auto sig = p.client.GetEndpointSignature("server", function_id_t{2});
  CHECK(sig && sig->function_name == "plus_one" && sig->input_payload_type == PayloadType::UCX_BUFFER);
}

EUX_TEST(errors_deadline_and_unknown_worker) {
  Pair p;
  p.server.RegisterFunction(function_id_t{1}, [](int32_t) -> int32_t { throw RpcException(RpcErrc::FAILED_PRECONDITION, "not today"); }, "fail");
  p.server.RegisterFunction(function_id_t{2}, [](int32_t ms) {
    std::this_thread::sleep_for(std::chrono::milliseconds(ms));
    return ms;
  }, "sleep");
  p.connect();
  auto r = ex::sync_wait(p.client.InvokeRpc("server", session_id_t{1}, function_id_t{1}, workflow_id_t{}, ClientMemoryPolicy{}, int32_t(1)));
  CHECK(r && r->header.status.value == int(RpcErrc::FAILED_PRECONDITION));
  CHECK(r->header.GetString(0) == "not today");
  auto nf = ex::sync_wait(p.client.InvokeRpc("server", session_id_t{1}, function_id_t{77}, workflow_id_t{}, ClientMemoryPolicy{}));
  CHECK(nf && nf->header.status.value == int(RpcErrc::NOT_FOUND));
  CHECK_THROWS(ex::sync_wait(p.client.InvokeRpc("nobody", session_id_t{1}, function_id_t{1}, workflow_id_t{}, ClientMemoryPolicy{})));
  // client deadline
  p.client.SetTimeout(50ms);
  auto t0 = std::chrono::steady_clock::now();
  bool deadline = false;
  try {
    ex::sync_wait(p.client.InvokeRpc("server", session_id_t{1}, function_id_t{2}, workflow_id_t{}, ClientMemoryPolicy{}, int32_t(400)));
  } catch (const RpcException& e) {
    deadline = e.code() == make_error_code(RpcErrc::DEADLINE_EXCEEDED);
  }
  CHECK(deadline);
  CHECK(std::chrono::steady_clock::now() - t0 < 350ms);
  CHECK_EQ(p.client.PendingRpcCount(), 0u);
  // server deadline: the handler overruns, the caller gets DEADLINE_EXCEEDED from the server
  p.client.SetTimeout(3000ms);
  p.server.SetTimeout(50ms);
  auto sd = ex::sync_wait(p.client.InvokeRpc("server", session_id_t{1}, function_id_t{2}, workflow_id_t{}, ClientMemoryPolicy{}, int32_t(300)));
  CHECK(sd && sd->header.status.value == int(RpcErrc::DEADLINE_EXCEEDED));
  std::this_thread::sleep_for(350ms);  // let the overrunning handler end before the workers go away
}

// A header image larger than a message may carry is refused where it is made: the caller of an oversize request
// gets the error at once, the caller of a function with oversize results gets it as the response, and the
// connection serves the next call (the receiving side would have closed it over such a frame).
EUX_TEST(oversize_headers_end_as_errors_and_the_connection_stays) {
  Pair p;
  p.server.RegisterFunction(function_id_t{1}, [](int32_t n) -> data::string {
    const std::string text(static_cast<size_t>(n), 'x');
    return data::string(text);
  }, "text");
  p.server.RegisterFunction(function_id_t{2}, [](const data::string& s) { return int64_t(s.size()); }, "length");
  p.server.RegisterFunction(function_id_t{3}, [](int32_t n) {
    data::vector<int64_t> squares;
    for (int32_t i = 0; i < n; ++i) squares.push_back(int64_t(i) * i);
    return squares;
  }, "squares");
  p.connect();
  const int32_t too_much = int32_t(eux::ucxx::transport::kMaxHeaderLen + 100);
  auto ok = ex::sync_wait(p.client.InvokeRpc("server", session_id_t{1}, function_id_t{1}, workflow_id_t{}, ClientMemoryPolicy{}, int32_t(1 << 20)));
  CHECK(ok && ok->header.status.ok() && ok->header.GetString(0).size() == size_t(1 << 20));
  auto t0 = std::chrono::steady_clock::now();
  auto big = ex::sync_wait(p.client.InvokeRpc("server", session_id_t{1}, function_id_t{1}, workflow_id_t{}, ClientMemoryPolicy{}, too_much));
  CHECK(big && big->header.status.value == int(RpcErrc::RESOURCE_EXHAUSTED));
  CHECK(std::chrono::steady_clock::now() - t0 < 1500ms);  // an answer, not the caller's deadline
  bool refused = false;
  const std::string oversize(static_cast<size_t>(too_much), 'y');
  try {
    ex::sync_wait(p.client.InvokeRpc("server", session_id_t{1}, function_id_t{2}, workflow_id_t{}, ClientMemoryPolicy{}, data::string(oversize)));
  } catch (const RpcException& e) {
    refused = e.code() == make_error_code(RpcErrc::RESOURCE_EXHAUSTED);
  }
  CHECK(refused);
  auto after = ex::sync_wait(p.client.InvokeRpc("server", session_id_t{1}, function_id_t{2}, workflow_id_t{}, ClientMemoryPolicy{}, data::string("four")));
  CHECK(after && after->header.status.ok() && after->header.GetPrimitive<int64_t>(0) == 4);
  // (a function may return one of the wire's containers by itself: they are values, not senders)
  auto sq = ex::sync_wait(p.client.InvokeRpc("server", session_id_t{1}, function_id_t{3}, workflow_id_t{}, ClientMemoryPolicy{}, int32_t(4)));
  CHECK(sq && sq->header.status.ok() && (sq->header.GetVector<int64_t>(0) == data::vector<int64_t>{0, 1, 4, 9}));
}

EUX_TEST(concurrent_calls_and_buffer_vec) {
  Pair p;
  p.server.RegisterFunction(function_id_t{1}, [](int32_t a) { return a * 2; }, "dbl");
  p.server.RegisterFunction(function_id_t{3}, [](const TensorMetaVec& metas, UcxBufferVec& bufs) {
    int64_t total = 0;
    for (size_t i = 0; i < bufs.size(); ++i) {
      const float* f = static_cast<const float*>(bufs[i].data);
      for (int64_t k = 0; k < metas[i].shape[0]; ++k) total += int64_t(f[k]);
    }
    return total;
  }, "sum_all");
  p.connect();
  // 64 calls in flight at once
  ex::async_scope scope;
  std::atomic<int> ok{0};
  for (int i = 0; i < 64; ++i) {
    scope.spawn_detached(ex::upon_error(ex::then(p.client.InvokeRpc("server", session_id_t{9}, function_id_t{1}, workflow_id_t{}, ClientMemoryPolicy{}, int32_t(i)),
                                                 [&ok, i](InvokeResult r) {
                                                   if (r.header.status.ok() && r.header.GetPrimitive<int32_t>(0) == 2 * i) ok.fetch_add(1);
                                                 }),
                                        [](std::exception_ptr) {}));
  }
  ex::sync_wait(scope.join());
  CHECK_EQ(ok.load(), 64);
  // three tensors as one scatter-gather payload
  TensorMetaVec metas{f32_meta(10), f32_meta(5000), f32_meta(3)};
  UcxBufferVec bufs(*p.mr, ucx_memory_type::HOST, std::vector<size_t>{40, 20000, 12});
  int64_t want = 0;
  for (size_t i = 0; i < 3; ++i) {
    float* f = static_cast<float*>(bufs[i].data);
    for (int64_t k = 0; k < metas[i].shape[0]; ++k) {
      f[k] = float(k % 7);
      want += k % 7;
    }
  }
  auto r = ex::sync_wait(p.client.InvokeRpc("server", session_id_t{9}, function_id_t{3}, workflow_id_t{}, ClientMemoryPolicy{}, metas, std::move(bufs)));
  CHECK(r && r->header.status.ok());
  CHECK_EQ(r->header.GetPrimitive<int64_t>(0), want);
}

EUX_TEST(memory_policy_backpressure_and_retention) {
  // written by the retention policy on the server's context thread; declared before the workers so that
  // they outlive those threads
  std::mutex ids_mu;
  std::vector<uint64_t> retained_ids;
  Pair p;
  std::atomic<int> provider_calls{0};
  // the server chooses the receive buffer itself for large payloads
  CustomMemoryPolicy<UcxBuffer> provider = [&](eux::rpc::utils::TensorMetaSpan metas) {
    provider_calls.fetch_add(1);
    return UcxBuffer(*p.mr, ucx_memory_type::HOST, eux::rpc::utils::CalculateTensorSize(metas[0]));
  };
  RetentionPolicy keep = [&](std::shared_ptr<autils::AxonRequest> req, autils::AxonMessageID id) {
    {
      std::lock_guard lk(ids_mu);
      retained_ids.push_back(id);
    }
    return req->header.GetTensor(0).shape[0] > 100000 ? LifecycleStatus::Preserve : LifecycleStatus::Discard;
  };
  std::atomic<int> handled{0};
  p.server.RegisterFunction<UcxBuffer>(function_id_t{1}, [&](const TensorMeta& m, const UcxBuffer& b) {
    handled.fetch_add(1);
    return int64_t(b.size());
  }, "sink", provider, keep);
  p.server.RegisterFunction(function_id_t{2}, [] { return int32_t(1); }, "control");
  p.connect();
  auto call = [&](int64_t n) {
    UcxBuffer buf(*p.mr, ucx_memory_type::HOST, size_t(n) * 4);
    std::memset(buf.data(), 1, buf.size());
    return ex::sync_wait(p.client.InvokeRpc("server", session_id_t{1}, function_id_t{1}, workflow_id_t{}, ClientMemoryPolicy{}, f32_meta(n), std::move(buf)));
  };
  auto small = call(16);  // eager: the provider is not consulted
  CHECK(small && small->header.GetPrimitive<int64_t>(0) == 64);
  CHECK_EQ(provider_calls.load(), 0);
  auto big = call(200000);  // rendezvous: provider picks the buffer, retention keeps the request
  CHECK(big && big->header.GetPrimitive<int64_t>(0) == 800000);
  CHECK_EQ(provider_calls.load(), 1);
  CHECK_EQ(p.server.GetStorage().size(), 1u);
  {
    std::lock_guard lk(ids_mu);
    CHECK_EQ(retained_ids.size(), 2u);
  }
  // stored requests can be run again and checkpointed
  CHECK_EQ(p.server.ProcessStoredRequests(), 1u);
  CHECK_EQ(handled.load(), 3);
  char dir[] = "/tmp/eux_axon_XXXXXX";
  CHECK(mkdtemp(dir) != nullptr);
  std::string path = p.server.GetStorage().save(*p.mr, dir, "ckpt");
  eux::axon::storage::AxonStorage restored;
  CHECK_EQ(restored.load(*p.mr, path), 1u);
  auto snap = restored.snapshot();
  CHECK_EQ(std::get<UcxBuffer>(snap[0].second->payload).size(), 800000u);
  CHECK(snap[0].second->header.GetTensor(0).shape[0] == 200000);
  unlink(path.c_str());
  rmdir(dir);
  CHECK_EQ(p.server.ProcessStoredRequests([](auto, auto) { return LifecycleStatus::Discard; }), 1u);
  CHECK_EQ(p.server.GetStorage().size(), 0u);
  // back-pressure with a bypass for the control function
  p.server.SetRejectMessages(true);
  p.server.SetBypassRejectionFunction([](const RpcRequestHeader& h) { return h.function_id.v_ == 2; });
  auto rejected = call(16);
  CHECK(rejected && !rejected->header.status.ok());
  CHECK(std::string(rejected->header.status.category_name) == "AxonErrc");
  CHECK_EQ(rejected->header.status.value, int(errors::AxonErrc::StorageBackpressure));
  auto ctl = ex::sync_wait(p.client.InvokeRpc("server", session_id_t{1}, function_id_t{2}, workflow_id_t{}, ClientMemoryPolicy{}));
  CHECK(ctl && ctl->header.status.ok());
  p.server.SetRejectMessages(false);
  CHECK(call(16)->header.status.ok());
}

EUX_TEST(inline_buffer_providers_run_on_the_context_threads) {
  // provider_inline: the providers are called by the server's and the client's context threads, never by a
  // pool thread (handlers run on the pool, so a handler's thread id tells the two apart), and the payload
  // still arrives in the buffers they returned.
  Pair p;
  std::mutex mu;
  std::set<std::thread::id> provider_threads, handler_threads;
  void* server_buffer = nullptr;
  eux::axon::ServerMemoryPolicy smp;
  smp.on_host = false;
  smp.provider_inline = true;
  smp.buffer_provider = [&](eux::rpc::utils::TensorMetaSpan metas) {
    UcxBuffer b(*p.mr, ucx_memory_type::HOST, eux::rpc::utils::CalculateTensorSize(metas[0]));
    std::lock_guard lk(mu);
    provider_threads.insert(std::this_thread::get_id());
    server_buffer = b.data();
    return b;
  };
  p.server.RegisterFunction(function_id_t{1}, [&](const TensorMeta& m, UcxBuffer& b) {
    {
      std::lock_guard lk(mu);
      handler_threads.insert(std::this_thread::get_id());
      CHECK(b.data() == server_buffer);
    }
    UcxBuffer out(*p.mr, ucx_memory_type::HOST, b.size());
    const float* f = static_cast<const float*>(b.data());
    float* g = static_cast<float*>(out.data());
    for (int64_t i = 0; i < m.shape[0]; ++i) g[i] = f[i] + 1.0f;
    return std::tuple<TensorMeta, UcxBuffer>(m, std::move(out));
  }, "plus_one", std::move(smp));
  p.connect();
  void* client_buffer = nullptr;
  ClientMemoryPolicy cmp;
  cmp.on_host = false;
  cmp.provider_inline = true;
  cmp.buffer_provider = [&](eux::rpc::utils::TensorMetaSpan metas) {
    UcxBuffer b(*p.mr, ucx_memory_type::HOST, eux::rpc::utils::CalculateTensorSize(metas[0]));
    std::lock_guard lk(mu);
    provider_threads.insert(std::this_thread::get_id());
    client_buffer = b.data();
    return b;
  };
  const int64_t n = 200000;  // rendezvous both ways
  for (int round = 0; round < 3; ++round) {
    UcxBuffer buf(*p.mr, ucx_memory_type::HOST, size_t(n) * 4);
    float* f = static_cast<float*>(buf.data());
    for (int64_t i = 0; i < n; ++i) f[i] = float(i % 977) + float(round);
    auto r = ex::sync_wait(p.client.InvokeRpc("server", session_id_t{1}, function_id_t{1}, workflow_id_t{}, cmp, f32_meta(n), std::move(buf)));
    CHECK(r && r->header.status.ok());
    const auto& out = std::get<UcxBuffer>(r->payload);
    CHECK(out.data() == client_buffer);
    const float* g = static_cast<const float*>(out.data());
    bool same = true;
    for (int64_t i = 0; i < n; ++i) same = same && g[i] == float(i % 977) + float(round) + 1.0f;
    CHECK(same);
  }
  std::lock_guard lk(mu);
  CHECK_EQ(provider_threads.size(), 2u);  // one context thread on each side
  for (auto id : handler_threads) CHECK(provider_threads.count(id) == 0);
}

EUX_TEST(inline_handlers_start_on_the_server_context_thread) {
  // handler_inline: a handler that only starts asynchronous work is called on the server's context thread
  // (the thread that also runs an inline buffer provider); without the flag it is called on a pool thread.
  // Either way its sender may finish elsewhere, here on the pool, and the reply is the same.
  ex::static_thread_pool elsewhere(1);  // made first, gone last: the workers' threads submit to it until they stop
  Pair p;
  std::mutex mu;
  std::thread::id inline_started, pooled_started, provider_thread;
  auto make_handler = [&](std::thread::id& started) {
    return [&, pstarted = &started](const TensorMeta& m, const UcxBuffer& b) {
      {
        std::lock_guard lk(mu);
        *pstarted = std::this_thread::get_id();
      }
      const int64_t n = m.shape[0];
      const float first = static_cast<const float*>(b.data())[0];
      return ex::on(elsewhere.get_scheduler(), ex::just_from([n, first] { return std::tuple<int64_t, float>(n, first + 1.0f); }));
    };
  };
  auto provider = [&](eux::rpc::utils::TensorMetaSpan metas) {
    std::lock_guard lk(mu);
    provider_thread = std::this_thread::get_id();
    return UcxBuffer(*p.mr, ucx_memory_type::HOST, eux::rpc::utils::CalculateTensorSize(metas[0]));
  };
  eux::axon::ServerMemoryPolicy on_loop;
  on_loop.on_host = false;
  on_loop.provider_inline = true;
  on_loop.handler_inline = true;
  on_loop.buffer_provider = provider;
  eux::axon::ServerMemoryPolicy on_pool = on_loop;
  on_pool.handler_inline = false;
  p.server.RegisterFunction(function_id_t{1}, make_handler(inline_started), "inline", std::move(on_loop));
  p.server.RegisterFunction(function_id_t{2}, make_handler(pooled_started), "pooled", std::move(on_pool));
  p.connect();
  const int64_t n = 100000;  // rendezvous, so the provider runs
  for (uint32_t fid : {1u, 2u}) {
    UcxBuffer buf(*p.mr, ucx_memory_type::HOST, size_t(n) * 4);
    static_cast<float*>(buf.data())[0] = 41.0f;
    auto r = ex::sync_wait(p.client.InvokeRpc("server", session_id_t{1}, function_id_t{fid}, workflow_id_t{}, ClientMemoryPolicy{}, f32_meta(n), std::move(buf)));
    CHECK(r && r->header.status.ok());
    CHECK_EQ(r->header.GetPrimitive<int64_t>(0), n);
    CHECK_EQ(r->header.GetPrimitive<float>(1), 42.0f);
  }
  std::lock_guard lk(mu);
  CHECK(provider_thread != std::thread::id{});
  CHECK(inline_started == provider_thread);
  CHECK(pooled_started != provider_thread && pooled_started != std::thread::id{});
}

EUX_TEST(stop_client_cancels_pending_and_peer_loss_is_an_error) {
  auto p = std::make_unique<Pair>();
  p->server.RegisterFunction(function_id_t{1}, [](int32_t ms) {
    std::this_thread::sleep_for(std::chrono::milliseconds(ms));
    return ms;
  }, "sleep");
  p->connect();
  p->client.SetTimeout(5000ms);
  ex::async_scope scope;
  std::atomic<int> cancelled{0};
  scope.spawn_detached(ex::upon_error(ex::then(p->client.InvokeRpc("server", session_id_t{1}, function_id_t{1}, workflow_id_t{}, ClientMemoryPolicy{}, int32_t(300)),
                                               [](InvokeResult) {}),
                                      [&](std::exception_ptr e) {
                                        if (ex::error_code_of(e) == make_error_code(RpcErrc::CANCELLED)) cancelled.fetch_add(1);
                                      }));
  std::this_thread::sleep_for(30ms);
  p->client.StopClient();
  ex::sync_wait(scope.join());
  CHECK_EQ(cancelled.load(), 1);
  std::this_thread::sleep_for(350ms);
  p.reset();
}

// Server and client in separate processes; the address travels through a pipe.
// Stop and start again: the same workers serve new connections after a restart of either side.
EUX_TEST(client_and_server_restart) {
  Pair p;
  p.server.RegisterFunction(function_id_t{1}, [](int32_t a) { return a + 1; }, "inc");
  p.connect();
  auto call = [&] {
    auto r = ex::sync_wait(p.client.InvokeRpc("server", session_id_t{1}, function_id_t{1}, workflow_id_t{}, ClientMemoryPolicy{}, int32_t(1)));
    return r && r->header.status.ok() && r->header.GetPrimitive<int32_t>(0) == 2;
  };
  CHECK(call());
  p.client.StopClient();
  CHECK(!p.client.StartClient());
  p.client.ConnectEndpoint(p.server.GetLocalAddress(), "server");
  CHECK(call());
  p.server.StopServer();
  CHECK(!p.server.StartServer());
  p.client.DisconnectEndpoint("server");
  p.client.ConnectEndpoint(p.server.GetLocalAddress(), "server");
  CHECK(call());
}

// Fault injection on the host: a response frame lost on the wire, a rendezvous reply lost, and
// a memory policy that cannot allocate. Each ends as an error at the caller within its deadline;
// nothing hangs, and the same workers serve the next call.
EUX_TEST(injected_faults_end_as_errors) {
  namespace tr = eux::ucxx::transport;
  Pair p;
  p.server.RegisterFunction(function_id_t{1}, [](int32_t a) { return a + 1; }, "inc");
  std::atomic<int> provider_calls{0};
  CustomMemoryPolicy<UcxBuffer> flaky = [&](eux::rpc::utils::TensorMetaSpan metas) -> UcxBuffer {
    if (provider_calls.fetch_add(1) == 0) throw std::bad_alloc();
    return UcxBuffer(*p.mr, ucx_memory_type::HOST, eux::rpc::utils::CalculateTensorSize(metas[0]));
  };
  p.server.RegisterFunction<UcxBuffer>(function_id_t{2}, [](const TensorMeta&, const UcxBuffer& b) { return int64_t(b.size()); }, "size_of",
                                       flaky, MessageLifecyclePolicy{});
  p.connect();
  p.client.SetTimeout(200ms);
  auto call_inc = [&](int32_t v) {
    return ex::sync_wait(p.client.InvokeRpc("server", session_id_t{1}, function_id_t{1}, workflow_id_t{}, ClientMemoryPolicy{}, v));
  };
  CHECK_EQ(call_inc(1)->header.GetPrimitive<int32_t>(0), 2);

  // 1. the server's next eager frame (the response) is lost
  std::atomic<int> dropped{0};
  tr::set_fault_hook([&](const std::string& worker, uint8_t type, uint64_t) {
    return worker == "server" && type == tr::kAmEager && dropped.fetch_add(1) == 0;
  });
  bool deadline = false;
  auto t0 = std::chrono::steady_clock::now();
  try {
    call_inc(5);
  } catch (const RpcException& e) {
    deadline = e.code() == make_error_code(RpcErrc::DEADLINE_EXCEEDED);
  }
  CHECK(deadline);
  CHECK(std::chrono::steady_clock::now() - t0 < 2000ms);
  tr::set_fault_hook(nullptr);
  CHECK_EQ(dropped.load() >= 1, true);
  CHECK_EQ(call_inc(7)->header.GetPrimitive<int32_t>(0), 8);
  CHECK_EQ(p.client.PendingRpcCount(), 0u);

  // 2. the memory policy fails once: the caller gets an error status, the next call goes through
  auto send_tensor = [&] {
    const int64_t n = 65536;
    UcxBuffer buf(*p.mr, ucx_memory_type::HOST, size_t(n) * 4);
    std::memset(buf.data(), 0, buf.size());
    return ex::sync_wait(p.client.InvokeRpc("server", session_id_t{1}, function_id_t{2}, workflow_id_t{}, ClientMemoryPolicy{}, f32_meta(n), std::move(buf)));
  };
  p.client.SetTimeout(2000ms);
  bool failed = false;
  try {
    auto r = send_tensor();
    failed = r && !r->header.status.ok();
  } catch (const std::exception&) {
    failed = true;
  }
  CHECK(failed);
  auto ok = send_tensor();
  CHECK(ok && ok->header.status.ok());
  CHECK_EQ(ok->header.GetPrimitive<int64_t>(0), int64_t(65536 * 4));

  // 3. the receiver's clear-to-send for a rendezvous payload is lost: the caller's deadline ends the call
  p.client.SetTimeout(200ms);
  std::atomic<int> cts_dropped{0};
  tr::set_fault_hook([&](const std::string& worker, uint8_t type, uint64_t) {
    return worker == "server" && type == tr::kRndvCts && cts_dropped.fetch_add(1) == 0;
  });
  bool timed_out = false;
  try {
    auto r = send_tensor();
    timed_out = r && !r->header.status.ok();
  } catch (const std::exception&) {
    timed_out = true;
  }
  tr::set_fault_hook(nullptr);
  CHECK(timed_out);
  CHECK_EQ(cts_dropped.load() >= 1, true);
  p.client.SetTimeout(2000ms);
  auto again = send_tensor();
  CHECK(again && again->header.status.ok());
}

EUX_TEST(forked_processes_echo) {
#if defined(__SANITIZE_THREAD__)
  // ThreadSanitizer's runtime does not let a forked child of a process that has had threads start threads
  // of its own, which a worker needs; the case runs in every other build.
  return;
#endif
  int addr_pipe[2], ctl_pipe[2];
  CHECK(pipe(addr_pipe) == 0 && pipe(ctl_pipe) == 0);
  pid_t pid = fork();
  CHECK(pid >= 0);
  if (pid == 0) {  // server child
    close(addr_pipe[0]);
    close(ctl_pipe[1]);
    int rc = 1;
    {
      AxonRuntime rt("forked_server", 2, 2000ms);
      rt.RegisterFunction(function_id_t{1}, [](const data::string& s, const data::vector<int64_t>& v) {
        int64_t sum = std::accumulate(v.begin(), v.end(), int64_t(0));
        return std::tuple<data::string, int64_t>(data::string(s.str() + "/ok"), sum);
      }, std::string("join"));
      if (!rt.StartServer()) {
        auto addr = rt.GetLocalAddress();
        uint32_t n = addr.size();
        if (write(addr_pipe[1], &n, 4) == 4 && write(addr_pipe[1], addr.data(), n) == (ssize_t)n) {
          char c;
          rc = read(ctl_pipe[0], &c, 1) == 1 ? 0 : 2;  // wait for the shutdown byte
        }
      }
      rt.Stop();
    }
    _exit(rc);
  }
  close(addr_pipe[1]);
  close(ctl_pipe[0]);
  uint32_t n = 0;
  CHECK(read(addr_pipe[0], &n, 4) == 4 && n > 0 && n < 4096);
  std::vector<std::byte> addr(n);
  CHECK(read(addr_pipe[0], addr.data(), n) == (ssize_t)n);
  {
    AxonRuntime rt("forked_client", 2, 2000ms);
    CHECK(!rt.StartClient());
    rt.ConnectEndpoint(addr, "forked_server");
    auto r = ex::sync_wait(rt.InvokeRpc("forked_server", session_id_t{3}, function_id_t{1}, workflow_id_t{}, ClientMemoryPolicy{}, data::string("ping"),
                                        data::vector<int64_t>{1, 2, 3, 4}));
    CHECK(r && r->header.status.ok());
    CHECK(r->header.GetString(0) == "ping/ok");
    CHECK_EQ(r->header.GetPrimitive<int64_t>(1), 10);
    rt.Stop();
  }
  CHECK(write(ctl_pipe[1], "x", 1) == 1);
  int status = 0;
  CHECK(waitpid(pid, &status, 0) == pid);
  CHECK(WIFEXITED(status) && WEXITSTATUS(status) == 0);
}

EUX_TEST_MAIN()
