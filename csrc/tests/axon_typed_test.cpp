// The typed call and registration forms of AxonWorker / AxonRuntime, written the way a user of the reference
// writes them: InvokeRpc<RespBufferT>(name | key, session, function, workflow[, policy], args...),
// InvokeRpc<PayloadT, RespBufferT[, MemPolicyT]>(name | key, header, payload[, policy]),
// RegisterFunction<ReceivedBufferT>(id, fn, name[, policy[, lifecycle]]) and the dynamic registration with an
// explicit signature (reference: axon/include/axon/axon_worker.hpp:300-500; the call shapes are those of
// axon/tests/axon_worker_test.cpp:95-130, 192-200, 321-327, 424-430).
#include <atomic>
#include <cstring>
#include <thread>

#include "check.hpp"
#include "eux/axon/axon_runtime.hpp"

using namespace eux::axon;
using namespace eux::rpc;
using eux::ucxx::DefaultUcxMemoryResourceManager;
using eux::ucxx::UcxBuffer;
using eux::ucxx::UcxBufferVec;
namespace ex = eux::exec;
using namespace std::chrono_literals;

namespace {

TensorMeta u8_meta(int64_t n) {
  TensorMeta m;
  m.ndim = 1;
  m.dtype = {kDLUInt, 8, 1};
  m.shape = {n};
  m.strides = {1};
  return m;
}

UcxBuffer text(DefaultUcxMemoryResourceManager& mr, const std::string& s) {
  UcxBuffer b(mr, ucx_memory_type::HOST, s.size());
  std::memcpy(b.data(), s.data(), s.size());
  return b;
}
std::string str(const UcxBuffer& b) { return std::string(static_cast<const char*>(b.data()), b.size()); }

RpcResponseHeader ok_header(const RpcRequestHeader& req) {
  RpcResponseHeader h;
  h.session_id = req.session_id;
  h.request_id = req.request_id;
  h.workflow_id = req.workflow_id;
  return h;
}

struct Pair {
  std::shared_ptr<DefaultUcxMemoryResourceManager> mr = std::make_shared<DefaultUcxMemoryResourceManager>();
  AxonWorker server{mr, "server", 4, 2000ms};
  AxonWorker client{mr, "client", 2, 2000ms};
  void connect() {
    CHECK(!server.StartServer());
    CHECK(!client.StartClient());
    client.ConnectEndpoint(server.GetLocalAddress(), "server");
  }
  // the echo of the reference's tests: header-and-payload handler that answers with a sender of a pair
  void register_echo(uint32_t id) {
    CHECK(server.RegisterFunction<UcxBuffer>(function_id_t{id}, [](const RpcRequestHeader& header, UcxBuffer&& payload) {
      return ex::just(std::make_pair(ok_header(header), std::move(payload)));
    }, "echo"));
  }
};

}  // namespace

EUX_TEST(typed_call_by_name_gives_header_pointer_and_buffer) {
  Pair p;
  p.register_echo(1001);
  p.connect();
  auto r = ex::sync_wait(p.client.InvokeRpc<UcxBuffer, UcxBuffer>("server", session_id_t{1}, function_id_t{1001}, workflow_id_t{0}, text(*p.mr, "Hello Axon")));
  CHECK(r.has_value());
  auto& [header, payload] = *r;
  static_assert(std::is_same_v<std::decay_t<decltype(header)>, ResponseHeaderUniquePtr>);
  static_assert(std::is_same_v<std::decay_t<decltype(payload)>, UcxBuffer>);
  CHECK(header->status.ok());
  CHECK_EQ(header->session_id.v_, 1u);
  CHECK(str(payload) == "Hello Axon");
}

EUX_TEST(typed_call_by_worker_key) {
  Pair p;
  p.register_echo(1);
  p.connect();
  auto key = p.client.GetWorkerKey("server");
  CHECK(key.has_value());
  CHECK(*p.client.GetWorkerName(*key) == "server");
  CHECK(p.client.GetConnectionId(*key) == p.client.GetConnectionId("server"));
  auto r = ex::sync_wait(p.client.InvokeRpc<UcxBuffer>(*key, session_id_t{3}, function_id_t{1}, workflow_id_t{9}, text(*p.mr, "by key")));
  CHECK(r && r->first->status.ok() && str(r->second) == "by key");
  CHECK_EQ(r->first->workflow_id.v_, 9u);
  // prepared header by key
  RpcRequestHeader h;
  h.session_id = session_id_t{4};
  h.function_id = function_id_t{1};
  auto d = ex::sync_wait(p.client.InvokeRpc<UcxBuffer, UcxBuffer>(*key, std::move(h), text(*p.mr, "dyn by key")));
  CHECK(d && str(d->second) == "dyn by key");
  // a key does not outlive its endpoint, and is not handed to the next one either
  CHECK(p.client.DisconnectEndpoint("server"));
  CHECK(!p.client.GetWorkerName(*key).has_value());
  CHECK_THROWS(ex::sync_wait(p.client.InvokeRpc<UcxBuffer>(*key, session_id_t{3}, function_id_t{1}, workflow_id_t{}, text(*p.mr, "gone"))));
  p.client.ConnectEndpoint(p.server.GetLocalAddress(), "server");
  auto key2 = p.client.GetWorkerKey("server");
  CHECK(key2 && !(*key2 == *key));
  CHECK_THROWS(ex::sync_wait(p.client.InvokeRpc<UcxBuffer>(*key, session_id_t{3}, function_id_t{1}, workflow_id_t{}, text(*p.mr, "stale"))));
  auto again = ex::sync_wait(p.client.InvokeRpc<UcxBuffer>(*key2, session_id_t{3}, function_id_t{1}, workflow_id_t{}, text(*p.mr, "fresh")));
  CHECK(again && str(again->second) == "fresh");
  CHECK(!p.client.GetWorkerKey("nobody").has_value());
}

EUX_TEST(typed_call_with_prepared_header_and_dynamic_function) {
  Pair p;
  DynamicAsyncRpcFunction dyn_echo = [](const RpcRequestHeader& req, PayloadVariant&& payload, const RpcResponseBuilder&) -> AsyncInvokeSender {
    RpcInvokeResult<ReturnedPayload> out;
    out.header = ok_header(req);
    if (auto* b = std::get_if<UcxBuffer>(&payload)) out.payload = std::move(*b);
    return ex::just(std::move(out));
  };
  CHECK(p.server.RegisterFunction<UcxBuffer>(function_id_t{2001}, "dyn_echo", data::vector<ParamType>{}, data::vector<ParamType>{}, PayloadType::UCX_BUFFER,
                                             PayloadType::UCX_BUFFER, std::move(dyn_echo)));
  p.connect();
  RpcRequestHeader header;
  header.session_id = session_id_t{1};
  header.function_id = function_id_t{2001};
  auto r = ex::sync_wait(p.client.InvokeRpc<UcxBuffer, UcxBuffer>("server", std::move(header), std::optional<UcxBuffer>(text(*p.mr, "Hello Axon Dynamic"))));
  CHECK(r.has_value());
  auto& [resp_header, resp_payload] = *r;
  CHECK(resp_header->status.ok());
  CHECK(str(resp_payload) == "Hello Axon Dynamic");
  // the payload given directly, not wrapped in an optional
  RpcRequestHeader h2;
  h2.session_id = session_id_t{1};
  h2.function_id = function_id_t{2001};
  auto r2 = ex::sync_wait(p.client.InvokeRpc<UcxBuffer, UcxBuffer>("server", std::move(h2), text(*p.mr, "direct")));
  CHECK(r2 && str(r2->second) == "direct");
  // the signature carries what was registered
  auto sigs = p.server.GetLocalSignatures();
  CHECK(p.client.RegisterEndpointSignatures("server", sigs.data(), sigs.size()));
  auto sig = p.client.GetEndpointSignature("server", function_id_t{2001});
  CHECK(sig && sig->function_name == "dyn_echo" && sig->return_payload_type == PayloadType::UCX_BUFFER);
}

EUX_TEST(typed_call_without_payload_either_way) {
  Pair p;
  p.server.RegisterFunction<std::monostate>(function_id_t{5}, [](int32_t a, int32_t b) { return a * b; }, "mul");
  p.connect();
  auto r = ex::sync_wait(p.client.InvokeRpc<std::monostate>("server", session_id_t{1}, function_id_t{5}, workflow_id_t{}, int32_t(6), int32_t(7)));
  CHECK(r.has_value());
  static_assert(std::is_same_v<std::decay_t<decltype(r->second)>, std::monostate>);
  CHECK(r->first->status.ok());
  CHECK_EQ(r->first->GetPrimitive<int32_t>(0), 42);
  // a prepared header and nothing else: every template argument at its default
  RpcRequestHeader h;
  h.session_id = session_id_t{2};
  h.function_id = function_id_t{5};
  h.AddParam(int32_t(3));
  h.AddParam(int32_t(5));
  auto d = ex::sync_wait(p.client.InvokeRpc("server", std::move(h)));
  CHECK(d && d->first->status.ok());
  CHECK_EQ(d->first->GetPrimitive<int32_t>(0), 15);
  // a function that is not there: the status travels in the header, the call itself succeeds
  auto nf = ex::sync_wait(p.client.InvokeRpc<std::monostate>("server", session_id_t{1}, function_id_t{404}, workflow_id_t{}));
  CHECK(nf && nf->first->status.value == int(RpcErrc::NOT_FOUND));
  // an endpoint that is not there: the call fails
  CHECK_THROWS(ex::sync_wait(p.client.InvokeRpc<std::monostate>("nobody", session_id_t{1}, function_id_t{5}, workflow_id_t{})));
}

EUX_TEST(typed_call_with_a_custom_memory_policy_on_both_sides) {
  Pair p;
  std::atomic<int> server_provider{0}, client_provider{0};
  CustomMemoryPolicy<UcxBuffer> server_policy = [&](eux::rpc::utils::TensorMetaSpan metas) {
    server_provider.fetch_add(1);
    return UcxBuffer(*p.mr, ucx_memory_type::HOST, size_t(metas[0].shape[0]));
  };
  CHECK(p.server.RegisterFunction<UcxBuffer>(function_id_t{7}, [](const TensorMeta& m, UcxBuffer&& payload) {
    return std::tuple<TensorMeta, UcxBuffer>(m, std::move(payload));
  }, "echo_tensor", server_policy));
  p.connect();
  const int64_t n = 1 << 20;  // rendezvous: only then is a policy consulted
  UcxBuffer big(*p.mr, ucx_memory_type::HOST, size_t(n));
  std::memset(big.data(), 0x5a, size_t(n));
  void* mine = nullptr;
  CustomMemoryPolicy<UcxBuffer> client_policy = [&](eux::rpc::utils::TensorMetaSpan metas) {
    client_provider.fetch_add(1);
    UcxBuffer b(*p.mr, ucx_memory_type::HOST, size_t(metas[0].shape[0]));
    mine = b.data();
    return b;
  };
  auto r = ex::sync_wait(p.client.InvokeRpc<UcxBuffer>("server", session_id_t{1}, function_id_t{7}, workflow_id_t{}, client_policy, u8_meta(n), std::move(big)));
  CHECK(r && r->first->status.ok());
  CHECK_EQ(server_provider.load(), 1);
  CHECK_EQ(client_provider.load(), 1);
  CHECK(r->second.data() == mine);  // the response landed in the buffer that the policy handed out
  CHECK_EQ(r->second.size(), size_t(n));
  CHECK_EQ(static_cast<const unsigned char*>(r->second.data())[n - 1], 0x5au);
  // the variant form of the policy, holding the always-on-host alternative
  UcxBuffer big2(*p.mr, ucx_memory_type::HOST, size_t(n));
  std::memset(big2.data(), 1, size_t(n));
  ReceiverMemoryPolicy<UcxBuffer> either = AlwaysOnHostPolicy{};
  auto r2 = ex::sync_wait(p.client.InvokeRpc<UcxBuffer>("server", session_id_t{1}, function_id_t{7}, workflow_id_t{}, either, u8_meta(n), std::move(big2)));
  CHECK(r2 && r2->second.size() == size_t(n));
  CHECK_EQ(client_provider.load(), 1);
}

EUX_TEST(typed_call_for_separate_buffers) {
  Pair p;
  // two tensors out of one: the response names them with a vector of metadata and carries separate buffers
  CHECK(p.server.RegisterFunction<UcxBuffer>(function_id_t{8}, [&p](const TensorMeta& m, UcxBuffer&& payload) {
    const size_t half = size_t(m.shape[0]) / 2;
    UcxBufferVec out(*p.mr, ucx_memory_type::HOST, std::vector<size_t>{half, half});
    std::memcpy(out.buffers()[0].data, payload.data(), half);
    std::memcpy(out.buffers()[1].data, static_cast<const char*>(payload.data()) + half, half);
    data::vector<TensorMeta> metas;
    metas.push_back(u8_meta(int64_t(half)));
    metas.push_back(u8_meta(int64_t(half)));
    return std::tuple<data::vector<TensorMeta>, UcxBufferVec>(std::move(metas), std::move(out));
  }, "split"));
  p.connect();
  for (int64_t n : {int64_t(64), int64_t(1) << 20}) {  // eager (arrives in one piece and is cut here) and rendezvous
    UcxBuffer in(*p.mr, ucx_memory_type::HOST, size_t(n));
    auto* c = static_cast<unsigned char*>(in.data());
    for (int64_t i = 0; i < n; ++i) c[i] = static_cast<unsigned char>(i < n / 2 ? 1 : 2);
    auto r = ex::sync_wait(p.client.InvokeRpc<UcxBufferVec>("server", session_id_t{1}, function_id_t{8}, workflow_id_t{}, u8_meta(n), std::move(in)));
    CHECK(r && r->first->status.ok());
    CHECK_EQ(r->second.size(), 2u);
    CHECK_EQ(r->second.buffers()[0].size, size_t(n / 2));
    CHECK_EQ(static_cast<const unsigned char*>(r->second.buffers()[0].data)[0], 1u);
    CHECK_EQ(static_cast<const unsigned char*>(r->second.buffers()[1].data)[n / 2 - 1], 2u);
  }
  // asking for one buffer where separate ones arrive is refused, not silently flattened
  UcxBuffer in(*p.mr, ucx_memory_type::HOST, size_t(1) << 20);
  std::memset(in.data(), 0, in.size());
  CHECK_THROWS(ex::sync_wait(p.client.InvokeRpc<UcxBuffer>("server", session_id_t{1}, function_id_t{8}, workflow_id_t{}, u8_meta(1 << 20), std::move(in))));
}

EUX_TEST(typed_call_for_whatever_arrives) {
  Pair p;
  p.register_echo(1);
  p.server.RegisterFunction<std::monostate>(function_id_t{2}, [](int32_t a) { return a + 1; }, "inc");
  p.connect();
  auto a = ex::sync_wait(p.client.InvokeRpc<PayloadVariant>("server", session_id_t{1}, function_id_t{1}, workflow_id_t{}, text(*p.mr, "variant")));
  CHECK(a && std::holds_alternative<UcxBuffer>(a->second) && str(std::get<UcxBuffer>(a->second)) == "variant");
  auto b = ex::sync_wait(p.client.InvokeRpc<PayloadVariant>("server", session_id_t{1}, function_id_t{2}, workflow_id_t{}, int32_t(1)));
  CHECK(b && std::holds_alternative<std::monostate>(b->second));
  CHECK_EQ(b->first->GetPrimitive<int32_t>(0), 2);
  // a buffer asked for, none sent: an empty one, not an error
  auto c = ex::sync_wait(p.client.InvokeRpc<UcxBuffer>("server", session_id_t{1}, function_id_t{2}, workflow_id_t{}, int32_t(1)));
  CHECK(c && c->second.size() == 0u);
}

EUX_TEST(typed_registration_with_lifecycle_policy) {
  Pair p;
  std::atomic<int> shown{0};
  RetentionPolicy keep = [&](std::shared_ptr<eux::axon::utils::AxonRequest> req, eux::axon::utils::AxonMessageID) {
    shown.fetch_add(1);
    return req->header.session_id.v_ == 7 ? LifecycleStatus::Preserve : LifecycleStatus::Discard;
  };
  CHECK(p.server.RegisterFunction<UcxBuffer>(function_id_t{1}, [](const RpcRequestHeader& header, UcxBuffer&& payload) {
    return ex::just(std::make_pair(ok_header(header), std::move(payload)));
  }, "kept", AlwaysOnHostPolicy{}, keep));
  // dynamic registration with a lifecycle policy and no memory policy
  DynamicAsyncRpcFunction fn = [](const RpcRequestHeader& req, PayloadVariant&&, const RpcResponseBuilder&) -> AsyncInvokeSender {
    RpcInvokeResult<ReturnedPayload> out;
    out.header = ok_header(req);
    return ex::just(std::move(out));
  };
  CHECK(p.server.RegisterFunction<std::monostate>(function_id_t{2}, "dyn_kept", data::vector<ParamType>{}, data::vector<ParamType>{}, PayloadType::NO_PAYLOAD,
                                                  PayloadType::NO_PAYLOAD, std::move(fn), keep));
  // a second function under a taken id is refused
  CHECK(!p.server.RegisterFunction<UcxBuffer>(function_id_t{1}, [](const RpcRequestHeader& header, UcxBuffer&& payload) {
    return ex::just(std::make_pair(ok_header(header), std::move(payload)));
  }, "again"));
  p.connect();
  CHECK(ex::sync_wait(p.client.InvokeRpc<UcxBuffer>("server", session_id_t{7}, function_id_t{1}, workflow_id_t{}, text(*p.mr, "keep me"))).has_value());
  CHECK(ex::sync_wait(p.client.InvokeRpc<UcxBuffer>("server", session_id_t{8}, function_id_t{1}, workflow_id_t{}, text(*p.mr, "drop me"))).has_value());
  CHECK(ex::sync_wait(p.client.InvokeRpc<std::monostate>("server", session_id_t{7}, function_id_t{2}, workflow_id_t{})).has_value());
  for (int i = 0; i < 100 && shown.load() < 3; ++i) std::this_thread::sleep_for(5ms);
  CHECK_EQ(shown.load(), 3);
  CHECK_EQ(p.server.GetStorage().size(), 2u);
}

EUX_TEST(typed_forms_through_the_runtime_facade) {
  auto mr = std::make_shared<DefaultUcxMemoryResourceManager>();
  AxonRuntime server("rt_server", 2, 2000ms, nullptr, mr), client("rt_client", 2, 2000ms, nullptr, mr);
  CHECK(server.RegisterFunction<UcxBuffer>(function_id_t{1}, [](const RpcRequestHeader& header, UcxBuffer&& payload) {
    return ex::just(std::make_pair(ok_header(header), std::move(payload)));
  }, "echo"));
  CHECK(!server.StartServer());
  CHECK(!client.StartClient());
  client.ConnectEndpoint(server.GetLocalAddress(), "rt_server");
  auto r = ex::sync_wait(client.InvokeRpc<UcxBuffer>("rt_server", session_id_t{1}, function_id_t{1}, workflow_id_t{}, text(*mr, "through the facade")));
  CHECK(r && r->first->status.ok() && str(r->second) == "through the facade");
  auto key = client.GetWorkerKey("rt_server");
  CHECK(key.has_value());
  auto k = ex::sync_wait(client.InvokeRpc<UcxBuffer>(*key, session_id_t{1}, function_id_t{1}, workflow_id_t{}, text(*mr, "facade, by key")));
  CHECK(k && str(k->second) == "facade, by key");
  // the untyped form still answers with the plain result
  auto u = ex::sync_wait(client.InvokeRpc("rt_server", session_id_t{1}, function_id_t{1}, workflow_id_t{}, ClientMemoryPolicy{}, text(*mr, "untyped")));
  CHECK(u && u->header.status.ok() && str(std::get<UcxBuffer>(u->payload)) == "untyped");
  client.Stop();
  server.Stop();
}

EUX_TEST_MAIN()
