// AxonWorker: the RPC runtime. It owns two active-message contexts (server and
// client, one thread each), a thread pool that runs handlers, a timer thread for
// deadlines, an asynchronous dispatcher, the retained-request storage and the
// observers (reference: axon/include/axon/axon_worker.hpp:151-1271,
// axon/src/axon_worker.cpp).
//
// Server: receive header -> parse, merge clock, back-pressure gate, find the
// handler -> receive the payload where the handler's memory policy says ->
// run the handler on the pool under a deadline -> apply the lifecycle policy ->
// send the response. Client: InvokeRpc registers the call in a 2048-slot table
// indexed by request id, sends, and completes when the response (and its
// payload) has arrived, the deadline passed, or the call was cancelled.
#pragma once

#include <atomic>
#include <chrono>
#include <functional>
#include <memory>
#include <mutex>
#include <optional>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "eux/axon/errors/error_types.hpp"
#include "eux/axon/memory_policy.hpp"
#include "eux/axon/message_lifecycle_policy.hpp"
#include "eux/axon/metrics/metrics_observer.hpp"
#include "eux/axon/storage/axon_storage.hpp"
#include "eux/axon/utils/axon_message.hpp"
#include "eux/axon/utils/hash.hpp"
#include "eux/axon/utils/ring_buffer.hpp"
#include "eux/axon/utils/slot_map.hpp"
#include "eux/exec/async_scope.hpp"
#include "eux/exec/contexts.hpp"
#include "eux/rpc/async_rpc_dispatcher.hpp"
#include "eux/ucxx/ucx_am_context.hpp"

namespace eux::axon {

constexpr size_t kPendingRpcBufferSize = 2048;

// What a finished call gives the caller.
struct InvokeResult {
  rpc::RpcResponseHeader header;
  rpc::PayloadVariant payload;
};
using InvokeSender = exec::any_sender_of<InvokeResult>;

// Either policy kind for either payload form, type-erased for the function table.
// `provider_inline`: the provider neither blocks nor takes long (it takes a block from a pool, say), so it is
// called on the context's own thread; otherwise it is user code of unknown cost and runs on the thread pool,
// which costs every rendezvous message two hand-overs between threads.
struct ServerMemoryPolicy {
  bool on_host = true;
  CustomMemoryPolicy<ucxx::UcxBuffer> buffer_provider;        // used when the function takes a UcxBuffer
  CustomMemoryPolicy<ucxx::UcxBufferVec> buffer_vec_provider;  // used when it takes a UcxBufferVec
  bool provider_inline = false;
  // The handler itself never blocks either (it only starts asynchronous work and returns a sender, as the
  // Python binding's handlers do, which hand the call to the event loop): start it on the server context's
  // thread as well instead of on the pool.
  bool handler_inline = false;
};
struct ClientMemoryPolicy {
  bool on_host = true;
  CustomMemoryPolicy<ucxx::UcxBuffer> buffer_provider;
  CustomMemoryPolicy<ucxx::UcxBufferVec> buffer_vec_provider;
  bool want_vec = false;  // receive a scatter-gather response as separate buffers
  bool provider_inline = false;
};

// What a call made through the typed overloads gives the caller: the response header and the payload in the
// form that the caller named (reference: axon/include/axon/axon_worker.hpp:985-992).
template <class RespBufferT>
using TypedInvokeResult = std::pair<rpc::ResponseHeaderUniquePtr, RespBufferT>;

namespace detail {
template <class T>
concept IsMonostate = std::is_same_v<std::decay_t<T>, std::monostate>;
template <class T>
concept IsBuffer = std::is_same_v<std::decay_t<T>, ucxx::UcxBuffer> || std::is_same_v<std::decay_t<T>, ucxx::UcxBufferVec>;
template <class T>
concept IsBufferOrVariant = IsBuffer<T> || std::is_same_v<std::decay_t<T>, rpc::PayloadVariant>;
template <class T>
concept ValidInvokePayload = IsBufferOrVariant<T> || IsMonostate<T>;
template <class T>
concept ValidInvokeResponse = IsBufferOrVariant<T> || IsMonostate<T>;
template <class T>
concept ValidRegisterBuffer = IsBufferOrVariant<T> || IsMonostate<T>;
// A memory policy as such, whatever it is used with.
template <class T>
concept IsMemoryPolicy = std::is_same_v<std::decay_t<T>, AlwaysOnHostPolicy> || std::is_same_v<std::decay_t<T>, CustomMemoryPolicy<ucxx::UcxBuffer>> ||
                         std::is_same_v<std::decay_t<T>, CustomMemoryPolicy<ucxx::UcxBufferVec>> ||
                         std::is_same_v<std::decay_t<T>, ReceiverMemoryPolicy<ucxx::UcxBuffer>> ||
                         std::is_same_v<std::decay_t<T>, ReceiverMemoryPolicy<ucxx::UcxBufferVec>>;
// ... and one that fits the buffer form it is used with: a provider of single buffers cannot serve a call that
// wants separate buffers and the other way round; a variant or no payload goes with either.
template <class MemPolicyT, class BufferT>
concept ValidMemPolicyFor =
    IsMemoryPolicy<MemPolicyT> &&
    (std::is_same_v<std::decay_t<MemPolicyT>, AlwaysOnHostPolicy> || IsMonostate<BufferT> || std::is_same_v<std::decay_t<BufferT>, rpc::PayloadVariant> ||
     std::is_same_v<std::decay_t<MemPolicyT>, CustomMemoryPolicy<std::decay_t<BufferT>>> ||
     std::is_same_v<std::decay_t<MemPolicyT>, ReceiverMemoryPolicy<std::decay_t<BufferT>>>);
template <class... Args>
struct first_arg_is_memory_policy : std::false_type {};
template <class A, class... Rest>
struct first_arg_is_memory_policy<A, Rest...> : std::bool_constant<IsMemoryPolicy<A>> {};

template <class BufferT, class MemPolicyT, class Erased>
Erased erase_policy(MemPolicyT&& p) {
  Erased out;
  using P = std::decay_t<MemPolicyT>;
  if constexpr (std::is_same_v<std::decay_t<BufferT>, ucxx::UcxBufferVec> && requires { out.want_vec; }) out.want_vec = true;
  if constexpr (std::is_same_v<P, CustomMemoryPolicy<ucxx::UcxBuffer>>) {
    out.on_host = false;
    out.buffer_provider = std::forward<MemPolicyT>(p);
  } else if constexpr (std::is_same_v<P, CustomMemoryPolicy<ucxx::UcxBufferVec>>) {
    out.on_host = false;
    out.buffer_vec_provider = std::forward<MemPolicyT>(p);
    if constexpr (requires { out.want_vec; }) out.want_vec = true;
  } else if constexpr (!std::is_same_v<P, AlwaysOnHostPolicy>) {  // the variant of the two
    std::visit([&](auto& alt) { out = erase_policy<BufferT, decltype(alt), Erased>(alt); }, p);
  }
  return out;
}
}  // namespace detail

class AxonWorker {
 public:
  using BypassRejectionFunction = std::function<bool(const rpc::RpcRequestHeader&)>;
  using StoredRequestVisitor = std::function<LifecycleStatus(std::shared_ptr<utils::AxonRequest>, utils::AxonMessageID)>;

  static size_t DefaultThreadPoolSize() { return std::thread::hardware_concurrency() < 16 ? 4 : 16; }

  AxonWorker(std::shared_ptr<ucxx::UcxMemoryResourceManager> mr, std::string worker_name,
             size_t thread_pool_size = DefaultThreadPoolSize(), std::chrono::milliseconds timeout = std::chrono::milliseconds(300),
             std::unique_ptr<ucxx::UcxAutoDeviceContext> device_context = nullptr);
  ~AxonWorker();
  AxonWorker(const AxonWorker&) = delete;

  // ---- lifecycle ----
  std::error_code StartServer();
  std::error_code StartClient();
  std::error_code Start() {
    if (auto ec = StartServer()) return ec;
    return StartClient();
  }
  void StopServer();
  void StopClient();  // pending calls end with CANCELLED
  void Stop() {
    StopClient();
    StopServer();
  }
  bool server_running() const { return server_running_.load(); }
  bool client_running() const { return client_running_.load(); }

  const std::string& name() const { return name_; }
  std::vector<std::byte> GetLocalAddress() const;  // of the server context
  rpc::byte_buf GetLocalSignatures() const { return dispatcher_.GetAllSignatures(); }

  // ---- endpoints (client side) ----
  exec::any_sender_of<uint64_t> ConnectEndpointAsync(std::vector<std::byte> address, std::string worker_name);
  uint64_t ConnectEndpoint(std::vector<std::byte> address, std::string worker_name);  // blocking form; throws on failure
  bool RegisterEndpointSignatures(std::string_view worker_name, const void* data, size_t size);
  std::optional<rpc::RpcFunctionSignature> GetEndpointSignature(std::string_view worker_name, rpc::function_id_t id) const;
  std::optional<uint64_t> GetConnectionId(std::string_view worker_name) const;
  // An endpoint's key: stable while the endpoint exists, never reused for another one (the slot's generation
  // differs), and cheaper to resolve than the name (reference: axon_worker.hpp:166, 1010-1042).
  using WorkerKey = utils::SlotKey;
  std::optional<WorkerKey> GetWorkerKey(std::string_view worker_name) const;
  std::optional<uint64_t> GetConnectionId(WorkerKey key) const;
  std::optional<std::string> GetWorkerName(WorkerKey key) const;
  bool DisconnectEndpoint(std::string_view worker_name);

  // ---- functions (server side) ----
  // Typed registration: `f` is any callable whose arguments are filled by type (see RpcDispatcher);
  // it may return a value or a sender.
  template <class F>
  bool RegisterFunction(rpc::function_id_t id, F&& f, const std::string& name, ServerMemoryPolicy mem_policy = {},
                        MessageLifecyclePolicy lc_policy = TransientPolicy{}) {
    if (!dispatcher_.RegisterFunction(id, std::forward<F>(f), rpc::data::string(name))) return false;
    return AddFunctionPolicies(id, std::move(mem_policy), std::move(lc_policy));
  }
  // RegisterFunction<ReceivedBufferT[, Fn, MemPolicyT, LcT]>(id, fn, name, policy, lifecycle): the reference's
  // parameter list (axon_worker.hpp:432-443). ReceivedBufferT names the form in which a rendezvous payload is
  // received for the policy: UcxBuffer, UcxBufferVec, PayloadVariant (either, as the sender's metadata says)
  // or std::monostate (the function takes no payload).
  template <class ReceivedBufferT, class Fn, class MemPolicyT = AlwaysOnHostPolicy, class LcT = TransientPolicy>
    requires detail::ValidRegisterBuffer<ReceivedBufferT> && detail::ValidMemPolicyFor<MemPolicyT, ReceivedBufferT> && is_message_lifecycle_policy_v<LcT> &&
             (!std::is_convertible_v<Fn, std::string_view>)
  bool RegisterFunction(rpc::function_id_t id, Fn&& fn, std::string_view name = {}, MemPolicyT mem_policy = AlwaysOnHostPolicy{}, LcT lc_policy = TransientPolicy{}) {
    return RegisterFunction(id, std::forward<Fn>(fn), std::string(name), detail::erase_policy<ReceivedBufferT, MemPolicyT, ServerMemoryPolicy>(std::move(mem_policy)),
                            MessageLifecyclePolicy(std::move(lc_policy)));
  }
  template <class ReceivedBufferT, class MemPolicyT = AlwaysOnHostPolicy, class LcT = TransientPolicy>
    requires detail::ValidRegisterBuffer<ReceivedBufferT> && detail::ValidMemPolicyFor<MemPolicyT, ReceivedBufferT> && is_message_lifecycle_policy_v<LcT>
  bool RegisterFunction(rpc::function_id_t id, std::string_view name, const rpc::data::vector<rpc::ParamType>& param_types,
                        const rpc::data::vector<rpc::ParamType>& return_types, rpc::PayloadType input_payload_type, rpc::PayloadType return_payload_type,
                        rpc::DynamicAsyncRpcFunction&& fn, MemPolicyT mem_policy = AlwaysOnHostPolicy{}, LcT lc_policy = TransientPolicy{}) {
    return RegisterFunction(id, std::string(name), param_types, return_types, input_payload_type, return_payload_type, std::move(fn),
                            detail::erase_policy<ReceivedBufferT, MemPolicyT, ServerMemoryPolicy>(std::move(mem_policy)), MessageLifecyclePolicy(std::move(lc_policy)));
  }
  template <class ReceivedBufferT, class LcT>
    requires detail::ValidRegisterBuffer<ReceivedBufferT> && is_message_lifecycle_policy_v<LcT> && (!detail::IsMemoryPolicy<LcT>)
  bool RegisterFunction(rpc::function_id_t id, std::string_view name, const rpc::data::vector<rpc::ParamType>& param_types,
                        const rpc::data::vector<rpc::ParamType>& return_types, rpc::PayloadType input_payload_type, rpc::PayloadType return_payload_type,
                        rpc::DynamicAsyncRpcFunction&& fn, LcT lc_policy) {
    return RegisterFunction<ReceivedBufferT>(id, name, param_types, return_types, input_payload_type, return_payload_type, std::move(fn), AlwaysOnHostPolicy{},
                                             std::move(lc_policy));
  }
  // Dynamic registration: explicit signature, type-erased callable.
  bool RegisterFunction(rpc::function_id_t id, const std::string& name, const rpc::data::vector<rpc::ParamType>& param_types,
                        const rpc::data::vector<rpc::ParamType>& return_types, rpc::PayloadType input_payload_type,
                        rpc::PayloadType return_payload_type, rpc::DynamicAsyncRpcFunction&& fn, ServerMemoryPolicy mem_policy = {},
                        MessageLifecyclePolicy lc_policy = TransientPolicy{});
  bool UnregisterFunction(rpc::function_id_t id);

  // ---- calls (client side) ----
  // High level: arguments are packed like RpcRequestBuilder::PrepareRequest (at most one payload).
  template <class... Args>
  InvokeSender InvokeRpc(std::string_view worker_name, rpc::session_id_t session, rpc::function_id_t function,
                         rpc::utils::workflow_id_t workflow, ClientMemoryPolicy mem_policy, Args&&... args) {
    rpc::RpcRequestBuilderOptions opt{session, rpc::request_id_t{0}, function, {}, workflow};
    if constexpr (rpc::payload_finder<Args...>::count == 1) {
      auto [header, payload] = rpc::RpcRequestBuilder{}.PrepareRequest(opt, std::forward<Args>(args)...);
      return InvokeRpc(worker_name, std::move(header), std::move(payload), std::move(mem_policy));
    } else {
      auto header = rpc::RpcRequestBuilder{}.PrepareRequest(opt, std::forward<Args>(args)...);
      return InvokeRpc(worker_name, std::move(header), rpc::PayloadVariant{}, std::move(mem_policy));
    }
  }
  // Dynamic: a prepared header (its request id and clock are assigned here) and an optional payload.
  InvokeSender InvokeRpc(std::string_view worker_name, rpc::RpcRequestHeader&& header, rpc::PayloadVariant&& payload, ClientMemoryPolicy mem_policy);
  InvokeSender InvokeRpc(WorkerKey worker_key, rpc::RpcRequestHeader&& header, rpc::PayloadVariant&& payload, ClientMemoryPolicy mem_policy);

  // ---- calls, typed (the reference's template parameter lists over the calls above) ----
  // InvokeRpc<RespBufferT[, MemPolicyT]>(name | key, session, function, workflow[, policy], args...): arguments
  // packed as above; completes with {unique_ptr<RpcResponseHeader>, RespBufferT}. RespBufferT is UcxBuffer,
  // UcxBufferVec, PayloadVariant or std::monostate (payload dropped); the policy is AlwaysOnHostPolicy, a
  // CustomMemoryPolicy<RespBufferT> or the variant of both. A response whose payload has another form than
  // the one named ends the call with INVALID_ARGUMENT. Errors arrive as in the untyped calls, as an exception
  // that carries the status (reference: axon_worker.hpp:300-378).
  template <class RespBufferT, class MemPolicyT, class... Args>
    requires detail::ValidInvokeResponse<RespBufferT> && detail::ValidMemPolicyFor<MemPolicyT, RespBufferT>
  auto InvokeRpc(std::string_view worker_name, rpc::session_id_t session, rpc::function_id_t function, rpc::utils::workflow_id_t workflow,
                 MemPolicyT mem_policy, Args&&... args) {
    return Typed<RespBufferT>(InvokeRpc(worker_name, session, function, workflow,
                                        detail::erase_policy<RespBufferT, MemPolicyT, ClientMemoryPolicy>(std::move(mem_policy)), std::forward<Args>(args)...));
  }
  template <class RespBufferT, class... Args>
    requires detail::ValidInvokeResponse<RespBufferT> && (!detail::first_arg_is_memory_policy<std::decay_t<Args>...>::value)
  auto InvokeRpc(std::string_view worker_name, rpc::session_id_t session, rpc::function_id_t function, rpc::utils::workflow_id_t workflow,
                 Args&&... args) {
    return InvokeRpc<RespBufferT>(worker_name, session, function, workflow, AlwaysOnHostPolicy{}, std::forward<Args>(args)...);
  }
  template <class RespBufferT, class MemPolicyT, class... Args>
    requires detail::ValidInvokeResponse<RespBufferT> && detail::ValidMemPolicyFor<MemPolicyT, RespBufferT>
  auto InvokeRpc(WorkerKey worker_key, rpc::session_id_t session, rpc::function_id_t function, rpc::utils::workflow_id_t workflow,
                 MemPolicyT mem_policy, Args&&... args) {
    rpc::RpcRequestBuilderOptions opt{session, rpc::request_id_t{0}, function, {}, workflow};
    auto policy = detail::erase_policy<RespBufferT, MemPolicyT, ClientMemoryPolicy>(std::move(mem_policy));
    if constexpr (rpc::payload_finder<Args...>::count == 1) {
      auto [header, payload] = rpc::RpcRequestBuilder{}.PrepareRequest(opt, std::forward<Args>(args)...);
      return Typed<RespBufferT>(InvokeRpc(worker_key, std::move(header), rpc::PayloadVariant(std::move(payload)), std::move(policy)));
    } else {
      auto header = rpc::RpcRequestBuilder{}.PrepareRequest(opt, std::forward<Args>(args)...);
      return Typed<RespBufferT>(InvokeRpc(worker_key, std::move(header), rpc::PayloadVariant{}, std::move(policy)));
    }
  }
  template <class RespBufferT, class... Args>
    requires detail::ValidInvokeResponse<RespBufferT> && (!detail::first_arg_is_memory_policy<std::decay_t<Args>...>::value)
  auto InvokeRpc(WorkerKey worker_key, rpc::session_id_t session, rpc::function_id_t function, rpc::utils::workflow_id_t workflow, Args&&... args) {
    return InvokeRpc<RespBufferT>(worker_key, session, function, workflow, AlwaysOnHostPolicy{}, std::forward<Args>(args)...);
  }
  // InvokeRpc<PayloadT, RespBufferT, MemPolicyT>(name | key, header, payload | optional<payload>, policy): a
  // prepared header (reference: axon_worker.hpp:381-429).
  template <class PayloadT = std::monostate, class RespBufferT = std::monostate, class MemPolicyT = AlwaysOnHostPolicy>
    requires detail::ValidInvokePayload<PayloadT> && detail::ValidInvokeResponse<RespBufferT> && detail::ValidMemPolicyFor<MemPolicyT, RespBufferT>
  auto InvokeRpc(std::string_view worker_name, rpc::RpcRequestHeader&& header, std::optional<PayloadT>&& payload = std::nullopt,
                 MemPolicyT mem_policy = AlwaysOnHostPolicy{}) {
    return Typed<RespBufferT>(InvokeRpc(worker_name, std::move(header), ErasePayload(std::move(payload)),
                                        detail::erase_policy<RespBufferT, MemPolicyT, ClientMemoryPolicy>(std::move(mem_policy))));
  }
  template <class PayloadT, class RespBufferT = std::monostate, class MemPolicyT = AlwaysOnHostPolicy>
    requires detail::ValidInvokePayload<PayloadT> && (!detail::IsMonostate<PayloadT>) && detail::ValidInvokeResponse<RespBufferT> &&
             detail::ValidMemPolicyFor<MemPolicyT, RespBufferT>
  auto InvokeRpc(std::string_view worker_name, rpc::RpcRequestHeader&& header, PayloadT&& payload, MemPolicyT mem_policy = AlwaysOnHostPolicy{}) {
    return InvokeRpc<PayloadT, RespBufferT, MemPolicyT>(worker_name, std::move(header), std::optional<PayloadT>(std::move(payload)), std::move(mem_policy));
  }
  template <class PayloadT = std::monostate, class RespBufferT = std::monostate, class MemPolicyT = AlwaysOnHostPolicy>
    requires detail::ValidInvokePayload<PayloadT> && detail::ValidInvokeResponse<RespBufferT> && detail::ValidMemPolicyFor<MemPolicyT, RespBufferT>
  auto InvokeRpc(WorkerKey worker_key, rpc::RpcRequestHeader&& header, std::optional<PayloadT>&& payload = std::nullopt,
                 MemPolicyT mem_policy = AlwaysOnHostPolicy{}) {
    return Typed<RespBufferT>(InvokeRpc(worker_key, std::move(header), ErasePayload(std::move(payload)),
                                        detail::erase_policy<RespBufferT, MemPolicyT, ClientMemoryPolicy>(std::move(mem_policy))));
  }
  template <class PayloadT, class RespBufferT = std::monostate, class MemPolicyT = AlwaysOnHostPolicy>
    requires detail::ValidInvokePayload<PayloadT> && (!detail::IsMonostate<PayloadT>) && detail::ValidInvokeResponse<RespBufferT> &&
             detail::ValidMemPolicyFor<MemPolicyT, RespBufferT>
  auto InvokeRpc(WorkerKey worker_key, rpc::RpcRequestHeader&& header, PayloadT&& payload, MemPolicyT mem_policy = AlwaysOnHostPolicy{}) {
    return InvokeRpc<PayloadT, RespBufferT, MemPolicyT>(worker_key, std::move(header), std::optional<PayloadT>(std::move(payload)), std::move(mem_policy));
  }

  // ---- knobs ----
  void SetTimeout(std::chrono::milliseconds t) { timeout_ms_.store(t.count()); }
  std::chrono::milliseconds GetTimeout() const { return std::chrono::milliseconds(timeout_ms_.load()); }
  // Back-pressure: while set, incoming requests are answered with StorageBackpressure unless the bypass function says otherwise.
  void SetRejectMessages(bool reject) { reject_messages_.store(reject); }
  bool GetRejectMessages() const { return reject_messages_.load(); }
  void SetBypassRejectionFunction(BypassRejectionFunction fn);
  void SetMetricsObserver(metrics::MetricsObserver obs);
  void SetErrorObserver(errors::ErrorObserver obs);
  void ReportServerMetrics();
  void ReportClientMetrics();

  // ---- retained requests ----
  storage::AxonStorage& GetStorage() { return *storage_; }
  // Counters of the transports under the server and the client context, added up (how many device
  // payloads were pulled, pushed, sent eagerly, staged through the host, ...). Read without
  // synchronisation: meant for tests and monitoring between calls.
  ucxx::transport::Worker::Stats GetTransportStats() const;
  // Re-run every stored request through its registered handler (responses are dropped); returns how many ran.
  size_t ProcessStoredRequests();
  // Show every stored request to a visitor; Discard removes it from the storage.
  size_t ProcessStoredRequests(const StoredRequestVisitor& visitor);

  ucxx::UcxMemoryResourceManager& DefaultMemoryProvider() { return *mr_; }
  // The contexts that run the two pipelines (null before StartServer / StartClient): a handler that returns a
  // sender can complete it on the server's loop, e.g. with its scheduler's schedule_when_flag().
  ucxx::ucx_am_context* server_context() noexcept { return server_ctx_.get(); }
  ucxx::ucx_am_context* client_context() noexcept { return client_ctx_.get(); }
  rpc::utils::HybridLogicalClock CurrentHlc() const;
  size_t PendingRpcCount() const { return pending_rpcs_.size(); }

 private:
  struct FunctionPolicies {
    ServerMemoryPolicy mem;
    MessageLifecyclePolicy lifecycle;
  };
  struct RemoteEndpoint {
    std::string name;
    uint64_t conn_id = 0;
    std::unordered_map<uint32_t, rpc::RpcFunctionSignature> signatures;
  };
  struct ResponseArrival {  // what the client loop hands to a pending call
    rpc::RpcResponseHeader header;
    std::optional<ucxx::UcxBuffer> eager;
    std::optional<size_t> rndv_key;
    uint64_t conn_id = 0;
  };
  struct PendingRpc {
    uint32_t session_id = 0;
    std::function<void(std::optional<ResponseArrival>&&, std::exception_ptr)> complete;
  };
  class InvokeOpState;
  struct invoke_sender;
  friend class InvokeOpState;

  InvokeSender InvokeOnConnection(std::optional<uint64_t> conn, std::string whom, rpc::RpcRequestHeader&& header, rpc::PayloadVariant&& payload,
                                  ClientMemoryPolicy mem_policy);
  template <class PayloadT>
  static rpc::PayloadVariant ErasePayload(std::optional<PayloadT>&& p) {
    if constexpr (detail::IsMonostate<PayloadT>) return {};
    else if (p) return rpc::PayloadVariant(std::move(*p));
    else return {};
  }
  // The untyped result in the form the caller named.
  template <class RespBufferT>
  TypedInvokeResult<RespBufferT> ToTyped(InvokeResult&& r) {
    auto header = std::make_unique<rpc::RpcResponseHeader>(std::move(r.header));
    if constexpr (detail::IsMonostate<RespBufferT>) {
      return {std::move(header), std::monostate{}};
    } else if constexpr (std::is_same_v<RespBufferT, rpc::PayloadVariant>) {
      return {std::move(header), std::move(r.payload)};
    } else {
      if (auto* b = std::get_if<RespBufferT>(&r.payload)) return {std::move(header), std::move(*b)};
      if constexpr (std::is_same_v<RespBufferT, ucxx::UcxBufferVec>) {
        // a small response arrives in one piece: cut it where the header's tensor metadata says
        if (auto* one = std::get_if<ucxx::UcxBuffer>(&r.payload)) {
          std::vector<size_t> sizes;
          size_t sum = 0;
          for (auto& m : utils::GetTensorMetas(header->results)) sum += sizes.emplace_back(rpc::utils::TensorPayloadBytes(m));
          if (sizes.empty() || sum != one->size()) sizes.assign(1, one->size());
          return {std::move(header), std::move(*one).to_buffer_vec(sizes)};
        }
      }
      if (!std::holds_alternative<std::monostate>(r.payload))
        throw std::system_error(rpc::make_error_code(rpc::RpcErrc::INVALID_ARGUMENT), "the response payload has another form than the one asked for");
      if constexpr (std::is_same_v<RespBufferT, ucxx::UcxBuffer>) return {std::move(header), ucxx::UcxBuffer(*mr_, ucx_memory_type::HOST, 0)};
      else return {std::move(header), ucxx::UcxBufferVec(*mr_, ucx_memory_type::HOST, std::vector<size_t>{})};
    }
  }
  template <class RespBufferT>
  auto Typed(InvokeSender&& s) {
    return exec::then(std::move(s), [this](InvokeResult&& r) { return ToTyped<RespBufferT>(std::move(r)); });
  }
  bool AddFunctionPolicies(rpc::function_id_t id, ServerMemoryPolicy mem, MessageLifecyclePolicy lc);
  std::optional<FunctionPolicies> FindPolicies(rpc::function_id_t id) const;
  rpc::utils::HybridLogicalClock TickHlc();
  void MergeHlc(const rpc::utils::HybridLogicalClock& remote);

  // server pipeline
  void ServerLoopStart();
  void ServerHandleArrival(ucxx::recv_header_result_t&& arrival);
  void ServerRunRequest(std::shared_ptr<struct ServerCall> call);
  void ServerDispatch(std::shared_ptr<struct ServerCall> call);
  void ServerSendResponse(std::shared_ptr<struct ServerCall> call, rpc::RpcResponseHeader&& header, rpc::PayloadVariant&& payload);
  void ServerSendError(uint64_t conn_id, const rpc::RpcRequestHeader& req, std::error_code ec, std::string_view what);
  void ReportError(errors::AxonErrorContext ctx);

  // client pipeline
  void ClientLoopStart();
  void ClientHandleArrival(ucxx::recv_header_result_t&& arrival);
  void ClientFinishWithPayload(std::shared_ptr<struct ClientCall> call);

  std::shared_ptr<ucxx::UcxMemoryResourceManager> mr_;
  std::string name_;
  std::atomic<int64_t> timeout_ms_;
  std::unique_ptr<ucxx::UcxAutoDeviceContext> device_context_;
  int device_id_ = -1;

  std::unique_ptr<ucxx::ucx_am_context> server_ctx_, client_ctx_;
  std::thread server_thread_, client_thread_;
  // re-created by every StartServer / StartClient: a stop source and a scope cannot be un-stopped
  std::unique_ptr<exec::inplace_stop_source> server_stop_ = std::make_unique<exec::inplace_stop_source>(),
                                             client_stop_ = std::make_unique<exec::inplace_stop_source>();
  std::unique_ptr<exec::inplace_stop_source> server_loop_stop_, client_loop_stop_;
  std::atomic<bool> server_running_{false}, client_running_{false};
  exec::static_thread_pool pool_;
  exec::timed_single_thread_context time_ctx_;
  std::unique_ptr<exec::async_scope> server_scope_ = std::make_unique<exec::async_scope>(),
                                     client_scope_ = std::make_unique<exec::async_scope>();

  rpc::AsyncRpcDispatcher dispatcher_;
  mutable std::mutex policies_mu_;
  std::unordered_map<uint32_t, FunctionPolicies> policies_;

  mutable std::mutex hlc_mu_;
  rpc::utils::HybridLogicalClock hlc_;
  std::atomic<uint32_t> next_request_id_{1};
  utils::RingBuffer<PendingRpc, kPendingRpcBufferSize> pending_rpcs_;

  mutable std::mutex endpoints_mu_;
  utils::SharedSlotMap<RemoteEndpoint> endpoints_;
  std::unordered_map<std::string, utils::SlotKey> endpoint_by_name_;

  std::atomic<bool> reject_messages_{false};
  mutable std::mutex hooks_mu_;
  BypassRejectionFunction bypass_fn_;
  metrics::MetricsObserver metrics_observer_;
  errors::ErrorObserver error_observer_;
  std::unique_ptr<storage::AxonStorage> storage_;
  std::atomic<size_t> client_pipe_failed_{0}, server_pipe_invoked_{0}, server_pipe_failed_{0};
  std::mutex rejected_mu_;
  std::vector<std::pair<uint64_t, time_t>> rejected_info_;
};

}  // namespace eux::axon
