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
  template <class ReceivedBufferT, class F>
  bool RegisterFunction(rpc::function_id_t id, F&& f, const std::string& name, CustomMemoryPolicy<ReceivedBufferT> provider,
                        MessageLifecyclePolicy lc_policy = TransientPolicy{}) {
    ServerMemoryPolicy mp;
    mp.on_host = false;
    if constexpr (std::is_same_v<ReceivedBufferT, ucxx::UcxBuffer>) mp.buffer_provider = std::move(provider);
    else mp.buffer_vec_provider = std::move(provider);
    return RegisterFunction(id, std::forward<F>(f), name, std::move(mp), std::move(lc_policy));
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
  InvokeSender InvokeRpc(std::string_view worker_name, rpc::RpcRequestHeader&& header, rpc::PayloadVariant&& payload = {},
                         ClientMemoryPolicy mem_policy = {});

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
