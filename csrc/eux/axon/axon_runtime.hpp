// AxonRuntime: owning facade over AxonWorker used by the language bindings and
// by applications that want one object with start/stop/connect/register/invoke
// (reference: axon/include/axon/axon_runtime.hpp:52-353, axon/src/axon_runtime.cpp).
#pragma once

#include <memory>
#include <string>

#include "eux/axon/axon_worker.hpp"

namespace eux::axon {

class AxonRuntime {
 public:
  AxonRuntime(std::string worker_name, size_t thread_pool_size = AxonWorker::DefaultThreadPoolSize(),
              std::chrono::milliseconds timeout = std::chrono::milliseconds(300),
              std::unique_ptr<ucxx::UcxAutoDeviceContext> device_context = nullptr,
              std::shared_ptr<ucxx::UcxMemoryResourceManager> mr = nullptr);
  ~AxonRuntime();
  AxonRuntime(const AxonRuntime&) = delete;

  std::error_code Start() { return worker_->Start(); }
  std::error_code StartServer() { return worker_->StartServer(); }
  std::error_code StartClient() { return worker_->StartClient(); }
  void Stop() { worker_->Stop(); }
  void StopServer() { worker_->StopServer(); }
  void StopClient() { worker_->StopClient(); }

  std::vector<std::byte> GetLocalAddress() const { return worker_->GetLocalAddress(); }
  rpc::byte_buf GetLocalSignatures() const { return worker_->GetLocalSignatures(); }
  const std::string& GetWorkerName() const { return worker_->name(); }

  exec::any_sender_of<uint64_t> ConnectEndpointAsync(std::vector<std::byte> address, std::string worker_name) {
    return worker_->ConnectEndpointAsync(std::move(address), std::move(worker_name));
  }
  uint64_t ConnectEndpoint(std::vector<std::byte> address, std::string worker_name) {
    return worker_->ConnectEndpoint(std::move(address), std::move(worker_name));
  }
  bool RegisterEndpointSignatures(std::string_view worker_name, const void* data, size_t size) {
    return worker_->RegisterEndpointSignatures(worker_name, data, size);
  }

  // Every overload of the worker, the typed ones with their template arguments included:
  // rt.InvokeRpc<ucxx::UcxBuffer>(...), rt.RegisterFunction<ucxx::UcxBuffer>(...).
  template <class... T, class... A>
  bool RegisterFunction(A&&... a) {
    if constexpr (sizeof...(T) == 0) return worker_->RegisterFunction(std::forward<A>(a)...);
    else return worker_->template RegisterFunction<T...>(std::forward<A>(a)...);
  }
  template <class... T, class... A>
  auto InvokeRpc(A&&... a) {
    if constexpr (sizeof...(T) == 0) return worker_->InvokeRpc(std::forward<A>(a)...);
    else return worker_->template InvokeRpc<T...>(std::forward<A>(a)...);
  }
  std::optional<AxonWorker::WorkerKey> GetWorkerKey(std::string_view worker_name) const { return worker_->GetWorkerKey(worker_name); }

  void SetTimeout(std::chrono::milliseconds t) { worker_->SetTimeout(t); }
  void SetRejectMessages(bool r) { worker_->SetRejectMessages(r); }
  void SetBypassRejectionFunction(AxonWorker::BypassRejectionFunction fn) { worker_->SetBypassRejectionFunction(std::move(fn)); }
  void SetMetricsObserver(metrics::MetricsObserver o) { worker_->SetMetricsObserver(std::move(o)); }
  void SetErrorObserver(errors::ErrorObserver o) { worker_->SetErrorObserver(std::move(o)); }

  AxonWorker& worker() { return *worker_; }
  std::shared_ptr<ucxx::UcxMemoryResourceManager> memory_resource() const { return mr_; }

 private:
  std::shared_ptr<ucxx::UcxMemoryResourceManager> mr_;
  std::unique_ptr<AxonWorker> worker_;
};

}  // namespace eux::axon
