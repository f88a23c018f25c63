#include "eux/axon/axon_worker.hpp"

#include <ctime>

#include "eux/axon/axon_worker_detail.hpp"
#include "eux/ucxx/ucx_context_logger.hpp"

namespace eux::axon {

using namespace eux::axon::detail;

// ---------------------------------------------------------------------------------------
AxonWorker::AxonWorker(std::shared_ptr<ucxx::UcxMemoryResourceManager> mr, std::string worker_name, size_t thread_pool_size,
                       std::chrono::milliseconds timeout, std::unique_ptr<ucxx::UcxAutoDeviceContext> device_context)
    : mr_(std::move(mr)), name_(std::move(worker_name)), timeout_ms_(timeout.count()), device_context_(std::move(device_context)),
      pool_(thread_pool_size ? thread_pool_size : 1), dispatcher_(name_), storage_(std::make_unique<storage::AxonStorage>()) {
  if (!mr_) throw std::invalid_argument("AxonWorker needs a memory resource manager");
  if (device_context_) device_id_ = device_context_->device_id();
  (void)errors::AxonErrcCategory();  // make sure the category is registered before any status arrives
  hlc_ = rpc::utils::HybridLogicalClock::Now();
}

AxonWorker::~AxonWorker() { Stop(); }

std::error_code AxonWorker::StartServer() {
  if (server_running_.exchange(true)) return {};
  try {
    server_ctx_ = std::make_unique<ucxx::ucx_am_context>(*mr_, name_, GetTimeout(), true, 0, clone_device_context(device_id_));
  } catch (const std::exception& e) {
    server_running_ = false;
    UCX_CTX_ERROR << name_ << ": server context failed to start: " << e.what();
    return errors::make_error_code(errors::AxonErrc::WorkerStartFailed);
  }
  server_loop_stop_ = std::make_unique<ex::inplace_stop_source>();
  server_stop_ = std::make_unique<ex::inplace_stop_source>();
  server_scope_ = std::make_unique<ex::async_scope>();
  server_thread_ = std::thread([this] { server_ctx_->run(server_stop_->get_token()); });
  ex::sync_wait(server_ctx_->get_scheduler().schedule());  // the loop is up
  ServerLoopStart();
  return {};
}

std::error_code AxonWorker::StartClient() {
  if (client_running_.exchange(true)) return {};
  try {
    client_ctx_ = std::make_unique<ucxx::ucx_am_context>(*mr_, name_ + ".client", GetTimeout(), true, 0, clone_device_context(device_id_));
  } catch (const std::exception& e) {
    client_running_ = false;
    UCX_CTX_ERROR << name_ << ": client context failed to start: " << e.what();
    return errors::make_error_code(errors::AxonErrc::WorkerStartFailed);
  }
  client_loop_stop_ = std::make_unique<ex::inplace_stop_source>();
  client_stop_ = std::make_unique<ex::inplace_stop_source>();
  client_scope_ = std::make_unique<ex::async_scope>();
  client_thread_ = std::thread([this] { client_ctx_->run(client_stop_->get_token()); });
  ex::sync_wait(client_ctx_->get_scheduler().schedule());
  ClientLoopStart();
  return {};
}

void AxonWorker::StopServer() {
  if (!server_running_.exchange(false)) return;
  server_loop_stop_->request_stop();
  server_scope_->request_stop();
  // handlers in flight get the time of one deadline to finish, then the context goes down under them
  ex::sync_wait(ex::stop_when(server_scope_->join(), ex::schedule_after(time_ctx_.get_scheduler(), GetTimeout() + std::chrono::milliseconds(200))));
  server_stop_->request_stop();
  if (server_thread_.joinable()) server_thread_.join();
  ex::sync_wait(server_scope_->join());
  server_ctx_.reset();
}

void AxonWorker::StopClient() {
  if (!client_running_.exchange(false)) return;
  client_loop_stop_->request_stop();
  // every pending call ends with CANCELLED
  pending_rpcs_.drain([](uint64_t, PendingRpc&& p) {
    if (p.complete) p.complete(std::nullopt, rpc_error(rpc::make_error_code(RpcErrc::CANCELLED), "the client was stopped"));
  });
  client_scope_->request_stop();
  ex::sync_wait(ex::stop_when(client_scope_->join(), ex::schedule_after(time_ctx_.get_scheduler(), GetTimeout() + std::chrono::milliseconds(200))));
  client_stop_->request_stop();
  if (client_thread_.joinable()) client_thread_.join();
  ex::sync_wait(client_scope_->join());
  {
    std::lock_guard lk(endpoints_mu_);
    endpoint_by_name_.clear();
    endpoints_.clear();
  }
  client_ctx_.reset();
}

std::vector<std::byte> AxonWorker::GetLocalAddress() const {
  // A client-only worker still has a reachable address (its client context listens too): peers that
  // want to call back, or tools that only print it, get that one.
  std::vector<std::byte> a;
  if (server_ctx_) server_ctx_->get_ucp_address(a);
  else if (client_ctx_) client_ctx_->get_ucp_address(a);
  return a;
}

ucxx::transport::Worker::Stats AxonWorker::GetTransportStats() const {
  ucxx::transport::Worker::Stats t;
  for (auto* ctx : {server_ctx_.get(), client_ctx_.get()}) {
    if (!ctx) continue;
    const auto& s = ctx->worker().stats();
    t.frames_refused += s.frames_refused;
    t.regions_ignored += s.regions_ignored;
    t.device_pulls += s.device_pulls;
    t.device_staged += s.device_staged;
    t.truncated += s.truncated;
    t.device_eager_sent += s.device_eager_sent;
    t.device_eager_recv += s.device_eager_recv;
    t.device_pushes += s.device_pushes;
    t.device_push_recv += s.device_push_recv;
    t.kernel_launches += s.kernel_launches;
    t.device_gathers += s.device_gathers;
    t.device_packs += s.device_packs;
    t.sends_held += s.sends_held;
    t.vmm_fds_sent += s.vmm_fds_sent;
    t.vmm_fds_recv += s.vmm_fds_recv;
  }
  return t;
}

// ---- clock, hooks -----------------------------------------------------------------------
rpc::utils::HybridLogicalClock AxonWorker::TickHlc() {
  std::lock_guard lk(hlc_mu_);
  hlc_.TickLocal();
  return hlc_;
}
void AxonWorker::MergeHlc(const rpc::utils::HybridLogicalClock& remote) {
  std::lock_guard lk(hlc_mu_);
  hlc_.Merge(remote);
}
rpc::utils::HybridLogicalClock AxonWorker::CurrentHlc() const {
  std::lock_guard lk(hlc_mu_);
  return hlc_;
}
void AxonWorker::SetBypassRejectionFunction(BypassRejectionFunction fn) {
  std::lock_guard lk(hooks_mu_);
  bypass_fn_ = std::move(fn);
}
void AxonWorker::SetMetricsObserver(metrics::MetricsObserver obs) {
  std::lock_guard lk(hooks_mu_);
  metrics_observer_ = std::move(obs);
}
void AxonWorker::SetErrorObserver(errors::ErrorObserver obs) {
  std::lock_guard lk(hooks_mu_);
  error_observer_ = std::move(obs);
}
void AxonWorker::ReportError(errors::AxonErrorContext ctx) {
  errors::ErrorObserver obs;
  {
    std::lock_guard lk(hooks_mu_);
    obs = error_observer_;
  }
  UCX_CTX_DEBUG << name_ << ": " << ctx.what << " (function " << ctx.function_id << ", session " << ctx.session_id << ")";
  if (obs) obs->OnError(ctx);
}
void AxonWorker::ReportServerMetrics() {
  metrics::MetricsObserver obs;
  {
    std::lock_guard lk(hooks_mu_);
    obs = metrics_observer_;
  }
  if (!obs) return;
  metrics::WorkerMetrics m;
  m.server_pipe_invoked_count = server_pipe_invoked_.load();
  m.server_pipe_failed_count = server_pipe_failed_.load();
  {
    std::lock_guard lk(rejected_mu_);
    m.server_ucx_rejected_messages_info = rejected_info_;
  }
  obs->OnWorkerStats(std::move(m));
}
void AxonWorker::ReportClientMetrics() {
  metrics::MetricsObserver obs;
  {
    std::lock_guard lk(hooks_mu_);
    obs = metrics_observer_;
  }
  if (!obs) return;
  metrics::WorkerMetrics m;
  m.pending_rpcs_count = pending_rpcs_.size();
  m.client_pipe_failed_count = client_pipe_failed_.load();
  obs->OnWorkerStats(std::move(m));
}

// ---- function table -----------------------------------------------------------------------
bool AxonWorker::AddFunctionPolicies(rpc::function_id_t id, ServerMemoryPolicy mem, MessageLifecyclePolicy lc) {
  std::lock_guard lk(policies_mu_);
  policies_[id.v_] = FunctionPolicies{std::move(mem), std::move(lc)};
  return true;
}
std::optional<AxonWorker::FunctionPolicies> AxonWorker::FindPolicies(rpc::function_id_t id) const {
  std::lock_guard lk(policies_mu_);
  auto it = policies_.find(id.v_);
  if (it == policies_.end()) return std::nullopt;
  return it->second;
}
bool AxonWorker::RegisterFunction(rpc::function_id_t id, const std::string& name, const rpc::data::vector<rpc::ParamType>& param_types,
                                  const rpc::data::vector<rpc::ParamType>& return_types, rpc::PayloadType input_payload_type,
                                  rpc::PayloadType return_payload_type, rpc::DynamicAsyncRpcFunction&& fn, ServerMemoryPolicy mem_policy,
                                  MessageLifecyclePolicy lc_policy) {
  if (!dispatcher_.RegisterFunction(id, rpc::data::string(name), param_types, return_types, input_payload_type, return_payload_type, std::move(fn)))
    return false;
  return AddFunctionPolicies(id, std::move(mem_policy), std::move(lc_policy));
}
bool AxonWorker::UnregisterFunction(rpc::function_id_t id) {
  {
    std::lock_guard lk(policies_mu_);
    policies_.erase(id.v_);
  }
  return dispatcher_.UnregisterFunction(id);
}

}  // namespace eux::axon
