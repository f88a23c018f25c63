// Observer interface for dispatch timing and worker statistics
// (reference: axon/include/axon/metrics/metrics_observer.hpp:36-69).
#pragma once

#include <chrono>
#include <cstdint>
#include <ctime>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "eux/rpc/utils/hybrid_logical_clock.hpp"

namespace eux::axon::metrics {

struct RpcMetricsContext {
  uint32_t session_id{0};
  uint32_t request_id{0};
  uint32_t function_id{0};
  std::string function_name;
  rpc::utils::HybridLogicalClock hlc{};
  uint32_t workflow_id{};
};

struct WorkerMetrics {
  size_t pending_rpcs_count{0};
  size_t client_pipe_failed_count{0};
  size_t server_pipe_invoked_count{0};
  size_t server_pipe_failed_count{0};
  std::vector<std::pair<uint64_t, time_t>> server_ucx_rejected_messages_info{};
};

class MetricsObserverBase {
 public:
  virtual ~MetricsObserverBase() = default;
  virtual void OnDispatchStart(const RpcMetricsContext&, std::chrono::steady_clock::time_point) {}
  virtual void OnDispatchComplete(const RpcMetricsContext&, std::chrono::steady_clock::time_point) {}
  virtual void OnWorkerStats(WorkerMetrics) {}
};
using MetricsObserver = std::shared_ptr<MetricsObserverBase>;

}  // namespace eux::axon::metrics
