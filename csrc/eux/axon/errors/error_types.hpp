// Axon error codes (category "AxonErrc", registered with the RPC category
// registry so they survive the wire), the context attached to every reported
// error, and the observer interface
// (reference: axon/include/axon/errors/error_types.hpp:37-96).
#pragma once

#include <exception>
#include <memory>
#include <string>
#include <system_error>

#include "eux/rpc/rpc_status.hpp"
#include "eux/rpc/utils/hybrid_logical_clock.hpp"

namespace eux::axon::errors {

enum class AxonErrc {
  Ok = 0,
  WorkerNotFound,
  WorkerStartFailed,
  CoordinatorError,
  ConnectError,
  SerializeError,
  StorageBackpressure,
  DeserializeError,
  RemoteRespondError,
};

const std::error_category& AxonErrcCategory();
std::error_code make_error_code(AxonErrc e);
std::string ToString(AxonErrc e);

struct AxonErrorContext {
  uint64_t conn_id{0};
  uint32_t session_id{0};
  uint32_t request_id{0};
  uint32_t function_id{0};
  rpc::RpcStatus status = rpc::RpcStatus(rpc::make_error_code(rpc::RpcErrc::INTERNAL));
  std::string what = "Unknown error";
  rpc::utils::HybridLogicalClock hlc{};
  uint32_t workflow_id{0};
};

class AxonErrorException : public std::exception {
 public:
  explicit AxonErrorException(AxonErrorContext context) : context_(std::move(context)) {}
  const char* what() const noexcept override { return context_.what.c_str(); }
  const AxonErrorContext& context() const noexcept { return context_; }
  AxonErrorContext& context() noexcept { return context_; }

 private:
  AxonErrorContext context_;
};
inline std::exception_ptr MakeExceptionPtr(AxonErrorContext context) {
  return std::make_exception_ptr(AxonErrorException(std::move(context)));
}

class ErrorObserverBase {
 public:
  virtual ~ErrorObserverBase() = default;
  virtual void OnError(const AxonErrorContext&) = 0;
};
using ErrorObserver = std::shared_ptr<ErrorObserverBase>;

}  // namespace eux::axon::errors

namespace std {
template <>
struct is_error_code_enum<eux::axon::errors::AxonErrc> : true_type {};
}  // namespace std
