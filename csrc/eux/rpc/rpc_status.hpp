// RPC status: gRPC-like error codes with their std::error_category ("RPC"), a
// registry that maps category names back to categories (so an error_code can
// cross the wire as {int32 value, category name}), RpcStatus (the wire form)
// and RpcException (reference: rpc_core/rpc_status.hpp:33-253).
#pragma once

#include <exception>
#include <mutex>
#include <string>
#include <string_view>
#include <system_error>
#include <unordered_map>

#include "eux/rpc/data.hpp"

namespace eux::rpc {

enum class RpcErrc {
  OK = 0,
  CANCELLED = 1,
  UNKNOWN = 2,
  INVALID_ARGUMENT = 3,
  DEADLINE_EXCEEDED = 4,
  NOT_FOUND = 5,
  ALREADY_EXISTS = 6,
  PERMISSION_DENIED = 7,
  RESOURCE_EXHAUSTED = 8,
  FAILED_PRECONDITION = 9,
  ABORTED = 10,
  OUT_OF_RANGE = 11,
  UNIMPLEMENTED = 12,
  INTERNAL = 13,
  UNAVAILABLE = 14,
  DATA_LOSS = 15,
  UNAUTHENTICATED = 16,
};

}  // namespace eux::rpc
namespace std {
template <>
struct is_error_code_enum<eux::rpc::RpcErrc> : true_type {};
}  // namespace std
namespace eux::rpc {

class RpcErrorCategory final : public std::error_category {
 public:
  const char* name() const noexcept override { return "RPC"; }
  std::string message(int ev) const override {
    switch (static_cast<RpcErrc>(ev)) {
      case RpcErrc::OK: return "OK";
      case RpcErrc::CANCELLED: return "The operation was cancelled";
      case RpcErrc::UNKNOWN: return "Unknown error";
      case RpcErrc::INVALID_ARGUMENT: return "Invalid argument";
      case RpcErrc::DEADLINE_EXCEEDED: return "Deadline exceeded";
      case RpcErrc::NOT_FOUND: return "Not found";
      case RpcErrc::ALREADY_EXISTS: return "Already exists";
      case RpcErrc::PERMISSION_DENIED: return "Permission denied";
      case RpcErrc::RESOURCE_EXHAUSTED: return "Resource exhausted";
      case RpcErrc::FAILED_PRECONDITION: return "Failed precondition";
      case RpcErrc::ABORTED: return "Aborted";
      case RpcErrc::OUT_OF_RANGE: return "Out of range";
      case RpcErrc::UNIMPLEMENTED: return "Unimplemented";
      case RpcErrc::INTERNAL: return "Internal error";
      case RpcErrc::UNAVAILABLE: return "Unavailable";
      case RpcErrc::DATA_LOSS: return "Data loss";
      case RpcErrc::UNAUTHENTICATED: return "Unauthenticated";
    }
    return "Unrecognised RPC error";
  }
};

inline const std::error_category& rpc_error_category() noexcept {
  static const RpcErrorCategory cat;
  return cat;
}
inline std::error_code make_error_code(RpcErrc e) noexcept { return {static_cast<int>(e), rpc_error_category()}; }

// name -> category, so a status received from a peer becomes a real error_code again
class RpcCategoryRegistry {
 public:
  static RpcCategoryRegistry& GetInstance() {
    static RpcCategoryRegistry instance;
    return instance;
  }
  void RegisterCategory(const std::error_category& category) {
    std::lock_guard lk(mu_);
    categories_[std::string(category.name())] = &category;
  }
  const std::error_category* FindCategory(std::string_view name) const {
    std::lock_guard lk(mu_);
    auto it = categories_.find(std::string(name));
    return it == categories_.end() ? nullptr : it->second;
  }

 private:
  RpcCategoryRegistry() {
    categories_[std::generic_category().name()] = &std::generic_category();
    categories_[std::system_category().name()] = &std::system_category();
    categories_[rpc_error_category().name()] = &rpc_error_category();
  }
  mutable std::mutex mu_;
  std::unordered_map<std::string, const std::error_category*> categories_;
};

// A std::system_error (so generic code can recover the error_code) whose text is the remote or local description.
class RpcException : public std::system_error {
 public:
  RpcException(std::error_code ec, std::string what = {}) : std::system_error(ec), what_(what.empty() ? ec.message() : std::move(what)) {}
  RpcException(RpcErrc e, std::string what = {}) : RpcException(make_error_code(e), std::move(what)) {}
  const char* what() const noexcept override { return what_.c_str(); }

 private:
  std::string what_;
};

// An error_code in wire form.
struct RpcStatus {
  RpcStatus() = default;
  explicit RpcStatus(const std::error_code& ec) : value(ec.value()), category_name(ec.category().name()) {}
  RpcStatus& operator=(const std::error_code& ec) {
    value = ec.value();
    category_name = data::string(ec.category().name());
    return *this;
  }
  operator std::error_code() const {
    if (const auto* cat = RpcCategoryRegistry::GetInstance().FindCategory(category_name.view())) return {value, *cat};
    return {value, std::generic_category()};
  }
  bool ok() const { return value == 0; }
  std::string GetErrorMessage() const {
    if (const auto* cat = RpcCategoryRegistry::GetInstance().FindCategory(category_name.view())) return cat->message(value);
    return "Unknown RPC error code: " + std::to_string(value);
  }
  bool operator==(const std::error_code& other) const { return value == other.value() && category_name == other.category().name(); }

  int32_t value{0};
  data::string category_name{std::generic_category().name()};
};

inline std::exception_ptr MakeRpcExceptionPtr(RpcErrc e, std::string what = {}) {
  return std::make_exception_ptr(RpcException(e, std::move(what)));
}

}  // namespace eux::rpc
