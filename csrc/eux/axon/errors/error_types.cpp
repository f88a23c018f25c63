#include "eux/axon/errors/error_types.hpp"

namespace eux::axon::errors {

std::string ToString(AxonErrc e) {
  switch (e) {
    case AxonErrc::Ok: return "Ok";
    case AxonErrc::WorkerNotFound: return "Worker not found";
    case AxonErrc::WorkerStartFailed: return "Worker failed to start";
    case AxonErrc::CoordinatorError: return "Coordinator error";
    case AxonErrc::ConnectError: return "Connect error";
    case AxonErrc::SerializeError: return "Serialization error";
    case AxonErrc::StorageBackpressure: return "Storage back-pressure: the worker rejects new messages";
    case AxonErrc::DeserializeError: return "Deserialization error";
    case AxonErrc::RemoteRespondError: return "The remote side could not respond";
  }
  return "Unknown Axon error";
}

namespace {
class Category final : public std::error_category {
 public:
  const char* name() const noexcept override { return "AxonErrc"; }
  std::string message(int ev) const override { return ToString(static_cast<AxonErrc>(ev)); }
};
const Category& category_instance() {
  static const Category c;
  return c;
}
// known to the registry before any status can arrive from a peer
const bool registered = [] {
  rpc::RpcCategoryRegistry::GetInstance().RegisterCategory(category_instance());
  return true;
}();
}  // namespace

const std::error_category& AxonErrcCategory() {
  (void)registered;
  return category_instance();
}
std::error_code make_error_code(AxonErrc e) { return {static_cast<int>(e), AxonErrcCategory()}; }

}  // namespace eux::axon::errors
