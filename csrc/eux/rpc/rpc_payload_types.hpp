// Payload kinds of an RPC: none, one contiguous buffer, or a vector of buffers
// (reference: rpc_core/rpc_payload_types.hpp:34-65).
#pragma once

#include <optional>
#include <variant>

#include "eux/ucxx/ucx_context_data.hpp"

namespace eux::rpc {

// Deleter that keeps a received buffer alive for as long as something parsed
// out of it is in use (zero-copy headers).
template <class T>
  requires std::is_same_v<T, ucxx::UcxBuffer> || std::is_same_v<T, ucxx::UcxBufferVec> || std::is_same_v<T, ucxx::UcxHeader>
struct UcxDataDeleter {
  UcxDataDeleter() = default;
  explicit UcxDataDeleter(T&& buffer) : buffer_(std::move(buffer)) {}
  template <class P>
  void operator()(P*) {
    buffer_.reset();
  }

 private:
  std::optional<T> buffer_;
};
using UcxHeaderDeleter = UcxDataDeleter<ucxx::UcxHeader>;
using UcxBufferDeleter = UcxDataDeleter<ucxx::UcxBuffer>;
using UcxBufferVecDeleter = UcxDataDeleter<ucxx::UcxBufferVec>;

enum class PayloadType : uint8_t {
  UCX_BUFFER = 0,
  UCX_BUFFER_VEC = 1,
  NO_PAYLOAD = 2,
  MONOSTATE = NO_PAYLOAD,
};

using PayloadVariant = std::variant<std::monostate, ucxx::UcxBuffer, ucxx::UcxBufferVec>;
using ReturnedPayload = PayloadVariant;

template <class T>
constexpr PayloadType payload_type_of() {
  using D = std::decay_t<T>;
  if constexpr (std::is_same_v<D, ucxx::UcxBuffer>) return PayloadType::UCX_BUFFER;
  else if constexpr (std::is_same_v<D, ucxx::UcxBufferVec>) return PayloadType::UCX_BUFFER_VEC;
  else return PayloadType::NO_PAYLOAD;
}
inline PayloadType payload_type_of(const PayloadVariant& v) {
  return v.index() == 1 ? PayloadType::UCX_BUFFER : (v.index() == 2 ? PayloadType::UCX_BUFFER_VEC : PayloadType::NO_PAYLOAD);
}

}  // namespace eux::rpc
