// Helpers for callables that accept "any payload alternative": invoke a generic
// callable with whichever alternative a PayloadVariant holds, and check at
// compile time that a callable accepts every alternative (the role of the
// proxy-convention fold in the reference's rpc_core/rpc_facade_helpers.hpp:42-85).
#pragma once

#include <utility>
#include <variant>

#include "eux/rpc/rpc_payload_types.hpp"

namespace eux::rpc {

template <class F, class Variant>
struct accepts_all_alternatives;
template <class F, class... Alt>
struct accepts_all_alternatives<F, std::variant<Alt...>> : std::bool_constant<(std::is_invocable_v<F&, Alt&&> && ...)> {};
template <class F>
inline constexpr bool accepts_every_payload_v = accepts_all_alternatives<F, PayloadVariant>::value;

template <class F>
  requires accepts_every_payload_v<F>
decltype(auto) visit_payload(F&& f, PayloadVariant&& payload) {
  return std::visit([&](auto&& alt) -> decltype(auto) { return f(std::move(alt)); }, std::move(payload));
}

}  // namespace eux::rpc
