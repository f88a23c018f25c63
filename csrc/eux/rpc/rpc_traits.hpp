// Compile-time helpers of the RPC layer: callable introspection, payload
// detection (at most one payload per call) and the C++ type -> ParamType map
// (reference: rpc_core/rpc_traits.hpp).
#pragma once

#include <functional>
#include <tuple>
#include <type_traits>

#include "eux/rpc/rpc_types.hpp"

namespace eux::rpc {

class RpcResponseBuilder;

// ---- function_traits -------------------------------------------------------
template <class F, class = void>
struct function_traits;
template <class R, class... A>
struct function_traits<R(A...)> {
  using return_type = R;
  using args_tuple = std::tuple<A...>;
  static constexpr size_t arity = sizeof...(A);
};
template <class R, class... A>
struct function_traits<R (*)(A...)> : function_traits<R(A...)> {};
template <class R, class... A>
struct function_traits<R (&)(A...)> : function_traits<R(A...)> {};
template <class C, class R, class... A>
struct function_traits<R (C::*)(A...)> : function_traits<R(A...)> {};
template <class C, class R, class... A>
struct function_traits<R (C::*)(A...) const> : function_traits<R(A...)> {};
template <class C, class R, class... A>
struct function_traits<R (C::*)(A...) noexcept> : function_traits<R(A...)> {};
template <class C, class R, class... A>
struct function_traits<R (C::*)(A...) const noexcept> : function_traits<R(A...)> {};
template <class R, class... A>
struct function_traits<std::function<R(A...)>> : function_traits<R(A...)> {};
template <class F>
struct function_traits<F, std::void_t<decltype(&std::remove_cvref_t<F>::operator())>>
    : function_traits<decltype(&std::remove_cvref_t<F>::operator())> {};

// ---- payload detection --------------------------------------------------------
template <class T>
inline constexpr bool is_payload_v = std::is_same_v<std::remove_cvref_t<T>, ucxx::UcxBuffer> ||
                                     std::is_same_v<std::remove_cvref_t<T>, ucxx::UcxBufferVec>;
template <class T>
inline constexpr bool is_payload_variant_v = std::is_same_v<std::remove_cvref_t<T>, PayloadVariant>;

template <class... T>
struct payload_finder {
  static constexpr size_t count = (size_t(0) + ... + (is_payload_v<T> || is_payload_variant_v<T> ? 1 : 0));
  static_assert(count <= 1, "an RPC function takes or returns at most one payload");
  static constexpr PayloadType type = [] {
    PayloadType t = PayloadType::NO_PAYLOAD;
    ((is_payload_v<T> ? (t = payload_type_of<T>(), 0) : 0), ...);
    return t;
  }();
};
template <class Tuple>
struct payload_finder_of;
template <class... T>
struct payload_finder_of<std::tuple<T...>> : payload_finder<T...> {};

template <class T>
struct is_tuple : std::false_type {};
template <class... T>
struct is_tuple<std::tuple<T...>> : std::true_type {};
template <class T>
struct is_pair : std::false_type {};
template <class A, class B>
struct is_pair<std::pair<A, B>> : std::true_type {};
template <class T>
struct is_strong : std::false_type {};
template <class T, class Tag>
struct is_strong<strong<T, Tag>> : std::true_type {};
template <class T>
struct is_data_vector : std::false_type {};
template <class E, class A>
struct is_data_vector<std::vector<E, A>> : std::true_type {};

// ---- C++ type -> ParamType (UNKNOWN for things that are not wire parameters) ----
template <class T>
constexpr ParamType get_param_type() {
  using D = std::remove_cvref_t<T>;
  if constexpr (std::is_void_v<D>) return ParamType::VOID;
  else if constexpr (std::is_same_v<D, TensorMeta>) return ParamType::TENSOR_META;
  else if constexpr (std::is_same_v<D, TensorMetaVec>) return ParamType::TENSOR_META_VEC;
  else if constexpr (std::is_same_v<D, data::string> || std::is_same_v<D, std::string> || std::is_same_v<D, std::string_view>) return ParamType::STRING;
  else if constexpr (std::is_enum_v<D>) return get_primitive_param_info<std::underlying_type_t<D>>().type;
  else if constexpr (std::is_arithmetic_v<D>) return get_primitive_param_info<D>().type;
  else if constexpr (is_strong<D>::value) return get_primitive_param_info<typename D::value_t>().type;
  else if constexpr (is_data_vector<D>::value) {
    using E0 = typename D::value_type;
    using E = std::conditional_t<std::is_same_v<E0, data::bool_t>, bool, E0>;
    if constexpr (std::is_arithmetic_v<E>) return get_vector_param_info<E>().type;
    else return ParamType::UNKNOWN;
  } else return ParamType::UNKNOWN;
}
template <class T>
inline constexpr bool is_wire_param_v = get_param_type<T>() != ParamType::UNKNOWN && !std::is_void_v<std::remove_cvref_t<T>>;

}  // namespace eux::rpc
