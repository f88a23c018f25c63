// Wire types of the RPC layer: ids, parameter kinds and values, request and
// response headers, function signatures. Numeric values and field order are the
// wire contract (reference: rpc_core/rpc_types.hpp:45-454).
#pragma once

#include <memory>

#include <cstdint>
#include <stdexcept>
#include <string>
#include <string_view>
#include <type_traits>

#include "eux/rpc/data.hpp"
#include "eux/rpc/rpc_payload_types.hpp"
#include "eux/rpc/rpc_status.hpp"
#include "eux/rpc/utils/hybrid_logical_clock.hpp"
#include "eux/rpc/utils/tensor_meta.hpp"

namespace eux::rpc {

using utils::HybridLogicalClock;
using utils::TensorMeta;
using utils::workflow_id_t;

using function_id_t = strong<uint32_t, struct function_id_tag>;
using session_id_t = strong<uint32_t, struct session_id_tag>;
using request_id_t = strong<uint32_t, struct request_id_tag>;

enum class ParamType : uint8_t {
  PRIMITIVE_BOOL = 0,
  PRIMITIVE_INT8 = 1,
  PRIMITIVE_INT16 = 2,
  PRIMITIVE_INT32 = 3,
  PRIMITIVE_INT64 = 4,
  PRIMITIVE_UINT8 = 5,
  PRIMITIVE_UINT16 = 6,
  PRIMITIVE_UINT32 = 7,
  PRIMITIVE_UINT64 = 8,
  PRIMITIVE_FLOAT32 = 9,
  PRIMITIVE_FLOAT64 = 10,
  VECTOR_BOOL = 11,
  VECTOR_INT8 = 12,
  VECTOR_INT16 = 13,
  VECTOR_INT32 = 14,
  VECTOR_INT64 = 15,
  VECTOR_UINT8 = 16,
  VECTOR_UINT16 = 17,
  VECTOR_UINT32 = 18,
  VECTOR_UINT64 = 19,
  VECTOR_FLOAT32 = 20,
  VECTOR_FLOAT64 = 21,
  STRING = 22,
  VOID = 23,
  TENSOR_META = 24,
  TENSOR_META_VEC = 25,
  UNKNOWN = 255,
  LAST = UNKNOWN,
};

// Two levels of variant, as on the wire: a parameter value is one of
// {primitive, vector of primitives, string, null, tensor meta, tensor meta list}.
using PrimitiveValue =
    data::variant<bool, int8_t, int16_t, int32_t, int64_t, uint8_t, uint16_t, uint32_t, uint64_t, float, double>;
using VectorValue = data::variant<data::vector<bool>, data::vector<int8_t>, data::vector<int16_t>, data::vector<int32_t>,
                                  data::vector<int64_t>, data::vector<uint8_t>, data::vector<uint16_t>, data::vector<uint32_t>,
                                  data::vector<uint64_t>, data::vector<float>, data::vector<double>>;
using TensorMetaVec = data::vector<TensorMeta>;
using ParamValue = data::variant<PrimitiveValue, VectorValue, data::string, std::nullptr_t, TensorMeta, TensorMetaVec>;

struct ParamInfo {
  ParamType type;
  std::string_view name;
};

template <class T>
constexpr ParamInfo get_primitive_param_info() {
  using D = std::remove_cvref_t<T>;
  if constexpr (std::is_same_v<D, bool>) return {ParamType::PRIMITIVE_BOOL, "bool"};
  else if constexpr (std::is_same_v<D, int8_t>) return {ParamType::PRIMITIVE_INT8, "int8"};
  else if constexpr (std::is_same_v<D, int16_t>) return {ParamType::PRIMITIVE_INT16, "int16"};
  else if constexpr (std::is_same_v<D, int32_t>) return {ParamType::PRIMITIVE_INT32, "int32"};
  else if constexpr (std::is_same_v<D, int64_t> || std::is_same_v<D, long long>) return {ParamType::PRIMITIVE_INT64, "int64"};
  else if constexpr (std::is_same_v<D, uint8_t>) return {ParamType::PRIMITIVE_UINT8, "uint8"};
  else if constexpr (std::is_same_v<D, uint16_t>) return {ParamType::PRIMITIVE_UINT16, "uint16"};
  else if constexpr (std::is_same_v<D, uint32_t>) return {ParamType::PRIMITIVE_UINT32, "uint32"};
  else if constexpr (std::is_same_v<D, uint64_t> || std::is_same_v<D, unsigned long long>) return {ParamType::PRIMITIVE_UINT64, "uint64"};
  else if constexpr (std::is_same_v<D, float>) return {ParamType::PRIMITIVE_FLOAT32, "float32"};
  else if constexpr (std::is_same_v<D, double>) return {ParamType::PRIMITIVE_FLOAT64, "float64"};
  else static_assert(!std::is_same_v<T, T>, "not a primitive parameter type");
}
template <class T>
constexpr ParamInfo get_vector_param_info() {
  constexpr auto p = get_primitive_param_info<T>();
  return {static_cast<ParamType>(static_cast<uint8_t>(p.type) + 11), p.name};
}
// the exact alternative of PrimitiveValue that holds a T (int64_t for long long, ...)
template <class T>
using primitive_alt_t = std::conditional_t<
    std::is_same_v<T, long long>, int64_t, std::conditional_t<std::is_same_v<T, unsigned long long>, uint64_t, T>>;

struct ParamMeta {
  ParamType type = ParamType::UNKNOWN;
  ParamValue value{nullptr};
  data::string name;

  ParamMeta() = default;
  ParamMeta(ParamType t, ParamValue v, data::string n = {}) : type(t), value(std::move(v)), name(std::move(n)) {}
  // construct from a C++ value, inferring the parameter type
  template <class T>
    requires(!std::is_same_v<std::remove_cvref_t<T>, ParamMeta>)
  explicit ParamMeta(T&& v, data::string n = {}) : name(std::move(n)) {
    assign(std::forward<T>(v));
  }

 private:
  template <class T>
  void assign(T&& v) {
    using D = std::remove_cvref_t<T>;
    if constexpr (std::is_same_v<D, TensorMeta>) {
      type = ParamType::TENSOR_META;
      value = ParamValue(std::in_place_type<TensorMeta>, std::forward<T>(v));
    } else if constexpr (std::is_same_v<D, TensorMetaVec>) {
      type = ParamType::TENSOR_META_VEC;
      value = ParamValue(std::in_place_type<TensorMetaVec>, std::forward<T>(v));
    } else if constexpr (std::is_same_v<D, std::nullptr_t>) {
      type = ParamType::VOID;
      value = ParamValue(nullptr);
    } else if constexpr (std::is_same_v<D, data::string> || std::is_same_v<D, std::string> || std::is_same_v<D, std::string_view> ||
                         std::is_convertible_v<D, const char*>) {
      type = ParamType::STRING;
      value = ParamValue(std::in_place_type<data::string>, std::string_view(v));
    } else if constexpr (std::is_enum_v<D>) {
      assign(static_cast<std::underlying_type_t<D>>(v));
    } else if constexpr (std::is_arithmetic_v<D>) {
      type = get_primitive_param_info<D>().type;
      value = ParamValue(std::in_place_type<PrimitiveValue>, PrimitiveValue(std::in_place_type<primitive_alt_t<D>>, v));
    } else if constexpr (requires { typename D::value_t; D{}.v_; }) {  // strong<T>
      assign(v.v_);
    } else if constexpr (requires { typename D::value_type; v.begin(); }) {  // vector of primitives
      using E0 = typename D::value_type;
      using E = std::conditional_t<std::is_same_v<E0, data::bool_t>, bool, E0>;
      type = get_vector_param_info<E>().type;
      data::vector<primitive_alt_t<E>> out(v.begin(), v.end());
      value = ParamValue(std::in_place_type<VectorValue>, VectorValue(std::in_place_type<data::vector<primitive_alt_t<E>>>, std::move(out)));
    } else {
      static_assert(!std::is_same_v<T, T>, "type cannot be carried as an RPC parameter");
    }
  }
};

struct RpcFunctionSignature {
  data::string instance_name;
  function_id_t id;
  data::string function_name;
  data::vector<ParamType> param_types;
  data::vector<ParamType> return_types;
  PayloadType input_payload_type = PayloadType::NO_PAYLOAD;
  PayloadType return_payload_type = PayloadType::NO_PAYLOAD;
};

// Typed access to params / results, shared by both headers (CRTP).
template <class Derived>
struct RpcMessageAccessor {
 private:
  const Derived& derived() const { return static_cast<const Derived&>(*this); }
  Derived& derived() { return static_cast<Derived&>(*this); }
  const ParamMeta& item(size_t index, ParamType want, const char* what) const {
    const auto& c = derived().GetParamsContainer();
    if (index >= c.size()) throw std::out_of_range("Item index out of bounds");
    if (c[index].type != want) throw std::runtime_error(std::string("Item type mismatch for ") + what);
    return c[index];
  }

 public:
  template <class T>
  T GetPrimitive(size_t index) const {
    constexpr auto info = get_primitive_param_info<T>();
    const auto& it = item(index, info.type, info.name.data());
    return static_cast<T>(std::get<primitive_alt_t<T>>(std::get<PrimitiveValue>(it.value)));
  }
  const data::string& GetString(size_t index) const { return std::get<data::string>(item(index, ParamType::STRING, "string").value); }
  template <class T>
  const data::vector<T>& GetVector(size_t index) const {
    constexpr auto info = get_vector_param_info<T>();
    return std::get<data::vector<T>>(std::get<VectorValue>(item(index, info.type, info.name.data()).value));
  }
  const TensorMeta& GetTensor(size_t index) const { return std::get<TensorMeta>(item(index, ParamType::TENSOR_META, "tensor metadata").value); }
  const TensorMetaVec& GetTensorVec(size_t index) const {
    return std::get<TensorMetaVec>(item(index, ParamType::TENSOR_META_VEC, "tensor metadata vector").value);
  }
  data::string&& MoveString(size_t index) {
    return std::move(std::get<data::string>(const_cast<ParamMeta&>(item(index, ParamType::STRING, "string")).value));
  }
  template <class T>
  data::vector<T>&& MoveVector(size_t index) {
    constexpr auto info = get_vector_param_info<T>();
    auto& it = const_cast<ParamMeta&>(item(index, info.type, info.name.data()));
    return std::move(std::get<data::vector<T>>(std::get<VectorValue>(it.value)));
  }
  TensorMeta&& MoveTensor(size_t index) {
    return std::move(std::get<TensorMeta>(const_cast<ParamMeta&>(item(index, ParamType::TENSOR_META, "tensor metadata")).value));
  }
  TensorMetaVec&& MoveTensorVec(size_t index) {
    return std::move(
        std::get<TensorMetaVec>(const_cast<ParamMeta&>(item(index, ParamType::TENSOR_META_VEC, "tensor metadata vector")).value));
  }
  void TickLocalHlc() noexcept { derived().GetHlc().TickLocal(); }
  void MergeRemoteHlc(uint64_t remote_raw_timestamp) noexcept { derived().GetHlc().Merge(remote_raw_timestamp); }
  void MergeRemoteHlc(const HybridLogicalClock& remote) noexcept { derived().GetHlc().Merge(remote); }
  void ClearWorkflowId() noexcept { derived().GetWorkflowId() = workflow_id_t{}; }
  void AssignWorkflowId(workflow_id_t id) noexcept { derived().GetWorkflowId() = id; }
};

struct RpcRequestHeader : RpcMessageAccessor<RpcRequestHeader> {
  session_id_t session_id;
  request_id_t request_id;
  function_id_t function_id;
  HybridLogicalClock hlc{};
  workflow_id_t workflow_id{};
  data::vector<ParamMeta> params;

  template <class T>
  void AddParam(T&& value) {
    if constexpr (std::is_same_v<std::remove_cvref_t<T>, ParamMeta>) params.push_back(std::forward<T>(value));
    else params.emplace_back(std::forward<T>(value));
  }
  const data::vector<ParamMeta>& GetParamsContainer() const { return params; }
  data::vector<ParamMeta>& GetParamsContainer() { return params; }
  const HybridLogicalClock& GetHlc() const { return hlc; }
  HybridLogicalClock& GetHlc() { return hlc; }
  const workflow_id_t& GetWorkflowId() const { return workflow_id; }
  workflow_id_t& GetWorkflowId() { return workflow_id; }
};

struct RpcResponseHeader : RpcMessageAccessor<RpcResponseHeader> {
  session_id_t session_id;
  request_id_t request_id;
  HybridLogicalClock hlc{};
  workflow_id_t workflow_id{};
  RpcStatus status{};
  data::vector<ParamMeta> results;

  RpcResponseHeader() = default;
  RpcResponseHeader(session_id_t s, request_id_t r, HybridLogicalClock h, workflow_id_t w, RpcStatus st, data::vector<ParamMeta> res)
      : session_id(s), request_id(r), hlc(h), workflow_id(w), status(std::move(st)), results(std::move(res)) {}

  template <class T>
  void AddResult(T&& value) {
    if constexpr (std::is_same_v<std::remove_cvref_t<T>, ParamMeta>) results.push_back(std::forward<T>(value));
    else results.emplace_back(std::forward<T>(value));
  }
  const data::vector<ParamMeta>& GetParamsContainer() const { return results; }
  data::vector<ParamMeta>& GetParamsContainer() { return results; }
  const HybridLogicalClock& GetHlc() const { return hlc; }
  HybridLogicalClock& GetHlc() { return hlc; }
  const workflow_id_t& GetWorkflowId() const { return workflow_id; }
  workflow_id_t& GetWorkflowId() { return workflow_id; }
};

// Owning pointers to parsed headers, as handed to callers of the typed invocation API.
using RequestHeaderUniquePtr = std::unique_ptr<RpcRequestHeader>;
using ResponseHeaderUniquePtr = std::unique_ptr<RpcResponseHeader>;

}  // namespace eux::rpc
