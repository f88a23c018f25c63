// RpcRequestBuilder: packs call arguments into an RpcRequestHeader; a payload
// among the arguments is returned beside the header
// (reference: rpc_core/rpc_request_builder.hpp:130-235).
#pragma once

#include <stdexcept>
#include <utility>

#include "eux/rpc/rpc_traits.hpp"

namespace eux::rpc {

struct RpcRequestBuilderOptions {
  session_id_t session_id{};
  request_id_t request_id{};
  function_id_t function_id{};
  HybridLogicalClock hlc{};
  workflow_id_t workflow_id{};
};

class RpcRequestBuilder {
 public:
  template <class... Args>
    requires(payload_finder<Args...>::count == 0)
  RpcRequestHeader PrepareRequest(const RpcRequestBuilderOptions& opt, Args&&... args) const {
    RpcRequestHeader h = base(opt);
    (h.params.emplace_back(std::forward<Args>(args)), ...);
    return h;
  }
  template <class... Args>
    requires(payload_finder<Args...>::count == 1)
  auto PrepareRequest(const RpcRequestBuilderOptions& opt, Args&&... args) const {
    RpcRequestHeader h = base(opt);
    PayloadVariant payload;
    auto one = [&](auto&& a) {
      using A = decltype(a);
      if constexpr (is_payload_v<A> || is_payload_variant_v<A>) payload = std::move(a);
      else h.params.emplace_back(std::forward<A>(a));
    };
    (one(std::forward<Args>(args)), ...);
    return std::pair<RpcRequestHeader, PayloadVariant>(std::move(h), std::move(payload));
  }
  // Checked against a signature obtained from the callee (service discovery).
  template <class... Args>
  auto PrepareRequest(const RpcFunctionSignature& sig, const RpcRequestBuilderOptions& opt, Args&&... args) const {
    constexpr size_t n_params = (size_t(0) + ... + (is_payload_v<Args> || is_payload_variant_v<Args> ? 0 : 1));
    if (sig.param_types.size() != n_params) throw std::invalid_argument("PrepareRequest: wrong number of arguments for " + sig.function_name.str());
    size_t i = 0;
    auto check = [&](auto&& a) {
      using A = decltype(a);
      if constexpr (!(is_payload_v<A> || is_payload_variant_v<A>)) {
        if (sig.param_types[i] != get_param_type<A>()) throw std::invalid_argument("PrepareRequest: argument type mismatch for " + sig.function_name.str());
        ++i;
      }
    };
    (check(args), ...);
    if (payload_finder<Args...>::type != sig.input_payload_type && payload_finder<Args...>::count == 1)
      throw std::invalid_argument("PrepareRequest: payload kind mismatch for " + sig.function_name.str());
    RpcRequestBuilderOptions o = opt;
    o.function_id = sig.id;
    return PrepareRequest(o, std::forward<Args>(args)...);
  }
  // Dynamic form: parameters already packed.
  RpcRequestHeader PrepareRequest(const RpcRequestBuilderOptions& opt, data::vector<ParamMeta>&& params) const {
    RpcRequestHeader h = base(opt);
    h.params = std::move(params);
    return h;
  }

 private:
  static RpcRequestHeader base(const RpcRequestBuilderOptions& opt) {
    RpcRequestHeader h;
    h.session_id = opt.session_id;
    h.request_id = opt.request_id;
    h.function_id = opt.function_id;
    h.hlc = opt.hlc;
    h.workflow_id = opt.workflow_id;
    return h;
  }
};

}  // namespace eux::rpc
