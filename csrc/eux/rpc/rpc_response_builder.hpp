// RpcResponseBuilder: packs result values into an RpcResponseHeader; a payload
// among the results is returned beside the header
// (reference: rpc_core/rpc_response_builder.hpp:88-164).
#pragma once

#include <utility>

#include "eux/rpc/rpc_traits.hpp"

namespace eux::rpc {

class RpcResponseBuilder {
 public:
  RpcResponseBuilder() = default;
  explicit RpcResponseBuilder(HybridLogicalClock hlc, workflow_id_t wf = workflow_id_t{}) : hlc_(hlc), workflow_id_(wf) {}

  // No payload among the results: returns the header.
  template <class... Results>
    requires(payload_finder<Results...>::count == 0)
  RpcResponseHeader PrepareResponse(session_id_t session, request_id_t request, Results&&... results) const {
    RpcResponseHeader h = base(session, request);
    (h.results.emplace_back(std::forward<Results>(results)), ...);
    return h;
  }
  // One payload among the results: returns {header, payload}.
  template <class... Results>
    requires(payload_finder<Results...>::count == 1)
  auto PrepareResponse(session_id_t session, request_id_t request, Results&&... results) const {
    RpcResponseHeader h = base(session, request);
    PayloadVariant payload;
    auto one = [&](auto&& r) {
      using R = decltype(r);
      if constexpr (is_payload_v<R>) payload = std::move(r);
      else if constexpr (is_payload_variant_v<R>) payload = std::move(r);
      else h.results.emplace_back(std::forward<R>(r));
    };
    (one(std::forward<Results>(results)), ...);
    return std::pair<RpcResponseHeader, PayloadVariant>(std::move(h), std::move(payload));
  }
  // Dynamic form: results already packed.
  RpcResponseHeader PrepareResponse(session_id_t session, request_id_t request, data::vector<ParamMeta>&& results) const {
    RpcResponseHeader h = base(session, request);
    h.results = std::move(results);
    return h;
  }
  RpcResponseHeader PrepareError(session_id_t session, request_id_t request, std::error_code ec, std::string_view what) const {
    RpcResponseHeader h = base(session, request);
    h.status = RpcStatus(ec);
    h.results.emplace_back(data::string(what));
    return h;
  }
  void set_hlc(HybridLogicalClock h) { hlc_ = h; }
  void set_workflow_id(workflow_id_t w) { workflow_id_ = w; }

 private:
  RpcResponseHeader base(session_id_t session, request_id_t request) const {
    RpcResponseHeader h;
    h.session_id = session;
    h.request_id = request;
    h.hlc = hlc_;
    h.workflow_id = workflow_id_;
    return h;
  }
  HybridLogicalClock hlc_{};
  workflow_id_t workflow_id_{};
};

}  // namespace eux::rpc
