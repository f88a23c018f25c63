// AxonMessage: an RPC header together with its payload, with tensor views over
// the payload described by the header's TENSOR_META / TENSOR_META_VEC parameter
// (reference: axon/include/axon/utils/axon_message.hpp, axon/src/utils/axon_message.cpp).
#pragma once

#include <optional>
#include <stdexcept>
#include <vector>

#include "eux/axon/utils/tensor.hpp"
#include "eux/rpc/rpc_payload_types.hpp"
#include "eux/rpc/rpc_types.hpp"

namespace eux::axon::utils {

using rpc::PayloadVariant;
using rpc::RpcRequestHeader;
using rpc::RpcResponseHeader;
using AxonMessageID = uint64_t;
using TensorMetaSpan = rpc::utils::TensorMetaSpan;

// index of the (single) tensor parameter, if any; two of them are an error
template <class Params>
std::optional<size_t> ExtractTensorParamIndex(const Params& params) {
  std::optional<size_t> idx;
  for (size_t i = 0; i < params.size(); ++i) {
    if (params[i].type == rpc::ParamType::TENSOR_META || params[i].type == rpc::ParamType::TENSOR_META_VEC) {
      if (idx) throw std::runtime_error("more than one tensor parameter: only one TENSOR_META or TENSOR_META_VEC is allowed");
      idx = i;
    }
  }
  return idx;
}
// The tensor metadata of a message; scanned from the back because senders append it last.
template <class Params>
TensorMetaSpan GetTensorMetas(const Params& params) noexcept {
  for (size_t i = params.size(); i-- > 0;) {
    const auto& p = params[i];
    if (p.type == rpc::ParamType::TENSOR_META_VEC) {
      const auto& v = std::get<rpc::TensorMetaVec>(p.value);
      return TensorMetaSpan{v.data(), v.size()};
    }
    if (p.type == rpc::ParamType::TENSOR_META) return TensorMetaSpan{&std::get<rpc::TensorMeta>(p.value), 1};
  }
  return {};
}

template <class HeaderType>
struct AxonMessage {
  HeaderType header;
  PayloadVariant payload;

  AxonMessage(HeaderType&& h, PayloadVariant&& p) : header(std::move(h)), payload(std::move(p)) {
    tensor_param_index_ = ExtractTensorParamIndex(header.GetParamsContainer());
  }
  AxonMessage(HeaderType&& h, PayloadVariant&& p, std::optional<size_t> tensor_param_index)
      : header(std::move(h)), payload(std::move(p)), tensor_param_index_(tensor_param_index) {}
  AxonMessage(const AxonMessage&) = delete;
  AxonMessage& operator=(const AxonMessage&) = delete;
  AxonMessage(AxonMessage&&) = default;
  AxonMessage& operator=(AxonMessage&&) = default;

  size_t GetTensorCount() const { return GetTensorMetas(header.GetParamsContainer()).size(); }
  std::optional<size_t> GetTensorParamIndex() const { return tensor_param_index_; }
  const PayloadVariant& GetPayload() const { return payload; }
  PayloadVariant& GetPayload() { return payload; }

  // View of tensor i: over segment i of a buffer vector, or at its running offset in a single buffer.
  Tensor<> GetTensor(size_t i) {
    auto metas = GetTensorMetas(header.GetParamsContainer());
    if (i >= metas.size()) throw std::out_of_range("tensor index out of range");
    if (auto* vec = std::get_if<ucxx::UcxBufferVec>(&payload)) {
      if (i >= vec->size()) throw std::out_of_range("the payload has fewer segments than tensors");
      return Tensor<>((*vec)[i].data, metas[i]);
    }
    if (auto* buf = std::get_if<ucxx::UcxBuffer>(&payload)) {
      size_t off = 0;
      for (size_t k = 0; k < i; ++k) off += rpc::utils::TensorPayloadBytes(metas[k]);
      if (off + rpc::utils::TensorPayloadBytes(metas[i]) > buf->size()) throw std::out_of_range("the payload is smaller than its tensors");
      return Tensor<>(static_cast<char*>(buf->data()) + off, metas[i]);
    }
    throw std::runtime_error("the message has no payload");
  }
  std::vector<Tensor<>> GetTensorVec() {
    std::vector<Tensor<>> out;
    const size_t n = GetTensorCount();
    out.reserve(n);
    for (size_t i = 0; i < n; ++i) out.push_back(GetTensor(i));
    return out;
  }

 private:
  std::optional<size_t> tensor_param_index_;
};

using ArrivalRequest = AxonMessage<RpcRequestHeader>;
using ArrivalResponse = AxonMessage<RpcResponseHeader>;
using AxonRequest = ArrivalRequest;
using AxonResponse = ArrivalResponse;

}  // namespace eux::axon::utils
