// Internals shared by the translation units of AxonWorker: payload views,
// header serialisation into owned memory, outgoing message assembly, and the
// per-request state of the server and client pipelines.
#pragma once

#include "eux/axon/axon_worker.hpp"
#include "eux/ucxx/cuda/ucx_cuda_context.hpp"

namespace eux::axon {

namespace detail {
namespace ex = eux::exec;
using rpc::PayloadVariant;
using rpc::RpcErrc;
using rpc::RpcRequestHeader;
using rpc::RpcResponseHeader;
using ucxx::UcxBuffer;
using ucxx::UcxBufferVec;
using ucxx::UcxHeader;

inline std::unique_ptr<ucxx::UcxAutoDeviceContext> clone_device_context(int device_id) {
  if (device_id < 0) return std::make_unique<ucxx::UcxAutoDefaultDeviceContext>();
  return std::make_unique<ucxx::UcxAutoCudaDeviceContext>(device_id);
}

// non-owning views of a payload (the original must outlive them)
inline PayloadVariant view_of(PayloadVariant& p) {
  if (auto* b = std::get_if<UcxBuffer>(&p)) return UcxBuffer(b->mr(), b->type(), b->data(), b->size(), b->mem_h(), false);
  if (auto* v = std::get_if<UcxBufferVec>(&p)) return UcxBufferVec(v->mr(), v->type(), v->buffers(), v->mem_h(), false);
  return {};
}

inline std::vector<size_t> sizes_of(utils::TensorMetaSpan metas) {
  std::vector<size_t> out;
  out.reserve(metas.size());
  for (auto& m : metas) out.push_back(rpc::utils::TensorPayloadBytes(m));
  return out;
}

// serialise a header into memory owned by an UcxHeader
template <class H>
UcxHeader serialize_header(ucxx::UcxMemoryResourceManager& mr, const H& h) {
  const size_t n = rpc::GetSerializedSize(h);
  UcxHeader out(mr, n);
  rpc::FixedBufferWriter w(out.data(), n);
  rpc::SerializeInto(w, h);
  return out;
}

// Build the message for connection_send: header owned, payload viewed.
struct OutMessage {
  std::optional<ucxx::UcxAmData> data;
  std::optional<ucxx::UcxAmIovec> iovec;
};
inline OutMessage make_message(ucxx::UcxMemoryResourceManager& mr, UcxHeader&& header, PayloadVariant& payload) {
  OutMessage m;
  if (auto* v = std::get_if<UcxBufferVec>(&payload); v && v->size() > 0) {
    ucx_am_iovec raw{};
    raw.header = header.release();
    raw.buffer_vec = v->buffers().data();
    raw.buffer_count = v->size();
    raw.buffer_type = v->type();
    raw.mem_h = v->mem_h();
    m.iovec.emplace(mr, std::move(raw), true, false);
  } else {
    ucx_am_data raw{};
    raw.header = header.release();
    raw.buffer_type = ucx_memory_type::HOST;
    if (auto* b = std::get_if<UcxBuffer>(&payload)) {
      raw.buffer = {b->data(), b->size()};
      raw.buffer_type = b->type();
      raw.mem_h = b->mem_h();
    }
    m.data.emplace(mr, std::move(raw), true, false);
  }
  return m;
}

// The remarks a payload carries for the transport, filed with the context under the message's header.
inline void attach_send_attr(ucxx::ucx_am_context& ctx, const OutMessage& m, const PayloadVariant& payload) {
  std::shared_ptr<const ucxx::UcxSendAttr> attr;
  if (auto* b = std::get_if<UcxBuffer>(&payload)) attr = b->send_attr();
  else if (auto* v = std::get_if<UcxBufferVec>(&payload)) attr = v->send_attr();
  if (!attr) return;
  const void* header = m.iovec ? m.iovec->get()->header.data : (m.data ? m.data->get()->header.data : nullptr);
  ctx.attach_send_attr(header, std::move(attr));
}

inline std::exception_ptr rpc_error(std::error_code ec, std::string what = {}) {
  return std::make_exception_ptr(rpc::RpcException(ec, std::move(what)));
}

}  // namespace detail

// One request on the server side.
struct ServerCall {
  uint64_t conn_id = 0;
  rpc::RpcRequestHeader req;
  rpc::PayloadVariant payload;
  std::shared_ptr<utils::AxonRequest> retained;  // set when a retention policy looked at the request
  std::optional<size_t> rndv_key;
  rpc::RpcFunctionSignature signature;
  ServerMemoryPolicy mem;
  MessageLifecyclePolicy lifecycle;
  metrics::RpcMetricsContext mctx;
  bool respond = true;
};

// One call on the client side, shared between the sender, the send continuation and the response path.
struct ClientCall {
  uint64_t conn_id = 0;
  uint32_t request_id = 0, session_id = 0, function_id = 0;
  std::optional<ucxx::UcxHeader> header_bytes;
  rpc::PayloadVariant payload;
  ClientMemoryPolicy mem;
  std::optional<detail::OutMessage> out;
  // set by the operation state
  std::function<void(InvokeResult&&)> finish_value;
  std::function<void(std::exception_ptr)> finish_error;
  // response being completed
  rpc::RpcResponseHeader response;
  std::optional<size_t> rndv_key;
};

}  // namespace eux::axon
