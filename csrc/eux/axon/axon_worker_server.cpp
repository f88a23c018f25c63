// Server pipeline of AxonWorker (reference: axon/src/axon_worker.cpp:522-1413).
#include <ctime>

#include "eux/axon/axon_worker_detail.hpp"
#include "eux/ucxx/nvtx_range.hpp"
#include "eux/ucxx/ucx_context_logger.hpp"

namespace eux::axon {

using namespace eux::axon::detail;

void AxonWorker::ServerLoopStart() {
  auto sched = server_ctx_->get_scheduler();
  auto* stop = server_loop_stop_.get();
  // one header at a time; everything after the header runs detached so the loop keeps receiving
  auto one = ex::defer([this, sched] {
    return ex::upon_error(ex::then(ucxx::connection_recv_header(sched), [this](ucxx::recv_header_result_t arrival) { ServerHandleArrival(std::move(arrival)); }),
                          [this](std::exception_ptr e) { UCX_CTX_WARN << name_ << ": receive failed: " << ex::what_of(e); });
  });
  server_scope_->spawn_detached(ex::with_query_value(ex::repeat_effect_until(std::move(one), [stop] { return stop->stop_requested(); }),
                                                    ex::get_stop_token, stop->get_token()));
}

void AxonWorker::ServerSendError(uint64_t conn_id, const RpcRequestHeader& req, std::error_code ec, std::string_view what) {
  server_pipe_failed_.fetch_add(1);
  errors::AxonErrorContext ectx;
  ectx.conn_id = conn_id;
  ectx.session_id = req.session_id.v_;
  ectx.request_id = req.request_id.v_;
  ectx.function_id = req.function_id.v_;
  ectx.status = rpc::RpcStatus(ec);
  ectx.what = std::string(what);
  ectx.hlc = req.hlc;
  ectx.workflow_id = req.workflow_id.v_;
  ReportError(std::move(ectx));
  auto call = std::make_shared<ServerCall>();
  call->conn_id = conn_id;
  call->req = req;
  rpc::RpcResponseBuilder b(TickHlc(), req.workflow_id);
  ServerSendResponse(std::move(call), b.PrepareError(req.session_id, req.request_id, ec, what), PayloadVariant{});
}

// Runs on the server context's thread.
void AxonWorker::ServerHandleArrival(ucxx::recv_header_result_t&& arrival) {
  auto call = std::make_shared<ServerCall>();
  const void* hdr_data = nullptr;
  size_t hdr_size = 0;
  std::optional<UcxBuffer> eager;
  if (arrival.index() == 0) {
    auto& [key, header] = std::get<0>(arrival);
    call->rndv_key = key;
    if (const auto* d = server_ctx_->view_pending_am_desc(key)) call->conn_id = d->conn_id;
    hdr_data = header.data();
    hdr_size = header.size();
  } else {
    auto& bundle = std::get<1>(arrival);
    call->conn_id = bundle.conn_id();
    hdr_data = bundle.header().data();
    hdr_size = bundle.header().size();
    if (bundle.buffer().size() > 0) eager.emplace(bundle.move_buffer());
  }
  auto drop_rndv = [&] {
    if (call->rndv_key) server_ctx_->release_rndv_am_desc(*call->rndv_key);
  };
  try {
    call->req = rpc::Deserialize<RpcRequestHeader>(hdr_data, hdr_size);
  } catch (const std::exception& e) {
    drop_rndv();
    server_pipe_failed_.fetch_add(1);
    errors::AxonErrorContext ectx;
    ectx.conn_id = call->conn_id;
    ectx.status = rpc::RpcStatus(errors::make_error_code(errors::AxonErrc::DeserializeError));
    ectx.what = std::string("request header could not be parsed: ") + e.what();
    ReportError(std::move(ectx));
    return;
  }
  MergeHlc(call->req.hlc);
  server_pipe_invoked_.fetch_add(1);

  // back-pressure gate
  if (reject_messages_.load()) {
    BypassRejectionFunction bypass;
    {
      std::lock_guard lk(hooks_mu_);
      bypass = bypass_fn_;
    }
    if (!(bypass && bypass(call->req))) {
      drop_rndv();
      {
        std::lock_guard lk(rejected_mu_);
        rejected_info_.emplace_back(call->conn_id, std::time(nullptr));
        if (rejected_info_.size() > 1024) rejected_info_.erase(rejected_info_.begin(), rejected_info_.begin() + 512);
      }
      ServerSendError(call->conn_id, call->req, errors::make_error_code(errors::AxonErrc::StorageBackpressure),
                      "the worker is rejecting messages (storage back-pressure)");
      return;
    }
  }
  auto sig = dispatcher_.GetSignature(call->req.function_id);
  if (!sig) {
    drop_rndv();
    ServerSendError(call->conn_id, call->req, rpc::make_error_code(RpcErrc::NOT_FOUND),
                    "function " + std::to_string(call->req.function_id.v_) + " is not registered on worker " + name_);
    return;
  }
  call->signature = *sig;
  if (auto pol = FindPolicies(call->req.function_id)) {
    call->mem = pol->mem;
    call->lifecycle = pol->lifecycle;
  }
  call->mctx = {call->req.session_id.v_, call->req.request_id.v_, call->req.function_id.v_, sig->function_name.str(), call->req.hlc,
                call->req.workflow_id.v_};
  const bool wants_vec = sig->input_payload_type == rpc::PayloadType::UCX_BUFFER_VEC;
  auto metas = utils::GetTensorMetas(call->req.params);

  if (!call->rndv_key) {
    // eager: the payload is already here, in host memory
    if (eager) {
      if (wants_vec) {
        std::vector<size_t> sizes = sizes_of(metas);
        if (sizes.empty()) sizes.push_back(eager->size());
        try {
          call->payload = std::move(*eager).to_buffer_vec(sizes);
        } catch (const std::exception& e) {
          ServerSendError(call->conn_id, call->req, rpc::make_error_code(RpcErrc::INVALID_ARGUMENT), e.what());
          return;
        }
      } else {
        call->payload = std::move(*eager);
      }
    }
    ServerDispatch(std::move(call));
    return;
  }
  ServerRunRequest(std::move(call));
}

// Rendezvous: choose where the payload lands, receive it, then dispatch.
void AxonWorker::ServerRunRequest(std::shared_ptr<ServerCall> call) {
  ucxx::NvtxRange range("axon.server.receive_payload");
  auto sched = server_ctx_->get_scheduler();
  const size_t key = *call->rndv_key;
  const bool wants_vec = call->signature.input_payload_type == rpc::PayloadType::UCX_BUFFER_VEC;
  auto metas = utils::GetTensorMetas(call->req.params);
  const auto* desc = server_ctx_->view_pending_am_desc(key);
  const size_t total = desc ? desc->data_length : 0;
  auto fail = [this, call, key](std::exception_ptr e) {
    server_ctx_->release_rndv_am_desc(key);
    ServerSendError(call->conn_id, call->req, ex::error_code_of(e), "payload receive failed: " + ex::what_of(e));
  };
  const bool custom = !call->mem.on_host && (wants_vec ? bool(call->mem.buffer_vec_provider) : bool(call->mem.buffer_provider));
  if (wants_vec) {
    // buffers: from the user's provider (run on the pool: it is user code), or host memory sized by the metadata
    auto make = [this, call, metas, total, custom]() -> UcxBufferVec {
      if (custom) return call->mem.buffer_vec_provider(metas);
      std::vector<size_t> sizes = sizes_of(metas);
      if (sizes.empty()) sizes.push_back(total);
      return UcxBufferVec(*mr_, ucx_memory_type::HOST, sizes);
    };
    auto recv = [this, sched, key, call](UcxBufferVec& bufs) {
      return ex::then(ucxx::connection_recv_buffer(sched, key, std::move(bufs)), [this, call](ucxx::active_message_iovec_buffer_bundle b) {
        call->payload = b.move_buffer();
        ServerDispatch(call);
      });
    };
    if (custom && !call->mem.provider_inline)
      server_scope_->spawn_detached(ex::upon_error(ex::let_value(ex::on(pool_.get_scheduler(), ex::just_from(make)), recv), fail));
    else server_scope_->spawn_detached(ex::upon_error(ex::let_value(ex::just_from(make), recv), fail));
    return;
  }
  auto done = [this, call](ucxx::active_message_buffer_bundle b) {
    call->payload = b.move_buffer();
    ServerDispatch(call);
  };
  if (custom) {
    auto make = [call, metas, total]() -> UcxBuffer {
      if (!metas.empty()) return call->mem.buffer_provider(metas);
      // no tensor metadata in the header: describe the payload as `total` opaque bytes
      rpc::TensorMeta opaque;
      opaque.ndim = 1;
      opaque.dtype = {kDLUInt, 8, 1};
      opaque.shape = {static_cast<int64_t>(total)};
      opaque.strides = {1};
      return call->mem.buffer_provider(utils::TensorMetaSpan{&opaque, 1});
    };
    auto recv = [sched, key, done](UcxBuffer& buf) { return ex::then(ucxx::connection_recv_buffer(sched, key, std::move(buf)), done); };
    if (call->mem.provider_inline) server_scope_->spawn_detached(ex::upon_error(ex::let_value(ex::just_from(make), recv), fail));
    else server_scope_->spawn_detached(ex::upon_error(ex::let_value(ex::on(pool_.get_scheduler(), ex::just_from(make)), recv), fail));
  } else {
    server_scope_->spawn_detached(ex::upon_error(ex::then(ucxx::connection_recv_buffer(sched, key, ucx_memory_type::HOST), done), fail));
  }
}

// Lifecycle policy, handler on the pool under the deadline, response.
void AxonWorker::ServerDispatch(std::shared_ptr<ServerCall> call) {
  ucxx::NvtxRange range("axon.server.dispatch");
  PayloadVariant for_handler;
  if (auto* retention = std::get_if<RetentionPolicy>(&call->lifecycle); retention && *retention) {
    const utils::AxonMessageID id = call->req.hlc.Raw();
    call->retained = std::make_shared<utils::AxonRequest>(RpcRequestHeader(call->req), std::move(call->payload));
    LifecycleStatus st = LifecycleStatus::Error;
    try {
      st = (*retention)(call->retained, id);
    } catch (const std::exception& e) {
      UCX_CTX_WARN << name_ << ": lifecycle policy threw: " << e.what();
    }
    if (st == LifecycleStatus::Error) {
      ServerSendError(call->conn_id, call->req, rpc::make_error_code(RpcErrc::INTERNAL), "the message lifecycle policy reported an error");
      return;
    }
    if (st == LifecycleStatus::Preserve) storage_->emplace(call->retained, id);
    for_handler = view_of(call->retained->payload);  // the handler sees the stored bytes
  } else {
    for_handler = std::move(call->payload);
  }
  metrics::MetricsObserver obs;
  {
    std::lock_guard lk(hooks_mu_);
    obs = metrics_observer_;
  }
  if (obs) obs->OnDispatchStart(call->mctx, std::chrono::steady_clock::now());
  // The handler and the deadline race; the first one to finish answers, the other is ignored.
  // (A handler that blocks its pool thread cannot be interrupted, so the deadline must not wait for it.
  // The timer runs on the server context's loop, which no handler can block.)
  struct Race {
    std::atomic<bool> answered{false};
    ex::inplace_stop_source stop_timer;
  };
  auto race = std::make_shared<Race>();
  auto payload_box = std::make_shared<PayloadVariant>(std::move(for_handler));
  const bool respond = call->respond;
  auto invoke = [this, call, payload_box] {
    rpc::RpcResponseBuilder b(TickHlc(), call->req.workflow_id);
    return dispatcher_.InvokeAsyncFunction(call->req, std::move(*payload_box), b);
  };
  auto finish = [this, call, obs, race, respond](rpc::RpcInvokeResult<rpc::ReturnedPayload> r) {
    if (race->answered.exchange(true)) return;
    race->stop_timer.request_stop();
    if (obs) obs->OnDispatchComplete(call->mctx, std::chrono::steady_clock::now());
    if (!r.header.status.ok()) {
      server_pipe_failed_.fetch_add(1);
      errors::AxonErrorContext ectx{call->conn_id, call->req.session_id.v_, call->req.request_id.v_, call->req.function_id.v_, r.header.status,
                                    r.header.results.empty() || r.header.results[0].type != rpc::ParamType::STRING ? std::string("handler failed")
                                                                                                                     : r.header.GetString(0).str(),
                                    call->req.hlc, call->req.workflow_id.v_};
      ReportError(std::move(ectx));
    }
    if (respond) ServerSendResponse(call, std::move(r.header), std::move(r.payload));
  };
  auto on_error = [this, call, race, respond](std::exception_ptr e) {
    if (race->answered.exchange(true)) return;
    race->stop_timer.request_stop();
    if (respond) ServerSendError(call->conn_id, call->req, rpc::make_error_code(RpcErrc::INTERNAL), ex::what_of(e));
  };
  auto on_done = [this, call, race, respond] {
    if (race->answered.exchange(true)) return;
    race->stop_timer.request_stop();
    if (respond) ServerSendError(call->conn_id, call->req, rpc::make_error_code(RpcErrc::CANCELLED), "the server is stopping");
  };
  auto on_deadline = [this, call, obs, race, respond] {
    if (race->answered.exchange(true)) return;
    if (obs) obs->OnDispatchComplete(call->mctx, std::chrono::steady_clock::now());
    if (respond)
      ServerSendError(call->conn_id, call->req, rpc::make_error_code(RpcErrc::DEADLINE_EXCEEDED), "the handler did not finish before the deadline");
  };
  if (call->mem.handler_inline)
    server_scope_->spawn_detached(ex::upon_done(ex::upon_error(ex::then(ex::defer(invoke), finish), on_error), on_done));
  else
    server_scope_->spawn_detached(
        ex::upon_done(ex::upon_error(ex::then(ex::on(pool_.get_scheduler(), ex::defer(invoke)), finish), on_error), on_done));
  server_scope_->spawn_detached(ex::upon_done(
      ex::with_query_value(ex::then(ex::schedule_after(server_ctx_->get_scheduler(), GetTimeout()), on_deadline), ex::get_stop_token,
                           race->stop_timer.get_token()),
      [race] {}));
}

void AxonWorker::ServerSendResponse(std::shared_ptr<ServerCall> call, RpcResponseHeader&& header, PayloadVariant&& payload) {
  ucxx::NvtxRange range("axon.server.send_response");
  if (!server_ctx_) return;
  header.session_id = call->req.session_id;
  header.request_id = call->req.request_id;
  if (header.hlc.Raw() == 0) header.hlc = TickHlc();
  header.workflow_id = call->req.workflow_id;
  auto sched = server_ctx_->get_scheduler();
  struct Out {
    PayloadVariant payload;
    OutMessage msg;
  };
  auto out = std::make_shared<Out>();
  out->payload = std::move(payload);
  try {
    auto image = serialize_header(*mr_, header);
    if (image.size() > ucxx::transport::kMaxHeaderLen) {
      // results too large for a message header (they belong in a payload): the caller hears that, at once,
      // instead of waiting for its deadline
      server_pipe_failed_.fetch_add(1);
      RpcResponseHeader err = rpc::RpcResponseBuilder{}.PrepareError(
          call->req.session_id, call->req.request_id, rpc::make_error_code(RpcErrc::RESOURCE_EXHAUSTED),
          "the response header is " + std::to_string(image.size()) + " bytes; a message carries at most " +
              std::to_string(ucxx::transport::kMaxHeaderLen) + " (large results belong in a tensor payload)");
      err.hlc = header.hlc;
      err.workflow_id = header.workflow_id;
      out->payload = PayloadVariant{};
      image = serialize_header(*mr_, err);
    }
    out->msg = make_message(*mr_, std::move(image), out->payload);
    attach_send_attr(*server_ctx_, out->msg, out->payload);
  } catch (const std::exception& e) {
    server_pipe_failed_.fetch_add(1);
    UCX_CTX_ERROR << name_ << ": response could not be serialised: " << e.what();
    return;
  }
  const uint64_t conn = call->conn_id;
  auto after = [out, call] {};  // keeps payload and request alive until the bytes are out
  auto failed = [this, out, call, conn](std::exception_ptr e) {
    server_pipe_failed_.fetch_add(1);
    errors::AxonErrorContext ectx;
    ectx.conn_id = conn;
    ectx.session_id = call->req.session_id.v_;
    ectx.request_id = call->req.request_id.v_;
    ectx.function_id = call->req.function_id.v_;
    ectx.status = rpc::RpcStatus(errors::make_error_code(errors::AxonErrc::RemoteRespondError));
    ectx.what = "response could not be sent: " + ex::what_of(e);
    ReportError(std::move(ectx));
  };
  if (out->msg.iovec) server_scope_->spawn_detached(ex::upon_error(ex::then(ucxx::connection_send(sched, conn, *out->msg.iovec->get()), after), failed));
  else server_scope_->spawn_detached(ex::upon_error(ex::then(ucxx::connection_send(sched, conn, *out->msg.data->get()), after), failed));
}

// ---- retained requests ---------------------------------------------------------------------
size_t AxonWorker::ProcessStoredRequests() {
  size_t n = 0;
  for (auto& [id, req] : storage_->snapshot()) {
    if (!dispatcher_.IsRegistered(req->header.function_id)) continue;
    rpc::RpcResponseBuilder b(TickHlc(), req->header.workflow_id);
    PayloadVariant view = view_of(req->payload);
    try {
      (void)ex::sync_wait(dispatcher_.InvokeAsyncFunction(req->header, std::move(view), b));
      ++n;
    } catch (const std::exception& e) {
      UCX_CTX_WARN << name_ << ": stored request " << id << " failed: " << e.what();
    }
  }
  return n;
}

size_t AxonWorker::ProcessStoredRequests(const StoredRequestVisitor& visitor) {
  size_t n = 0;
  for (auto& [id, req] : storage_->snapshot()) {
    LifecycleStatus st = visitor(req, id);
    ++n;
    if (st == LifecycleStatus::Discard) storage_->erase(id);
  }
  return n;
}

}  // namespace eux::axon
