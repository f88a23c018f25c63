// Client pipeline of AxonWorker: endpoints, InvokeRpc, response handling
// (reference: axon/include/axon/axon_worker.hpp:1052-1208, axon/src/axon_worker.cpp:1424-1667).
#include "eux/axon/axon_worker_detail.hpp"
#include "eux/ucxx/nvtx_range.hpp"
#include "eux/ucxx/ucx_context_logger.hpp"

namespace eux::axon {

using namespace eux::axon::detail;

// ---- endpoints ----------------------------------------------------------------------------
exec::any_sender_of<uint64_t> AxonWorker::ConnectEndpointAsync(std::vector<std::byte> address, std::string worker_name) {
  if (!client_ctx_) return ex::just_error<uint64_t>(errors::make_error_code(errors::AxonErrc::WorkerStartFailed));
  auto sched = client_ctx_->get_scheduler();
  return ex::then(ucxx::connect_endpoint(sched, std::move(address)), [this, worker_name](ucxx::conn_id_t conn) -> uint64_t {
    std::lock_guard lk(endpoints_mu_);
    auto it = endpoint_by_name_.find(worker_name);
    if (it != endpoint_by_name_.end()) {
      endpoints_.modify(it->second, [&](RemoteEndpoint& e) { e.conn_id = conn; });
    } else {
      endpoint_by_name_[worker_name] = endpoints_.emplace(RemoteEndpoint{worker_name, conn, {}});
    }
    return conn;
  });
}

uint64_t AxonWorker::ConnectEndpoint(std::vector<std::byte> address, std::string worker_name) {
  auto r = ex::sync_wait(ConnectEndpointAsync(std::move(address), std::move(worker_name)));
  if (!r) throw rpc::RpcException(errors::make_error_code(errors::AxonErrc::ConnectError), "connect was cancelled");
  return *r;
}

bool AxonWorker::RegisterEndpointSignatures(std::string_view worker_name, const void* data, size_t size) {
  rpc::data::vector<rpc::RpcFunctionSignature> sigs;
  try {
    sigs = rpc::RpcDispatcher::DeserializeSignatures(data, size);
  } catch (const std::exception&) {
    return false;
  }
  std::lock_guard lk(endpoints_mu_);
  auto it = endpoint_by_name_.find(std::string(worker_name));
  if (it == endpoint_by_name_.end()) it = endpoint_by_name_.emplace(std::string(worker_name), endpoints_.emplace(RemoteEndpoint{std::string(worker_name), 0, {}})).first;
  return endpoints_.modify(it->second, [&](RemoteEndpoint& e) {
    for (auto& s : sigs) e.signatures[s.id.v_] = s;
  });
}

std::optional<rpc::RpcFunctionSignature> AxonWorker::GetEndpointSignature(std::string_view worker_name, rpc::function_id_t id) const {
  std::lock_guard lk(endpoints_mu_);
  auto it = endpoint_by_name_.find(std::string(worker_name));
  if (it == endpoint_by_name_.end()) return std::nullopt;
  auto r = endpoints_.access(it->second, [&](const RemoteEndpoint& e) -> std::optional<rpc::RpcFunctionSignature> {
    auto s = e.signatures.find(id.v_);
    if (s == e.signatures.end()) return std::nullopt;
    return s->second;
  });
  return r ? *r : std::nullopt;
}

std::optional<uint64_t> AxonWorker::GetConnectionId(std::string_view worker_name) const {
  std::lock_guard lk(endpoints_mu_);
  auto it = endpoint_by_name_.find(std::string(worker_name));
  if (it == endpoint_by_name_.end()) return std::nullopt;
  auto r = endpoints_.access(it->second, [](const RemoteEndpoint& e) { return e.conn_id; });
  if (!r || *r == 0) return std::nullopt;
  return *r;
}

std::optional<AxonWorker::WorkerKey> AxonWorker::GetWorkerKey(std::string_view worker_name) const {
  std::lock_guard lk(endpoints_mu_);
  auto it = endpoint_by_name_.find(std::string(worker_name));
  if (it == endpoint_by_name_.end()) return std::nullopt;
  return it->second;
}

std::optional<uint64_t> AxonWorker::GetConnectionId(WorkerKey key) const {
  auto r = endpoints_.access(key, [](const RemoteEndpoint& e) { return e.conn_id; });
  if (!r || *r == 0) return std::nullopt;
  return *r;
}

std::optional<std::string> AxonWorker::GetWorkerName(WorkerKey key) const {
  return endpoints_.access(key, [](const RemoteEndpoint& e) { return e.name; });
}

bool AxonWorker::DisconnectEndpoint(std::string_view worker_name) {
  std::optional<uint64_t> conn = GetConnectionId(worker_name);
  {
    std::lock_guard lk(endpoints_mu_);
    auto it = endpoint_by_name_.find(std::string(worker_name));
    if (it == endpoint_by_name_.end()) return false;
    endpoints_.erase(it->second);
    endpoint_by_name_.erase(it);
  }
  if (conn && client_ctx_) {
    auto* ctx = client_ctx_.get();
    ex::sync_wait(ex::then(ctx->get_scheduler().schedule(), [ctx, c = *conn] {
      ctx->connections().disconnect(c);
      ctx->connections().reap_disconnected();
    }));
  }
  return true;
}

// ---- the receive loop -------------------------------------------------------------------------
void AxonWorker::ClientLoopStart() {
  auto sched = client_ctx_->get_scheduler();
  auto* stop = client_loop_stop_.get();
  auto one = ex::defer([this, sched] {
    return ex::upon_error(ex::then(ucxx::connection_recv_header(sched), [this](ucxx::recv_header_result_t arrival) { ClientHandleArrival(std::move(arrival)); }),
                          [this](std::exception_ptr e) { UCX_CTX_WARN << name_ << ": client receive failed: " << ex::what_of(e); });
  });
  client_scope_->spawn_detached(ex::with_query_value(ex::repeat_effect_until(std::move(one), [stop] { return stop->stop_requested(); }),
                                                    ex::get_stop_token, stop->get_token()));
}

// Runs on the client context's thread: match the response with its pending call.
void AxonWorker::ClientHandleArrival(ucxx::recv_header_result_t&& arrival) {
  ResponseArrival r;
  const void* hdr_data = nullptr;
  size_t hdr_size = 0;
  if (arrival.index() == 0) {
    auto& [key, header] = std::get<0>(arrival);
    r.rndv_key = key;
    if (const auto* d = client_ctx_->view_pending_am_desc(key)) r.conn_id = d->conn_id;
    hdr_data = header.data();
    hdr_size = header.size();
  } else {
    auto& bundle = std::get<1>(arrival);
    r.conn_id = bundle.conn_id();
    hdr_data = bundle.header().data();
    hdr_size = bundle.header().size();
    if (bundle.buffer().size() > 0) r.eager.emplace(bundle.move_buffer());
  }
  auto drop_rndv = [&] {
    if (r.rndv_key) client_ctx_->release_rndv_am_desc(*r.rndv_key);
  };
  try {
    r.header = rpc::Deserialize<RpcResponseHeader>(hdr_data, hdr_size);
  } catch (const std::exception& e) {
    drop_rndv();
    client_pipe_failed_.fetch_add(1);
    errors::AxonErrorContext ectx;
    ectx.conn_id = r.conn_id;
    ectx.status = rpc::RpcStatus(errors::make_error_code(errors::AxonErrc::DeserializeError));
    ectx.what = std::string("response header could not be parsed: ") + e.what();
    ReportError(std::move(ectx));
    return;
  }
  MergeHlc(r.header.hlc);
  const uint32_t session = r.header.session_id.v_;
  auto pending = pending_rpcs_.take_if(r.header.request_id.v_, [session](const PendingRpc& p) { return p.session_id == session; });
  if (!pending) {  // nobody waits any more (deadline passed, cancelled)
    drop_rndv();
    return;
  }
  pending->complete(std::move(r), nullptr);
}

// ---- InvokeRpc ------------------------------------------------------------------------------------
// The operation: publish the call in the pending table, send, and complete exactly once, by
// whoever removes the table entry (response, send failure, stop request, client shutdown).
struct AxonWorker::invoke_sender {
  using value_type = InvokeResult;
  AxonWorker* w;
  std::shared_ptr<ClientCall> call;

  template <class R>
  struct op {
    struct stop_fn {
      op* o;
      void operator()() const noexcept {
        if (auto p = o->w->pending_rpcs_.take(o->id)) p->complete(std::nullopt, nullptr);  // null error = cancelled
      }
    };
    using stop_cb_t = typename ex::stop_token_of_t<R>::template callback_type<stop_fn>;
    AxonWorker* w;
    std::shared_ptr<ClientCall> call;
    R r;
    uint32_t id;
    std::optional<stop_cb_t> stop_cb;

    op(AxonWorker* w_, std::shared_ptr<ClientCall> c, R&& r_) : w(w_), call(std::move(c)), r(std::move(r_)), id(call->request_id) {}
    op(op&&) = delete;

    void start() noexcept {
      // what completes the operation, from whichever thread owns the table entry
      call->finish_value = [this](InvokeResult&& v) {
        stop_cb.reset();
        // the caller reads the response's tensors by their descriptions: they must lie inside the payload that came
        if (!rpc::RpcDispatcher::TensorsFitPayload(v.header.results, std::get_if<ucxx::UcxBuffer>(&v.payload), std::get_if<ucxx::UcxBufferVec>(&v.payload))) {
          r.set_error(rpc_error(rpc::make_error_code(RpcErrc::INVALID_ARGUMENT), "the response's tensor metadata describes more bytes than its payload holds"));
          return;
        }
        r.set_value(std::move(v));
      };
      call->finish_error = [this](std::exception_ptr e) {
        stop_cb.reset();
        if (e) r.set_error(std::move(e));
        else r.set_done();
      };
      AxonWorker* worker = w;
      std::shared_ptr<ClientCall> c = call;
      auto tok = ex::get_stop_token(r);
      stop_cb.emplace(tok, stop_fn{this});
      PendingRpc entry;
      entry.session_id = c->session_id;
      entry.complete = [worker, c](std::optional<ResponseArrival>&& arrival, std::exception_ptr err) {
        if (!arrival) {
          c->finish_error(std::move(err));
          return;
        }
        c->response = std::move(arrival->header);
        if (arrival->rndv_key) {
          c->rndv_key = arrival->rndv_key;
          worker->ClientFinishWithPayload(c);
        } else {
          InvokeResult res{std::move(c->response), PayloadVariant{}};
          if (arrival->eager) res.payload = std::move(*arrival->eager);
          c->finish_value(std::move(res));
        }
      };
      const uint32_t rid = id;
      if (!worker->pending_rpcs_.emplace(rid, std::move(entry))) {
        stop_cb.reset();
        r.set_error(rpc_error(rpc::make_error_code(RpcErrc::RESOURCE_EXHAUSTED),
                              "too many calls in flight: the slot of this request id is taken"));
        return;
      }
      // From here on the operation may complete on another thread at any moment: only locals are used.
      if (tok.stop_requested()) {
        if (auto p = worker->pending_rpcs_.take(rid)) p->complete(std::nullopt, nullptr);
        return;
      }
      auto sched = worker->client_ctx_->get_scheduler();
      auto sent = [c] {};
      auto send_failed = [worker, c, rid](std::exception_ptr e) {
        worker->client_pipe_failed_.fetch_add(1);
        if (auto p = worker->pending_rpcs_.take(rid))
          p->complete(std::nullopt, rpc_error(ex::error_code_of(e), "request could not be sent: " + ex::what_of(e)));
      };
      try {
        if (c->out->iovec) worker->client_scope_->spawn_detached(ex::upon_error(ex::then(ucxx::connection_send(sched, c->conn_id, *c->out->iovec->get()), sent), send_failed));
        else worker->client_scope_->spawn_detached(ex::upon_error(ex::then(ucxx::connection_send(sched, c->conn_id, *c->out->data->get()), sent), send_failed));
      } catch (...) {
        send_failed(std::current_exception());
      }
    }
  };
  template <class R>
  auto connect(R&& r) && {
    return op<std::decay_t<R>>(w, std::move(call), std::decay_t<R>(std::forward<R>(r)));
  }
};

InvokeSender AxonWorker::InvokeRpc(std::string_view worker_name, RpcRequestHeader&& header, PayloadVariant&& payload, ClientMemoryPolicy mem_policy) {
  return InvokeOnConnection(GetConnectionId(worker_name), std::string(worker_name), std::move(header), std::move(payload), std::move(mem_policy));
}

InvokeSender AxonWorker::InvokeRpc(WorkerKey worker_key, RpcRequestHeader&& header, PayloadVariant&& payload, ClientMemoryPolicy mem_policy) {
  return InvokeOnConnection(GetConnectionId(worker_key), "key " + std::to_string(worker_key.index) + "/" + std::to_string(worker_key.generation),
                            std::move(header), std::move(payload), std::move(mem_policy));
}

InvokeSender AxonWorker::InvokeOnConnection(std::optional<uint64_t> conn, std::string whom, RpcRequestHeader&& header, PayloadVariant&& payload,
                                            ClientMemoryPolicy mem_policy) {
  ucxx::NvtxRange range("axon.client.invoke");
  if (!client_running_.load() || !client_ctx_)
    return ex::just_error<InvokeResult>(rpc_error(errors::make_error_code(errors::AxonErrc::WorkerStartFailed), "the client is not running"));
  if (!conn) return ex::just_error<InvokeResult>(rpc_error(errors::make_error_code(errors::AxonErrc::WorkerNotFound), "no endpoint named " + whom));
  auto call = std::make_shared<ClientCall>();
  call->conn_id = *conn;
  header.request_id = rpc::request_id_t{next_request_id_.fetch_add(1)};
  header.hlc = TickHlc();
  call->request_id = header.request_id.v_;
  call->session_id = header.session_id.v_;
  call->function_id = header.function_id.v_;
  call->payload = std::move(payload);
  call->mem = std::move(mem_policy);
  try {
    auto image = serialize_header(*mr_, header);
    if (image.size() > ucxx::transport::kMaxHeaderLen)
      return ex::just_error<InvokeResult>(rpc_error(rpc::make_error_code(RpcErrc::RESOURCE_EXHAUSTED),
                                                    "the request header is " + std::to_string(image.size()) + " bytes; a message carries at most " +
                                                        std::to_string(ucxx::transport::kMaxHeaderLen) + " (large arguments belong in a tensor payload)"));
    call->out.emplace(make_message(*mr_, std::move(image), call->payload));
    attach_send_attr(*client_ctx_, *call->out, call->payload);
  } catch (const std::exception& e) {
    return ex::just_error<InvokeResult>(rpc_error(errors::make_error_code(errors::AxonErrc::SerializeError), e.what()));
  }
  // deadline: done caused by the timer becomes DEADLINE_EXCEEDED, any other done stays a cancellation.
  // The timer lives on the client context's own loop, where the call completes too: arming and
  // withdrawing it costs a queue node, not a wake-up of another thread.
  auto timed_out = std::make_shared<std::atomic<bool>>(false);
  auto deadline = ex::then(ex::schedule_after(client_ctx_->get_scheduler(), GetTimeout()), [timed_out] { timed_out->store(true); });
  const uint32_t fid = call->function_id, sid = call->session_id;
  return ex::let_done(ex::stop_when(invoke_sender{this, std::move(call)}, std::move(deadline)), [timed_out, fid, sid]() -> InvokeSender {
    if (timed_out->load())
      return ex::just_error<InvokeResult>(rpc_error(rpc::make_error_code(RpcErrc::DEADLINE_EXCEEDED),
                                                    "no response before the deadline (function_id: " + std::to_string(fid) +
                                                        ") (session_id: " + std::to_string(sid) + ")"));
    return ex::just_done<InvokeResult>();
  });
}

// The response announced a rendezvous payload: receive it where the caller's policy says, then finish.
void AxonWorker::ClientFinishWithPayload(std::shared_ptr<ClientCall> call) {
  ucxx::NvtxRange range("axon.client.receive_payload");
  auto sched = client_ctx_->get_scheduler();
  const size_t key = *call->rndv_key;
  auto metas = utils::GetTensorMetas(call->response.results);
  const auto* desc = client_ctx_->view_pending_am_desc(key);
  const size_t total = desc ? desc->data_length : 0;
  // a response that describes its payload with a TENSOR_META_VEC is received as separate buffers
  bool meta_vec = false;
  for (auto& r : call->response.results) meta_vec = meta_vec || r.type == rpc::ParamType::TENSOR_META_VEC;
  const bool as_vec = call->mem.want_vec || meta_vec || (!call->mem.on_host && call->mem.buffer_vec_provider && !call->mem.buffer_provider);
  auto fail = [this, call, key](std::exception_ptr e) {
    client_pipe_failed_.fetch_add(1);
    client_ctx_->release_rndv_am_desc(key);
    call->finish_error(rpc_error(ex::error_code_of(e), "response payload could not be received: " + ex::what_of(e)));
  };
  if (as_vec) {
    const bool custom = !call->mem.on_host && bool(call->mem.buffer_vec_provider);
    auto make = [this, call, metas, total, custom]() -> UcxBufferVec {
      if (custom) return call->mem.buffer_vec_provider(metas);
      std::vector<size_t> sizes = sizes_of(metas);
      if (sizes.empty()) sizes.push_back(total);
      return UcxBufferVec(*mr_, ucx_memory_type::HOST, sizes);
    };
    auto recv = [sched, key, call](UcxBufferVec& bufs) {
      return ex::then(ucxx::connection_recv_buffer(sched, key, std::move(bufs)), [call](ucxx::active_message_iovec_buffer_bundle b) {
        call->finish_value(InvokeResult{std::move(call->response), PayloadVariant(b.move_buffer())});
      });
    };
    if (custom && !call->mem.provider_inline)
      client_scope_->spawn_detached(ex::upon_error(ex::let_value(ex::on(pool_.get_scheduler(), ex::just_from(make)), recv), fail));
    else client_scope_->spawn_detached(ex::upon_error(ex::let_value(ex::just_from(make), recv), fail));
    return;
  }
  auto done = [call](ucxx::active_message_buffer_bundle b) {
    call->finish_value(InvokeResult{std::move(call->response), PayloadVariant(b.move_buffer())});
  };
  if (!call->mem.on_host && call->mem.buffer_provider) {
    auto make = [call, metas, total]() -> UcxBuffer {
      if (!metas.empty()) return call->mem.buffer_provider(metas);
      rpc::TensorMeta opaque;
      opaque.ndim = 1;
      opaque.dtype = {kDLUInt, 8, 1};
      opaque.shape = {static_cast<int64_t>(total)};
      opaque.strides = {1};
      return call->mem.buffer_provider(utils::TensorMetaSpan{&opaque, 1});
    };
    auto recv = [sched, key, done](UcxBuffer& buf) { return ex::then(ucxx::connection_recv_buffer(sched, key, std::move(buf)), done); };
    if (call->mem.provider_inline) client_scope_->spawn_detached(ex::upon_error(ex::let_value(ex::just_from(make), recv), fail));
    else client_scope_->spawn_detached(ex::upon_error(ex::let_value(ex::on(pool_.get_scheduler(), ex::just_from(make)), recv), fail));
  } else {
    client_scope_->spawn_detached(ex::upon_error(ex::then(ucxx::connection_recv_buffer(sched, key, ucx_memory_type::HOST), done), fail));
  }
}

}  // namespace eux::axon
