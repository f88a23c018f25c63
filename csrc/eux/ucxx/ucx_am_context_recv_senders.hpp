// Two-phase receive (header first, payload by key), the connection-error
// handler, and the tag_invoke overloads that bind the customisation points to
// ucx_am_context::scheduler (third part of ucx_am_context_senders.hpp).
#pragma once

namespace eux::ucxx {

// ============================================================================================
// connection_recv_header
// ============================================================================================
struct recv_header_sender {
  using value_type = recv_header_result_t;
  ucx_am_context* ctx;
  template <class R>
  struct op : detail::io_op_base<op<R>, R> {
    using base = detail::io_op_base<op<R>, R>;
    op(ucx_am_context* c, R&& r) : base(*c, std::move(r)) {}
    void step() noexcept {
      auto& ctx = this->ctx;
      auto& mr = ctx.memory_resource();
      if (ctx.am_queue().empty()) {
        ctx.park_recv(this);
        return;
      }
      UcxAmDesc d = ctx.am_queue().front();
      ctx.am_queue().pop_front();
      UcxHeader header(mr, ucx_header_t{d.header, d.header_length}, true);
      d.header = nullptr;
      d.header_length = 0;
      if (d.rndv) {
        const size_t key = ctx.stash_rndv_desc(std::move(d));
        auto res = std::make_shared<recv_header_result_t>(std::in_place_index<0>, key, std::move(header));
        this->finish([this, res] { this->r.set_value(std::move(*res)); });
        return;
      }
      UcxConnection* conn = ctx.connections().get_connection(d.conn_id);
      // Eager bytes: host memory owned by the buffer from here on, or a slot of the device receive ring,
      // which goes back to the sender when the buffer drops its keep-alive token.
      UcxBuffer buffer = d.data_keep ? UcxBuffer(mr, d.data_mem_type, d.data, d.data_length, nullptr, true,
                                                 [keep = std::move(d.data_keep)](void*) mutable { keep.reset(); })
                                     : UcxBuffer(mr, ucx_memory_type::HOST, d.data, d.data_length, nullptr, true);
      auto res = std::make_shared<recv_header_result_t>(
          std::in_place_index<1>, active_message_header_buffer_bundle(std::move(header), std::move(buffer), d.conn_id, conn));
      this->finish([this, res] { this->r.set_value(std::move(*res)); });
    }
    bool try_cancel() noexcept {
      this->ctx.unpark_recv(this);
      return true;
    }
  };
  template <class R>
  auto connect(R&& r) const {
    return op<std::decay_t<R>>(ctx, std::decay_t<R>(std::forward<R>(r)));
  }
};

// ============================================================================================
// connection_recv_buffer
// ============================================================================================
template <class Target>
struct recv_buffer_args {
  ucx_am_context* ctx;
  size_t key;
  std::shared_ptr<Target> target;  // null: allocate `alloc_type` memory of the announced size
  ucx_memory_type_t alloc_type = ucx_memory_type::HOST;
};
template <class Target>  // UcxBuffer or UcxBufferVec
struct recv_buffer_sender : recv_buffer_args<Target> {
  using value_type = std::conditional_t<std::is_same_v<Target, UcxBuffer>, active_message_buffer_bundle, active_message_iovec_buffer_bundle>;

  template <class R>
  struct op : detail::io_op_base<op<R>, R> {
    using base = detail::io_op_base<op<R>, R>;
    recv_buffer_args<Target> s;
    UcxAmDesc desc{};
    UcxConnection* conn = nullptr;
    bool submitted = false;
    DirectEntryCallback cb;
    op(recv_buffer_args<Target>&& snd, R&& r)
        : base(*snd.ctx, std::move(r)), s(std::move(snd)), cb(this, [](void* o, int st) { static_cast<op*>(o)->on_transport_result(st); }) {}
    void deliver() noexcept {
      this->finish([this] { this->r.set_value(value_type(std::move(*s.target), desc.conn_id, conn)); });
    }
    void step() noexcept {
      auto& ctx = this->ctx;
      auto& mr = ctx.memory_resource();
      if (submitted) {
        if (!this->have_result) return;
        if (this->result_status != UCS_OK) this->finish_error(this->result_status);
        else deliver();
        return;
      }
      auto d = ctx.pop_pending_am_desc(s.key);
      if (!d) {
        this->finish_error(UCS_ERR_NO_ELEM);
        return;
      }
      desc = *d;
      conn = ctx.connections().get_connection(desc.conn_id);
      if (!conn || !conn->is_established()) {
        desc.release(mr);
        this->finish_error(UCS_ERR_NOT_CONNECTED);
        return;
      }
      int st;
      try {
        if constexpr (std::is_same_v<Target, UcxBuffer>) {
          if (!s.target) s.target = std::make_shared<UcxBuffer>(mr, s.alloc_type, desc.data_length);
          st = conn->recv_am_data(desc, s.target->data(), s.target->size(), s.target->type(), &cb, s.target->send_attr());
        } else {
          if (!s.target) {
            auto sizes64 = conn->rndv_segment_sizes(desc);
            std::vector<size_t> sizes(sizes64.begin(), sizes64.end());
            if (sizes.empty()) sizes.push_back(desc.data_length);
            s.target = std::make_shared<UcxBufferVec>(mr, s.alloc_type, sizes);
          }
          st = conn->recv_am_iov_data(desc, s.target->buffers().data(), s.target->size(), s.target->type(), &cb, s.target->send_attr());
        }
      } catch (...) {
        conn->release_rndv(desc);
        desc.release(mr);
        this->finish([this, e = std::current_exception()] { this->r.set_error(e); });
        return;
      }
      desc.release(mr);
      if (st == UCS_OK) deliver();
      else if (st == UCS_INPROGRESS) submitted = true;
      else this->finish_error(st);
    }
    bool try_cancel() noexcept { return !submitted || (conn && conn->cancel_recv(desc.msg_id)); }
  };
  template <class R>
  auto connect(R&& r) && {
    return op<std::decay_t<R>>(recv_buffer_args<Target>(std::move(*this)), std::decay_t<R>(std::forward<R>(r)));
  }
  template <class R>
  auto connect(R&& r) const& {
    return op<std::decay_t<R>>(recv_buffer_args<Target>(*this), std::decay_t<R>(std::forward<R>(r)));
  }
};

// ============================================================================================
// handle_error_connection
// ============================================================================================
template <class Handler>
struct dispatch_connection_error_sender {
  using value_type = void;
  ucx_am_context* ctx;
  Handler handler;
  template <class R>
  struct op : detail::io_op_base<op<R>, R> {
    using base = detail::io_op_base<op<R>, R>;
    Handler handler;
    UcxConnection* reconnecting = nullptr;
    DirectEntryCallback cb;
    op(ucx_am_context* c, Handler&& h, R&& r)
        : base(*c, std::move(r)), handler(std::move(h)), cb(this, [](void* o, int st) { static_cast<op*>(o)->on_transport_result(st); }) {}
    void step() noexcept {
      auto& ctx = this->ctx;
      if (reconnecting) {
        if (!this->have_result) return;
        if (this->result_status == UCS_OK) ctx.register_connection(reconnecting);
        else ctx.drop_connection(reconnecting);
        reconnecting = nullptr;
        this->finish([this] { this->r.set_value(); });
        return;
      }
      if (!ctx.connection_handle_error()) {
        this->finish_error(UCS_ERR_UNSUPPORTED);  // the context was created without error handling
        return;
      }
      auto failed = ctx.connections().pop_failed();
      if (!failed) {
        ctx.park_error(this);
        return;
      }
      bool want_reconnect = false;
      try {
        if constexpr (std::is_invocable_v<Handler&, conn_id_t, std::error_code>) {
          want_reconnect = handler(failed->id, make_ucx_error(failed->status));
        } else {
          want_reconnect = handler(failed->id, static_cast<ucs_status_t>(failed->status));
        }
      } catch (...) {
        this->finish([this, e = std::current_exception()] { this->r.set_error(e); });
        return;
      }
      if (want_reconnect && ctx.reconnect(*failed, &cb, &reconnecting) == UCS_INPROGRESS) return;
      reconnecting = nullptr;
      this->finish([this] { this->r.set_value(); });
    }
    bool try_cancel() noexcept {
      if (reconnecting) {
        this->ctx.drop_connection(reconnecting);
        reconnecting = nullptr;
      }
      this->ctx.unpark_error(this);
      return true;
    }
  };
  template <class R>
  auto connect(R&& r) && {
    return op<std::decay_t<R>>(ctx, std::move(handler), std::decay_t<R>(std::forward<R>(r)));
  }
  template <class R>
  auto connect(R&& r) const& {
    return op<std::decay_t<R>>(ctx, Handler(handler), std::decay_t<R>(std::forward<R>(r)));
  }
};

// ============================================================================================
// tag_invoke overloads for ucx_am_context::scheduler
// ============================================================================================
namespace detail {
inline std::shared_ptr<sockaddr_storage> copy_sockaddr(const sockaddr* sa, socklen_t len) {
  if (!sa) return nullptr;
  auto out = std::make_shared<sockaddr_storage>();
  std::memset(out.get(), 0, sizeof(sockaddr_storage));
  std::memcpy(out.get(), sa, std::min<size_t>(len, sizeof(sockaddr_storage)));
  return out;
}
inline void set_conn(send_args& s, conn_id_t id) { s.conn_id = id; }
inline void set_conn(send_args& s, conn_pair_t& p) {
  s.conn_id = p.first;
  s.conn_ptr = &p.second.get();
}
inline void set_conn(send_args& s, UcxConnection& c) {
  s.conn_id = c.id();
  s.conn_ptr = &c;
}
}  // namespace detail

inline accept_connection tag_invoke(accept_endpoint_cpo, const ucx_am_context::scheduler& sched, std::unique_ptr<sockaddr> addr,
                                    socklen_t addrlen) {
  auto st = std::make_shared<accept_connection::state>();
  st->ctx = &sched.context();
  st->addr = detail::copy_sockaddr(addr.get(), addrlen);
  st->addrlen = addrlen;
  return accept_connection(std::move(st));
}
inline accept_connection tag_invoke(accept_endpoint_cpo, const ucx_am_context::scheduler& sched, port_t port) {
  auto st = std::make_shared<accept_connection::state>();
  st->ctx = &sched.context();
  st->port = port;
  return accept_connection(std::move(st));
}

inline connect_sender tag_invoke(connect_endpoint_cpo, const ucx_am_context::scheduler& sched, std::unique_ptr<sockaddr> src,
                                 std::unique_ptr<sockaddr> dst, socklen_t addrlen) {
  connect_sender s;
  s.ctx = &sched.context();
  s.src = detail::copy_sockaddr(src.get(), addrlen);
  s.dst = detail::copy_sockaddr(dst.get(), addrlen);
  s.addrlen = addrlen;
  return s;
}
inline connect_sender tag_invoke(connect_endpoint_cpo, const ucx_am_context::scheduler& sched, std::vector<std::byte> address) {
  connect_sender s;
  s.ctx = &sched.context();
  s.address = std::move(address);
  return s;
}

template <class Conn>
  requires detail::is_conn_ref_v<Conn>
send_sender tag_invoke(connection_send_cpo, const ucx_am_context::scheduler& sched, Conn&& conn, ucx_am_data& data) {
  send_sender s;
  s.ctx = &sched.context();
  if constexpr (std::is_convertible_v<Conn, conn_id_t>) detail::set_conn(s, static_cast<conn_id_t>(conn));
  else detail::set_conn(s, conn);
  s.data_ref = &data;
  return s;
}
template <class Conn>
  requires detail::is_conn_ref_v<Conn>
send_sender tag_invoke(connection_send_cpo, const ucx_am_context::scheduler& sched, Conn&& conn, UcxAmData&& data) {
  send_sender s;
  s.ctx = &sched.context();
  if constexpr (std::is_convertible_v<Conn, conn_id_t>) detail::set_conn(s, static_cast<conn_id_t>(conn));
  else detail::set_conn(s, conn);
  s.data_owned = std::make_shared<UcxAmData>(std::move(data));
  return s;
}
template <class Conn>
  requires detail::is_conn_ref_v<Conn>
send_sender tag_invoke(connection_send_cpo, const ucx_am_context::scheduler& sched, Conn&& conn, ucx_am_iovec& iov) {
  send_sender s;
  s.ctx = &sched.context();
  if constexpr (std::is_convertible_v<Conn, conn_id_t>) detail::set_conn(s, static_cast<conn_id_t>(conn));
  else detail::set_conn(s, conn);
  s.iovec_ref = &iov;
  return s;
}
template <class Conn>
  requires detail::is_conn_ref_v<Conn>
send_sender tag_invoke(connection_send_cpo, const ucx_am_context::scheduler& sched, Conn&& conn, UcxAmIovec&& iov) {
  send_sender s;
  s.ctx = &sched.context();
  if constexpr (std::is_convertible_v<Conn, conn_id_t>) detail::set_conn(s, static_cast<conn_id_t>(conn));
  else detail::set_conn(s, conn);
  s.iovec_owned = std::make_shared<UcxAmIovec>(std::move(iov));
  return s;
}

inline recv_sender tag_invoke(connection_recv_cpo, const ucx_am_context::scheduler& sched, ucx_am_data& data) {
  recv_sender s;
  s.ctx = &sched.context();
  s.user = &data;
  s.data_type = data.buffer_type;
  return s;
}
inline recv_sender tag_invoke(connection_recv_cpo, const ucx_am_context::scheduler& sched, ucx_memory_type data_type) {
  recv_sender s;
  s.ctx = &sched.context();
  s.data_type = data_type;
  return s;
}

inline recv_header_sender tag_invoke(connection_recv_header_cpo, const ucx_am_context::scheduler& sched) {
  return recv_header_sender{&sched.context()};
}

inline recv_buffer_sender<UcxBuffer> tag_invoke(connection_recv_buffer_cpo, const ucx_am_context::scheduler& sched, size_t key,
                                                UcxBuffer&& buffer) {
  recv_buffer_sender<UcxBuffer> s;
  s.ctx = &sched.context();
  s.key = key;
  s.target = std::make_shared<UcxBuffer>(std::move(buffer));
  return s;
}
inline recv_buffer_sender<UcxBufferVec> tag_invoke(connection_recv_buffer_cpo, const ucx_am_context::scheduler& sched, size_t key,
                                                   UcxBufferVec&& buffers) {
  recv_buffer_sender<UcxBufferVec> s;
  s.ctx = &sched.context();
  s.key = key;
  s.target = std::make_shared<UcxBufferVec>(std::move(buffers));
  return s;
}
inline recv_buffer_sender<UcxBuffer> tag_invoke(connection_recv_buffer_cpo, const ucx_am_context::scheduler& sched, size_t key,
                                                ucx_memory_type data_type) {
  recv_buffer_sender<UcxBuffer> s;
  s.ctx = &sched.context();
  s.key = key;
  s.alloc_type = data_type;
  return s;
}

template <class Handler>
  requires(std::is_invocable_r_v<bool, Handler&, conn_id_t, std::error_code> ||
           std::is_invocable_r_v<bool, Handler&, conn_id_t, ucs_status_t>)
dispatch_connection_error_sender<std::decay_t<Handler>> tag_invoke(handle_error_connection_cpo, const ucx_am_context::scheduler& sched,
                                                                  Handler&& handler) {
  return {&sched.context(), std::forward<Handler>(handler)};
}

}  // namespace eux::ucxx
