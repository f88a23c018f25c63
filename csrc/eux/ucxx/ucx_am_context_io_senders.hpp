// Connection and message senders of ucx_am_context (second half of
// ucx_am_context_senders.hpp): connect, accept stream, send, receive.
#pragma once

namespace eux::ucxx {

// ============================================================================================
// connect_endpoint
// ============================================================================================
struct connect_args {
  ucx_am_context* ctx;
  std::shared_ptr<sockaddr_storage> src;  // may be null
  std::shared_ptr<sockaddr_storage> dst;  // socket-address form
  socklen_t addrlen = 0;
  std::vector<std::byte> address;         // worker-address form
};
struct connect_sender : connect_args {
  using value_type = conn_id_t;

  template <class R>
  struct op : detail::io_op_base<op<R>, R> {
    using base = detail::io_op_base<op<R>, R>;
    struct my_timer : ucx_am_context::timer_op {
      op* self = nullptr;
    } timer;
    connect_args s;
    UcxConnection* conn = nullptr;
    bool started = false;
    DirectEntryCallback cb;
    op(connect_args&& snd, R&& r) : base(*snd.ctx, std::move(r)), s(std::move(snd)), cb(this, [](void* o, int st) { static_cast<op*>(o)->connected(st); }) {
      timer.self = this;
      timer.execute = [](ucx_am_context::operation_base* b) noexcept { static_cast<my_timer*>(b)->self->timed_out(); };
    }
    void connected(int st) noexcept {
      this->ctx.cancel_timer(&timer);
      this->on_transport_result(st);
    }
    void timed_out() noexcept {
      if (this->finished || this->have_result) return;
      if (conn) this->ctx.drop_connection(conn);
      conn = nullptr;
      this->finish_error(UCS_ERR_TIMED_OUT);
    }
    void step() noexcept {
      if (!started) {
        started = true;
        conn = this->ctx.new_connection();
        int st;
        if (!s.address.empty()) {
          transport::WorkerAddress wa;
          if (!transport::WorkerAddress::parse(s.address.data(), s.address.size(), &wa)) st = UCS_ERR_INVALID_ADDR;
          else st = conn->connect(wa, &cb);
        } else if (s.dst) {
          st = conn->connect(s.src ? reinterpret_cast<sockaddr*>(s.src.get()) : nullptr, reinterpret_cast<sockaddr*>(s.dst.get()),
                             s.addrlen, &cb);
        } else {
          st = UCS_ERR_INVALID_PARAM;
        }
        if (st != UCS_INPROGRESS) {
          this->ctx.drop_connection(conn);
          conn = nullptr;
          this->finish_error(st);
          return;
        }
        timer.due = ucx_am_context::clock_t::now() + std::max(this->ctx.connection_timeout(), std::chrono::milliseconds(1));
        this->ctx.schedule_timer(&timer);
        return;
      }
      if (!this->have_result) return;
      if (this->result_status != UCS_OK) {
        this->ctx.drop_connection(conn);
        conn = nullptr;
        this->finish_error(this->result_status);
        return;
      }
      const conn_id_t id = this->ctx.register_connection(conn);
      this->finish([this, id] { this->r.set_value(id); });
    }
    bool try_cancel() noexcept {
      if (started) {
        this->ctx.cancel_timer(&timer);
        if (conn) this->ctx.drop_connection(conn);
        conn = nullptr;
      }
      return true;
    }
  };
  template <class R>
  auto connect(R&& r) && {
    return op<std::decay_t<R>>(connect_args(std::move(*this)), std::decay_t<R>(std::forward<R>(r)));
  }
  template <class R>
  auto connect(R&& r) const& {
    return op<std::decay_t<R>>(connect_args(*this), std::decay_t<R>(std::forward<R>(r)));
  }
};

// ============================================================================================
// accept_endpoint: a stream of batches of accepted connections
// ============================================================================================
class accept_connection {
 public:
  using batch_t = std::vector<std::pair<conn_id_t, std::error_code>>;
  struct state {
    ucx_am_context* ctx;
    std::shared_ptr<sockaddr_storage> addr;
    socklen_t addrlen = 0;
    port_t port = 0;
    bool listening = false;
    bool closed = false;
  };
  explicit accept_connection(std::shared_ptr<state> st) : st_(std::move(st)) {}

  struct next_sender {
    using value_type = batch_t;
    std::shared_ptr<state> st;
    template <class R>
    struct op : detail::io_op_base<op<R>, R> {
      using base = detail::io_op_base<op<R>, R>;
      std::shared_ptr<state> st;
      op(std::shared_ptr<state> s, R&& r) : base(*s->ctx, std::move(r)), st(std::move(s)) {}
      void step() noexcept {
        auto& ctx = this->ctx;
        if (st->closed) {
          this->finish([this] { this->r.set_done(); });
          return;
        }
        if (!st->listening) {
          int rc = st->addr ? ctx.start_listening(reinterpret_cast<sockaddr*>(st->addr.get()), st->addrlen) : ctx.start_listening(st->port);
          if (rc != UCS_OK) {
            this->finish_error(rc);
            return;
          }
          st->listening = true;
        }
        auto& reqs = ctx.conn_requests();
        if (reqs.empty()) {
          ctx.park_accept(this);
          return;
        }
        batch_t batch;
        while (!reqs.empty()) {
          transport::ConnRequest req = std::move(reqs.front());
          reqs.pop_front();
          UcxConnection* c = ctx.new_connection();
          int rc = c->accept(std::move(req));
          if (rc == UCS_OK) {
            batch.emplace_back(ctx.register_connection(c), std::error_code{});
          } else {
            ctx.drop_connection(c);
            batch.emplace_back(0, make_ucx_error(rc));
          }
        }
        this->finish([this, b = std::move(batch)]() mutable { this->r.set_value(std::move(b)); });
      }
      bool try_cancel() noexcept {
        this->ctx.unpark_accept(this);
        return true;
      }
    };
    template <class R>
    auto connect(R&& r) const {
      return op<std::decay_t<R>>(st, std::decay_t<R>(std::forward<R>(r)));
    }
  };
  // Stops listening; completes with done (a stream's cleanup never produces a value).
  struct cleanup_sender {
    using value_type = void;
    std::shared_ptr<state> st;
    template <class R>
    struct op : detail::io_op_base<op<R>, R> {
      using base = detail::io_op_base<op<R>, R>;
      std::shared_ptr<state> st;
      op(std::shared_ptr<state> s, R&& r) : base(*s->ctx, std::move(r)), st(std::move(s)) {}
      void step() noexcept {
        if (st->listening) this->ctx.stop_listening();
        st->listening = false;
        st->closed = true;
        this->finish([this] { this->r.set_done(); });
      }
      bool try_cancel() noexcept { return false; }
    };
    template <class R>
    auto connect(R&& r) const {
      return op<std::decay_t<R>>(st, std::decay_t<R>(std::forward<R>(r)));
    }
  };
  next_sender next() { return {st_}; }
  cleanup_sender cleanup() { return {st_}; }

 private:
  std::shared_ptr<state> st_;
};

// ============================================================================================
// connection_send
// ============================================================================================
struct send_args {
  ucx_am_context* ctx;
  conn_id_t conn_id = 0;
  UcxConnection* conn_ptr = nullptr;
  // exactly one of the four payload forms is set
  ucx_am_data* data_ref = nullptr;
  ucx_am_iovec* iovec_ref = nullptr;
  std::shared_ptr<UcxAmData> data_owned;
  std::shared_ptr<UcxAmIovec> iovec_owned;
};
struct send_sender : send_args {
  using value_type = void;
  template <class R>
  struct op : detail::io_op_base<op<R>, R> {
    using base = detail::io_op_base<op<R>, R>;
    send_args s;
    UcxConnection* conn = nullptr;
    bool submitted = false;
    uint64_t request_id = 0;
    DirectEntryCallback cb;
    op(send_args&& snd, R&& r)
        : base(*snd.ctx, std::move(r)), s(std::move(snd)), cb(this, [](void* o, int st) { static_cast<op*>(o)->on_transport_result(st); }) {}
    void step() noexcept {
      if (submitted) {
        if (!this->have_result) return;
        if (this->result_status == UCS_OK) this->finish([this] { this->r.set_value(); });
        else this->finish_error(this->result_status);
        return;
      }
      const ucx_am_data* d = s.data_ref ? s.data_ref : (s.data_owned ? s.data_owned->get() : nullptr);
      const ucx_am_iovec* v = s.iovec_ref ? s.iovec_ref : (s.iovec_owned ? s.iovec_owned->get() : nullptr);
      // remarks filed for this message are collected whatever becomes of the send: none may stay behind
      // for a later message whose header happens to lie at the same address
      auto attr = this->ctx.take_send_attr(d ? d->header.data : (v ? v->header.data : nullptr));
      conn = s.conn_ptr ? s.conn_ptr : detail::resolve_conn(this->ctx, s.conn_id);
      if (!conn || !conn->is_established()) {
        this->finish_error(UCS_ERR_NOT_CONNECTED);
        return;
      }
      int st;
      if (d) {
        if (!d->header.data || d->header.size == 0) st = UCS_ERR_INVALID_PARAM;  // a message needs a header
        else st = conn->send_am_data(d->header.data, d->header.size, d->buffer.data, d->buffer.size, d->buffer_type, &cb, &request_id, std::move(attr));
      } else if (v) {
        if (!v->header.data || v->header.size == 0) st = UCS_ERR_INVALID_PARAM;
        else st = conn->send_am_iov_data(v->header.data, v->header.size, v->buffer_vec, v->buffer_count, v->buffer_type, &cb, &request_id, std::move(attr));
      } else {
        st = UCS_ERR_INVALID_PARAM;
      }
      if (st == UCS_OK) {
        this->finish([this] { this->r.set_value(); });
      } else if (st == UCS_INPROGRESS) {
        submitted = true;
      } else {
        this->finish_error(st);
      }
    }
    bool try_cancel() noexcept { return !submitted || (conn && conn->cancel_send(request_id)); }
  };
  template <class R>
  auto connect(R&& r) && {
    return op<std::decay_t<R>>(send_args(std::move(*this)), std::decay_t<R>(std::forward<R>(r)));
  }
  template <class R>
  auto connect(R&& r) const& {
    return op<std::decay_t<R>>(send_args(*this), std::decay_t<R>(std::forward<R>(r)));
  }
};

// ============================================================================================
// connection_recv: a whole message
// ============================================================================================
struct recv_args {
  ucx_am_context* ctx;
  ucx_am_data* user = nullptr;  // fill the caller's message in place ...
  ucx_memory_type_t data_type = ucx_memory_type::HOST;  // ... or allocate a payload of this kind
};
struct recv_sender : recv_args {
  using value_type = active_message_bundle;

  template <class R>
  struct op : detail::io_op_base<op<R>, R> {
    using base = detail::io_op_base<op<R>, R>;
    recv_args s;
    UcxAmDesc desc{};
    bool have_desc = false, submitted = false;
    UcxConnection* conn = nullptr;
    std::optional<UcxAmData> msg;  // message being assembled (owning form)
    DirectEntryCallback cb;
    op(recv_args&& snd, R&& r)
        : base(*snd.ctx, std::move(r)), s(std::move(snd)), cb(this, [](void* o, int st) { static_cast<op*>(o)->on_transport_result(st); }) {}

    void deliver() noexcept {
      const conn_id_t id = desc.conn_id;
      if (s.user) {
        this->finish([this, id] { this->r.set_value(active_message_bundle(UcxAmData(this->ctx.memory_resource(), *s.user, false, false), id, conn)); });
      } else {
        this->finish([this, id] { this->r.set_value(active_message_bundle(std::move(*msg), id, conn)); });
      }
    }
    // make sure the caller's struct has room; (re)allocates through the memory resource
    void ensure_user_room() {
      auto& mr = this->ctx.memory_resource();
      ucx_am_data& u = *s.user;
      if (!u.header.data || u.header.size < desc.header_length) {
        if (u.header.data) mr.deallocate(ucx_memory_type::HOST, u.header.data, u.header.size);
        u.header.data = desc.header_length ? mr.allocate(ucx_memory_type::HOST, desc.header_length) : nullptr;
      }
      u.header.size = desc.header_length;
      if (!u.buffer.data || u.buffer.size < desc.data_length) {
        if (u.buffer.data) mr.deallocate(u.buffer_type, u.buffer.data, u.buffer.size);
        u.buffer.data = desc.data_length ? mr.allocate(u.buffer_type, desc.data_length) : nullptr;
      }
      u.buffer.size = desc.data_length;
    }
    void step() noexcept {
      auto& ctx = this->ctx;
      auto& mr = ctx.memory_resource();
      if (submitted) {
        if (!this->have_result) return;
        if (this->result_status != UCS_OK) {
          msg.reset();
          this->finish_error(this->result_status);
          return;
        }
        deliver();
        return;
      }
      if (!have_desc) {
        if (ctx.am_queue().empty()) {
          ctx.park_recv(this);
          return;
        }
        desc = ctx.am_queue().front();
        ctx.am_queue().pop_front();
        have_desc = true;
      }
      conn = ctx.connections().get_connection(desc.conn_id);
      try {
        if (s.user) {
          ensure_user_room();
          if (desc.header_length) std::memcpy(s.user->header.data, desc.header, desc.header_length);
        } else {
          // header: adopt the arrival's host bytes; payload: adopt (eager, host) or allocate
          ucx_am_data raw{};
          raw.header = {desc.header, desc.header_length};
          raw.buffer_type = s.data_type;
          desc.header = nullptr;
          if (!desc.rndv && s.data_type == ucx_memory_type::HOST && desc.data_mem_type == ucx_memory_type::HOST) {
            raw.buffer = {desc.data, desc.data_length};
            desc.data = nullptr;
          } else {
            raw.buffer = {desc.data_length ? mr.allocate(s.data_type, desc.data_length) : nullptr, desc.data_length};
          }
          msg.emplace(mr, std::move(raw), true, true);
        }
        ucx_am_data& target = s.user ? *s.user : *msg->get();
        if (!desc.rndv) {
          // eager bytes sit in host memory, or (small device payloads between GPUs of one host) in a slot of
          // the worker's device receive ring
          if (desc.data && desc.data_length) mr.memcpy(target.buffer_type, target.buffer.data, desc.data_mem_type, desc.data, desc.data_length);
          desc.release(mr);
          deliver();
          return;
        }
        if (!conn) {
          desc.release(mr);
          msg.reset();
          this->finish_error(UCS_ERR_NOT_CONNECTED);
          return;
        }
        int st = conn->recv_am_data(desc, target.buffer.data, target.buffer.size, target.buffer_type, &cb);
        desc.release(mr);
        if (st == UCS_OK) {
          deliver();
        } else if (st == UCS_INPROGRESS) {
          submitted = true;
        } else {
          msg.reset();
          this->finish_error(st);
        }
      } catch (...) {
        desc.release(mr);
        msg.reset();
        this->finish([this, e = std::current_exception()] { this->r.set_error(e); });
      }
    }
    bool try_cancel() noexcept {
      if (this->parked) {
        this->ctx.unpark_recv(this);
        return true;
      }
      if (submitted) {
        if (conn && !conn->cancel_recv(desc.msg_id)) return false;
        msg.reset();
        return true;
      }
      return !have_desc;
    }
  };
  template <class R>
  auto connect(R&& r) && {
    return op<std::decay_t<R>>(recv_args(std::move(*this)), std::decay_t<R>(std::forward<R>(r)));
  }
  template <class R>
  auto connect(R&& r) const& {
    return op<std::decay_t<R>>(recv_args(*this), std::decay_t<R>(std::forward<R>(r)));
  }
};

}  // namespace eux::ucxx

#include "eux/ucxx/ucx_am_context_recv_senders.hpp"
