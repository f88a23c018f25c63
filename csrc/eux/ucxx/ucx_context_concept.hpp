// Customisation points of the active-message layer. Each one is a function
// object that forwards to `tag_invoke(cpo, scheduler, args...)`, found by ADL on
// the scheduler type, and returns a sender. A different context can provide the
// same operations by defining tag_invoke overloads for its own scheduler
// (reference: ucx_context/ucx_context_concept.hpp:67-542).
#pragma once

#include <sys/socket.h>

#include <cstdint>
#include <functional>
#include <memory>
#include <system_error>
#include <type_traits>
#include <utility>
#include <vector>

#include "eux/ucxx/ucx_connection.hpp"
#include "eux/ucxx/ucx_context_data.hpp"
#include "eux/ucxx/ucx_context_def.h"

namespace eux::ucxx {

namespace detail {
template <class T>
inline constexpr bool is_am_payload_v =
    std::is_same_v<std::remove_cvref_t<T>, ucx_am_data> || std::is_same_v<std::remove_cvref_t<T>, UcxAmData> ||
    std::is_same_v<std::remove_cvref_t<T>, ucx_am_iovec> || std::is_same_v<std::remove_cvref_t<T>, UcxAmIovec>;
template <class T>
inline constexpr bool is_conn_ref_v = std::is_same_v<std::remove_cvref_t<T>, conn_pair_t> ||
                                      std::is_convertible_v<T, conn_id_t> ||
                                      std::is_same_v<std::remove_cvref_t<T>, UcxConnection>;
}  // namespace detail

// accept_endpoint(sched, unique_ptr<sockaddr>, addrlen) / (sched, port): a stream of
// accepted connections: `.next()` completes with vector<pair<conn_id, error_code>>,
// `.cleanup()` stops listening.
inline constexpr struct accept_endpoint_cpo {
  template <class Scheduler>
  auto operator()(Scheduler&& sched, std::unique_ptr<sockaddr> addr, socklen_t addrlen) const
      -> decltype(tag_invoke(*this, std::forward<Scheduler>(sched), std::move(addr), addrlen)) {
    return tag_invoke(*this, std::forward<Scheduler>(sched), std::move(addr), addrlen);
  }
  template <class Scheduler>
  auto operator()(Scheduler&& sched, port_t port) const -> decltype(tag_invoke(*this, std::forward<Scheduler>(sched), port)) {
    return tag_invoke(*this, std::forward<Scheduler>(sched), port);
  }
} accept_endpoint{};

// connect_endpoint(sched, src_saddr | nullptr, dst_saddr, addrlen) / (sched, worker_address_bytes)
// completes with the new connection id.
inline constexpr struct connect_endpoint_cpo {
  template <class Scheduler>
  auto operator()(Scheduler&& sched, std::unique_ptr<sockaddr> src, std::unique_ptr<sockaddr> dst, socklen_t addrlen) const
      -> decltype(tag_invoke(*this, std::forward<Scheduler>(sched), std::move(src), std::move(dst), addrlen)) {
    return tag_invoke(*this, std::forward<Scheduler>(sched), std::move(src), std::move(dst), addrlen);
  }
  template <class Scheduler>
  auto operator()(Scheduler&& sched, std::vector<std::byte> ucp_address) const
      -> decltype(tag_invoke(*this, std::forward<Scheduler>(sched), std::move(ucp_address))) {
    return tag_invoke(*this, std::forward<Scheduler>(sched), std::move(ucp_address));
  }
} connect_endpoint{};

// connection_send(sched, conn, data): conn is a conn_pair_t&, a connection id or a
// UcxConnection&; data is ucx_am_data&, UcxAmData&&, ucx_am_iovec& or UcxAmIovec&&.
inline constexpr struct connection_send_cpo {
  template <class Scheduler, class Conn, class Data>
    requires(detail::is_conn_ref_v<Conn> && detail::is_am_payload_v<Data>)
  auto operator()(Scheduler&& sched, Conn&& conn, Data&& data) const
      -> decltype(tag_invoke(*this, std::forward<Scheduler>(sched), std::forward<Conn>(conn), std::forward<Data>(data))) {
    return tag_invoke(*this, std::forward<Scheduler>(sched), std::forward<Conn>(conn), std::forward<Data>(data));
  }
} connection_send{};

// connection_recv(sched, ucx_am_data&) -- into the caller's message --
// connection_recv(sched, ucx_memory_type) -- payload allocated by the context --
// completes with an active_message_bundle.
inline constexpr struct connection_recv_cpo {
  template <class Scheduler>
  auto operator()(Scheduler&& sched, ucx_am_data& data) const -> decltype(tag_invoke(*this, std::forward<Scheduler>(sched), data)) {
    return tag_invoke(*this, std::forward<Scheduler>(sched), data);
  }
  template <class Scheduler>
  auto operator()(Scheduler&& sched, ucx_memory_type data_type) const
      -> decltype(tag_invoke(*this, std::forward<Scheduler>(sched), data_type)) {
    return tag_invoke(*this, std::forward<Scheduler>(sched), data_type);
  }
} connection_recv{};

// connection_recv_header(sched): next message's header. Rendezvous messages give
// {key, header} (the payload is fetched later by key); eager ones give the whole message.
inline constexpr struct connection_recv_header_cpo {
  template <class Scheduler>
  auto operator()(Scheduler&& sched) const -> decltype(tag_invoke(*this, std::forward<Scheduler>(sched))) {
    return tag_invoke(*this, std::forward<Scheduler>(sched));
  }
} connection_recv_header{};

// connection_recv_buffer(sched, key, UcxBuffer&& | UcxBufferVec&& | ucx_memory_type)
inline constexpr struct connection_recv_buffer_cpo {
  template <class Scheduler, class Target>
  auto operator()(Scheduler&& sched, size_t am_desc_key, Target&& target) const
      -> decltype(tag_invoke(*this, std::forward<Scheduler>(sched), am_desc_key, std::forward<Target>(target))) {
    return tag_invoke(*this, std::forward<Scheduler>(sched), am_desc_key, std::forward<Target>(target));
  }
} connection_recv_buffer{};

// handle_error_connection(sched, bool(conn_id, error_code)): waits for the next failed
// connection and calls the handler; a `true` return asks for a reconnect.
inline constexpr struct handle_error_connection_cpo {
  template <class Scheduler, class Handler>
  auto operator()(Scheduler&& sched, Handler&& handler) const
      -> decltype(tag_invoke(*this, std::forward<Scheduler>(sched), std::forward<Handler>(handler))) {
    return tag_invoke(*this, std::forward<Scheduler>(sched), std::forward<Handler>(handler));
  }
} handle_error_connection{};

}  // namespace eux::ucxx
