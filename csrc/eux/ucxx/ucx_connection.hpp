// UcxConnection: one peer as seen by the active-message context. It wraps a
// transport endpoint, gives it a stable 64-bit id, tracks the operations in
// flight so they can be cancelled or failed together, and carries the
// callback objects through which completions reach the context (reference:
// ucx_context/ucx_connection.hpp:56-556).
#pragma once

#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <unordered_map>
#include <utility>

#include "eux/ucxx/transport.hpp"
#include "eux/ucxx/ucx_context_def.h"
#include "eux/ucxx/ucx_status.hpp"

namespace eux::ucxx {

constexpr uint16_t DEFAULT_AM_MSG_ID = 0;
using conn_id_t = std::uint64_t;
using conn_pair_t = std::pair<conn_id_t, std::reference_wrapper<class UcxConnection>>;
using port_t = std::uint16_t;

// Descriptor of a received active message waiting in the context's queue.
struct UcxAmDesc {
  conn_id_t conn_id = 0;
  void* header = nullptr;  // HOST memory from the context's memory resource; owned until consumed
  size_t header_length = 0;
  void* data = nullptr;    // eager payload (HOST, same resource) or nullptr for rendezvous
  size_t data_length = 0;
  bool rndv = false;
  uint64_t msg_id = 0;
  uint32_t seg_count = 0;
  ucx_memory_type_t sender_mem_type = ucx_memory_type::HOST;
  // Eager data is HOST memory of the context's resource, unless `data_keep` is set: then it is a slot
  // of the transport's device receive ring (`data_mem_type`), never deallocated, and handed back to the
  // sender when the last copy of the token is dropped.
  ucx_memory_type_t data_mem_type = ucx_memory_type::HOST;
  std::shared_ptr<void> data_keep;
  void release(UcxMemoryResourceManager& mr) noexcept;  // frees header/data that are still attached
};

// ---- completion callbacks ---------------------------------------------------
class UcxCallback {
 public:
  virtual ~UcxCallback() = default;
  virtual void operator()(int status) = 0;
};
class EmptyCallback final : public UcxCallback {
 public:
  void operator()(int) override {}
  static EmptyCallback* get() {
    static EmptyCallback cb;
    return &cb;
  }
};
// Writes a completion entry {user_data, res} into a ring owned by the context.
class CqeEntryCallback final : public UcxCallback {
 public:
  using push_fn = std::function<void(const ucx_am_cqe_t&)>;
  CqeEntryCallback(size_t user_data, push_fn push) : user_data_(user_data), push_(std::move(push)) {}
  void operator()(int status) override { push_(ucx_am_cqe_t{user_data_, status, 0}); }

 private:
  size_t user_data_;
  push_fn push_;
};
// Calls the operation's completion function directly.
class DirectEntryCallback final : public UcxCallback {
 public:
  using fn_t = void (*)(void* op, int status);
  DirectEntryCallback(void* op, fn_t fn) : op_(op), fn_(fn) {}
  void operator()(int status) override { fn_(op_, status); }

 private:
  void* op_;
  fn_t fn_;
};

// One operation in flight on a connection.
struct UcxRequest {
  uint64_t msg_id = 0;
  bool is_send = true;
  UcxCallback* callback = nullptr;
};

class UcxConnection {
 public:
  enum class Status { kConnecting, kConnected, kDisconnecting, kFailed, kClosed };

  UcxConnection(transport::Worker& worker, bool handle_errors) : worker_(worker), handle_errors_(handle_errors) {}
  ~UcxConnection();
  UcxConnection(const UcxConnection&) = delete;

  // -- establishing --
  int connect(const sockaddr* src, const sockaddr* dst, socklen_t len, UcxCallback* cb);
  int connect(const transport::WorkerAddress& addr, UcxCallback* cb);
  int accept(transport::ConnRequest&& req);
  void adopt(transport::Endpoint* ep);  // endpoint that the worker accepted by itself

  // -- active messages (return UCS_OK = finished inline, UCS_INPROGRESS, or an error) --
  // `attr`: optional remarks about a device payload (strided layout, readiness event; ucx_send_attr.hpp)
  int send_am_data(const void* header, size_t header_len, const void* buffer, size_t length, ucx_memory_type_t type,
                   UcxCallback* cb, uint64_t* request_id = nullptr, std::shared_ptr<const UcxSendAttr> attr = nullptr);
  int send_am_iov_data(const void* header, size_t header_len, const ucx_buffer_t* iov, size_t count,
                       ucx_memory_type_t type, UcxCallback* cb, uint64_t* request_id = nullptr,
                       std::shared_ptr<const UcxSendAttr> attr = nullptr);
  // `attr` of a receive buffer: only its event is looked at (the buffer may be written once it has completed)
  int recv_am_data(const UcxAmDesc& desc, void* buffer, size_t length, ucx_memory_type_t type, UcxCallback* cb,
                   std::shared_ptr<const UcxSendAttr> attr = nullptr);
  int recv_am_iov_data(const UcxAmDesc& desc, const ucx_buffer_t* iov, size_t count, ucx_memory_type_t type, UcxCallback* cb,
                       std::shared_ptr<const UcxSendAttr> attr = nullptr);
  bool cancel_send(uint64_t request_id);
  bool cancel_recv(uint64_t msg_id);
  void release_rndv(const UcxAmDesc& desc);
  std::vector<uint64_t> rndv_segment_sizes(const UcxAmDesc& desc) const;

  void disconnect();
  void mark_failed(int status) {
    status_ = Status::kFailed;
    ucs_status_ = status;
  }

  conn_id_t id() const { return reinterpret_cast<conn_id_t>(ep_ ? static_cast<const void*>(ep_) : static_cast<const void*>(this)); }
  Status status() const { return status_; }
  bool is_established() const { return status_ == Status::kConnected; }
  int ucs_status() const { return ucs_status_; }
  const std::string& peer_name() const { return peer_name_; }
  std::string remote_worker_name() const { return ep_ ? ep_->remote_worker_name() : std::string(); }
  uint64_t remote_client_id() const { return ep_ ? ep_->remote_client_id() : 0; }
  transport::Endpoint* endpoint() const { return ep_; }
  bool handle_errors() const { return handle_errors_; }
  // payloads of at least this many bytes are sent by rendezvous (zero copy)
  bool should_use_zcopy(size_t length) const { return length >= worker_.options().eager_limit; }

 private:
  transport::Worker& worker_;
  transport::Endpoint* ep_ = nullptr;
  Status status_ = Status::kConnecting;
  int ucs_status_ = UCS_OK;
  bool handle_errors_;
  std::string peer_name_;
};

}  // namespace eux::ucxx
