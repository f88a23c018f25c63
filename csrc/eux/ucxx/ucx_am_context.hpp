// ucx_am_context: the active-message execution context.
//
// One worker thread runs `run(stop_token)`: a proactor loop that interleaves a
// sender/receiver scheduler (local queue, cross-thread remote queue, timers) with
// progress of the transport. Every asynchronous operation of the layer is a
// sender obtained through the customisation points in ucx_context_concept.hpp
// and the context's scheduler. Shape and public surface follow the reference's
// ucx_context/ucx_am_context/ucx_am_context.hpp:361-1002 (context), :2828-2967
// (scheduler) and :128-318 (result bundles); timers use the loop's clock instead
// of POSIX timers + SIGUSR2.
#pragma once
#include <mutex>

#include <atomic>
#include <chrono>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <optional>
#include <string>
#include <thread>
#include <unordered_map>
#include <variant>
#include <vector>

#include "eux/exec/exec.hpp"
#include "eux/ucxx/transport.hpp"
#include "eux/ucxx/ucx_connection.hpp"
#include "eux/ucxx/ucx_connection_manager.hpp"
#include "eux/ucxx/ucx_context_concept.hpp"
#include "eux/ucxx/ucx_context_data.hpp"
#include "eux/ucxx/ucx_device_context.hpp"
#include "eux/ucxx/ucx_status.hpp"

namespace eux::ucxx {

constexpr size_t kCompletionQueueEntryCount = 256;

// ---- result bundles -----------------------------------------------------------------
// A received message plus the connection it came from.
class active_message_bundle {
 public:
  active_message_bundle(UcxAmData&& data, conn_id_t id, UcxConnection* conn) : data_(std::move(data)), id_(id), conn_(conn) {}
  UcxAmData& data() { return data_; }
  const UcxAmData& data() const { return data_; }
  UcxAmData&& move_data() { return std::move(data_); }
  ucx_am_data& get_raw_data() { return *data_.get(); }
  UcxConnection& connection() { return *conn_; }
  conn_id_t conn_id() const { return id_; }
  conn_pair_t conn_pair() { return {id_, std::ref(*conn_)}; }

 private:
  UcxAmData data_;
  conn_id_t id_;
  UcxConnection* conn_;
};

// An eager message delivered by connection_recv_header: header and payload are both there.
class active_message_header_buffer_bundle {
 public:
  active_message_header_buffer_bundle(UcxHeader&& h, UcxBuffer&& b, conn_id_t id, UcxConnection* conn)
      : header_(std::move(h)), buffer_(std::move(b)), id_(id), conn_(conn) {}
  UcxHeader& header() { return header_; }
  UcxBuffer& buffer() { return buffer_; }
  UcxHeader&& move_header() { return std::move(header_); }
  UcxBuffer&& move_buffer() { return std::move(buffer_); }
  UcxConnection& connection() { return *conn_; }
  conn_id_t conn_id() const { return id_; }

 private:
  UcxHeader header_;
  UcxBuffer buffer_;
  conn_id_t id_;
  UcxConnection* conn_;
};

class active_message_buffer_bundle {
 public:
  active_message_buffer_bundle(UcxBuffer&& b, conn_id_t id, UcxConnection* conn) : buffer_(std::move(b)), id_(id), conn_(conn) {}
  UcxBuffer& buffer() { return buffer_; }
  UcxBuffer&& move_buffer() { return std::move(buffer_); }
  UcxConnection& connection() { return *conn_; }
  conn_id_t conn_id() const { return id_; }

 private:
  UcxBuffer buffer_;
  conn_id_t id_;
  UcxConnection* conn_;
};

class active_message_iovec_buffer_bundle {
 public:
  active_message_iovec_buffer_bundle(UcxBufferVec&& b, conn_id_t id, UcxConnection* conn)
      : buffer_(std::move(b)), id_(id), conn_(conn) {}
  UcxBufferVec& buffer() { return buffer_; }
  UcxBufferVec&& move_buffer() { return std::move(buffer_); }
  UcxConnection& connection() { return *conn_; }
  conn_id_t conn_id() const { return id_; }

 private:
  UcxBufferVec buffer_;
  conn_id_t id_;
  UcxConnection* conn_;
};

using recv_header_result_t = std::variant<std::pair<size_t, UcxHeader>, active_message_header_buffer_bundle>;

// ---- the context ----------------------------------------------------------------------
// Settings shared by the contexts of a process: what stands in for a UCP context here.
struct eux_shared_transport_context {
  std::string name;
  bool mt_workers_shared = false;
  size_t eager_limit = 0;      // 0 = the worker's default
  size_t send_copy_limit = 0;  // 0 = the worker's default
};
using ucp_context_h = eux_shared_transport_context*;

class ucx_am_context {
 public:
  using clock_t = std::chrono::steady_clock;
  using time_point = clock_t::time_point;
  class scheduler;

  // Intrusive work item: everything the loop runs is one of these.
  struct operation_base {
    operation_base* next = nullptr;
    void (*execute)(operation_base*) noexcept = nullptr;
  };
  struct timer_op : operation_base {
    time_point due;
    bool armed = false;
  };
  // Waits for a 64-bit word in host memory (normally mapped pinned memory that a kernel writes when its
  // work is done) to reach a value. The loop looks at every watched word once per pass.
  struct flag_op : operation_base {
    const volatile uint64_t* flag = nullptr;
    uint64_t at_least = 0;
    bool armed = false;
  };
  // An operation that parks until a message / connection event arrives.
  struct parked_op : operation_base {
    parked_op* prev_parked = nullptr;
    parked_op* next_parked = nullptr;
    bool parked = false;
    bool queued = false;  // sitting in a run queue; execute() will be called
  };

  explicit ucx_am_context(UcxMemoryResourceManager& mr, std::string_view name = "default",
                          std::chrono::milliseconds connectionTimeout = std::chrono::milliseconds(300),
                          bool connectionHandleError = false, uint64_t clientId = 0,
                          std::unique_ptr<UcxAutoDeviceContext> deviceContext = nullptr);
  // The same with transport settings shared between several contexts of a process
  // (reference: the overload that takes an external ucp_context_h,
  // ucx_context/ucx_am_context/ucx_am_context.hpp:424-452). The shared context must outlive
  // the contexts built on it.
  ucx_am_context(UcxMemoryResourceManager& mr, ucp_context_h sharedContext, std::string_view name = "default",
                 std::chrono::milliseconds connectionTimeout = std::chrono::milliseconds(300),
                 bool connectionHandleError = false, uint64_t clientId = 0,
                 std::unique_ptr<UcxAutoDeviceContext> deviceContext = nullptr);
  // Creates / destroys a shared transport context: the eager and copy limits (from the
  // environment: EUX_EAGER_LIMIT, UCX_RNDV_THRESH) are read once, `printConfig` logs them.
  // `mtWorkersShared` is recorded for parity; every context still owns its worker thread.
  static ucs_status_t init_ucp_context(std::string_view name, ucp_context_h& ucpContext, bool mtWorkersShared = false,
                                       bool printConfig = false);
  static void destroy_ucp_context(ucp_context_h ucpContext);
  ~ucx_am_context();
  ucx_am_context(const ucx_am_context&) = delete;

  // Runs the loop on the calling thread until stop is requested.
  template <class StopToken>
  void run(StopToken token) {
    run_impl([&]() noexcept { return token.stop_requested(); });
  }
  scheduler get_scheduler() noexcept;

  // Opaque endpoint descriptor of this context (host, port, pid, device, name), for connect_endpoint.
  ucs_status_t get_ucp_address(std::vector<std::byte>& address) const;
  // Registers user memory for transfers; `memh` receives the handle to put into ucx_am_data::mem_h.
  ucs_status_t register_ucx_memory(void* ptr, size_t size, void*& memh);
  void unregister_ucx_memory(void* memh);

  // Rendezvous descriptors parked by connection_recv_header, by key.
  const UcxAmDesc* view_pending_am_desc(size_t key) const;
  std::optional<UcxAmDesc> pop_pending_am_desc(size_t key);
  void release_rndv_am_desc(size_t key);

  // Remarks about the device payload of a message that is about to be sent (ucx_send_attr.hpp), filed under
  // the address of the message's header bytes, which no other message in flight shares; the send operation
  // collects them. Any thread. (The C message structs have no room for them.)
  void attach_send_attr(const void* header_data, std::shared_ptr<const UcxSendAttr> attr);
  std::shared_ptr<const UcxSendAttr> take_send_attr(const void* header_data);

  UcxMemoryResourceManager& memory_resource() { return mr_; }
  const std::string& name() const { return name_; }
  bool is_running_on_io_thread() const noexcept { return io_thread_.load(std::memory_order_relaxed) == std::this_thread::get_id(); }
  bool connection_handle_error() const { return handle_errors_; }
  std::chrono::milliseconds connection_timeout() const { return conn_timeout_; }
  ConnectionManager& connections() { return conn_mgr_; }
  transport::Worker& worker() { return *worker_; }
  size_t pending_message_count() const { return am_queue_.size(); }

  // ---- used by the operation states (IO thread unless noted) ----
  void schedule_local(operation_base* op) noexcept;
  void schedule_remote(operation_base* op) noexcept;  // any thread
  void schedule_timer(timer_op* op) noexcept;
  bool cancel_timer(timer_op* op) noexcept;
  void watch_flag(flag_op* op) noexcept;
  bool unwatch_flag(flag_op* op) noexcept;
  void park_recv(parked_op* op) noexcept { park(recv_waiters_head_, recv_waiters_tail_, op); }
  void unpark_recv(parked_op* op) noexcept { unpark(recv_waiters_head_, recv_waiters_tail_, op); }
  void park_accept(parked_op* op) noexcept { park(accept_waiters_head_, accept_waiters_tail_, op); }
  void unpark_accept(parked_op* op) noexcept { unpark(accept_waiters_head_, accept_waiters_tail_, op); }
  void park_error(parked_op* op) noexcept { park(error_waiters_head_, error_waiters_tail_, op); }
  void unpark_error(parked_op* op) noexcept { unpark(error_waiters_head_, error_waiters_tail_, op); }
  std::deque<UcxAmDesc>& am_queue() { return am_queue_; }
  size_t stash_rndv_desc(UcxAmDesc&& d);
  std::deque<transport::ConnRequest>& conn_requests() { return conn_requests_; }
  int start_listening(const sockaddr* addr, socklen_t len);
  int start_listening(port_t port);
  void stop_listening();
  // create + register a connection object for a connect in progress
  UcxConnection* new_connection();
  conn_id_t register_connection(UcxConnection* c);
  void drop_connection(UcxConnection* c);
  int reconnect(const ConnectionManager::FailedConnection& f, UcxCallback* cb, UcxConnection** out);
  bool stopping() const { return stopping_; }
  void push_cqe(const ucx_am_cqe_t& cqe);

 private:
  template <class F>
  void run_impl(F should_stop);
  void run_loop(const std::function<bool()>& should_stop);
  void execute_pending_local() noexcept;
  void acquire_remote_queued_items() noexcept;
  void update_timers() noexcept;
  void poll_flags() noexcept;
  void acquire_completion_queue_items() noexcept;
  void on_am(transport::AmArrival&& a);
  void on_endpoint_error(transport::Endpoint* ep, int status);
  void wake_one(parked_op*& head, parked_op*& tail) noexcept;
  void wake_all(parked_op*& head, parked_op*& tail) noexcept;
  void reject_stale_requests();
  void teardown();
  static void park(parked_op*& head, parked_op*& tail, parked_op* op) noexcept;
  static void unpark(parked_op*& head, parked_op*& tail, parked_op* op) noexcept;

  UcxMemoryResourceManager& mr_;
  std::string name_;
  std::chrono::milliseconds conn_timeout_;
  bool handle_errors_;
  uint64_t client_id_;
  std::unique_ptr<UcxAutoDeviceContext> device_ctx_;
  std::unique_ptr<transport::Worker> worker_;
  std::mutex send_attr_mu_;
  std::unordered_map<const void*, std::shared_ptr<const UcxSendAttr>> send_attrs_;
  std::atomic<size_t> send_attr_count_{0};
  ConnectionManager conn_mgr_;
  std::vector<std::unique_ptr<UcxConnection>> connecting_;  // not yet registered

  std::atomic<std::thread::id> io_thread_{};
  operation_base* local_head_ = nullptr;
  operation_base* local_tail_ = nullptr;
  std::atomic<operation_base*> remote_head_{nullptr};
  std::multimap<time_point, timer_op*> timers_;
  std::vector<flag_op*> flag_ops_;
  ucx_am_cqe_t cq_entries_[kCompletionQueueEntryCount];
  size_t cq_head_ = 0, cq_tail_ = 0;

  std::deque<UcxAmDesc> am_queue_;
  std::unordered_map<size_t, UcxAmDesc> am_desc_map_;
  size_t next_desc_key_ = 1;
  std::deque<transport::ConnRequest> conn_requests_;
  parked_op *recv_waiters_head_ = nullptr, *recv_waiters_tail_ = nullptr;
  parked_op *accept_waiters_head_ = nullptr, *accept_waiters_tail_ = nullptr;
  parked_op *error_waiters_head_ = nullptr, *error_waiters_tail_ = nullptr;
  bool stopping_ = false;
  bool running_ = false;
};

template <class F>
void ucx_am_context::run_impl(F should_stop) {
  std::function<bool()> fn = [&]() { return should_stop(); };
  run_loop(fn);
}

}  // namespace eux::ucxx

#include "eux/ucxx/ucx_am_context_senders.hpp"
