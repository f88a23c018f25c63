#include "eux/ucxx/ucx_am_context.hpp"

#include <arpa/inet.h>
#include <sched.h>

#include <cstdlib>

#include "eux/ucxx/ucx_context_logger.hpp"

namespace eux::ucxx {

ucx_am_context::ucx_am_context(UcxMemoryResourceManager& mr, std::string_view name,
                               std::chrono::milliseconds connectionTimeout, bool connectionHandleError, uint64_t clientId,
                               std::unique_ptr<UcxAutoDeviceContext> deviceContext)
    : mr_(mr), name_(name), conn_timeout_(connectionTimeout), handle_errors_(connectionHandleError), client_id_(clientId),
      device_ctx_(std::move(deviceContext)) {
  std::unique_ptr<OperationRAII> guard;
  if (device_ctx_) guard = (*device_ctx_)();  // the transport is created with the device current
  transport::WorkerOptions opt;
  opt.name = name_;
  opt.client_id = client_id_;
  opt.device = device_ctx_ ? device_ctx_->device_id() : -1;
  worker_ = std::make_unique<transport::Worker>(mr_, opt);
  worker_->on_am = [this](transport::AmArrival&& a) { on_am(std::move(a)); };
  worker_->on_conn_request = [this](transport::ConnRequest&& r) {
    conn_requests_.push_back(std::move(r));
    wake_one(accept_waiters_head_, accept_waiters_tail_);
  };
  worker_->on_auto_accept = [this](transport::Endpoint* ep) {
    auto c = std::make_unique<UcxConnection>(*worker_, handle_errors_);
    c->adopt(ep);
    conn_mgr_.add_connection(std::move(c));
  };
  worker_->on_ep_error = [this](transport::Endpoint* ep, int status) { on_endpoint_error(ep, status); };
}

ucx_am_context::ucx_am_context(UcxMemoryResourceManager& mr, ucp_context_h sharedContext, std::string_view name,
                               std::chrono::milliseconds connectionTimeout, bool connectionHandleError, uint64_t clientId,
                               std::unique_ptr<UcxAutoDeviceContext> deviceContext)
    : ucx_am_context(mr, name, connectionTimeout, connectionHandleError, clientId, std::move(deviceContext)) {
  if (sharedContext) worker_->set_limits(sharedContext->eager_limit, sharedContext->send_copy_limit);
}

ucs_status_t ucx_am_context::init_ucp_context(std::string_view name, ucp_context_h& ucpContext, bool mtWorkersShared,
                                              bool printConfig) {
  auto* c = new eux_shared_transport_context();
  c->name = std::string(name);
  c->mt_workers_shared = mtWorkersShared;
  if (const char* e = std::getenv("EUX_EAGER_LIMIT")) c->eager_limit = std::strtoull(e, nullptr, 10);
  if (const char* e = std::getenv("UCX_RNDV_THRESH")) c->eager_limit = std::strtoull(e, nullptr, 10);
  if (printConfig)
    UCX_CTX_INFO << "shared transport context '" << c->name << "': eager_limit=" << c->eager_limit
                 << " send_copy_limit=" << c->send_copy_limit << " (0 = default)";
  ucpContext = c;
  return UCS_OK;
}

void ucx_am_context::destroy_ucp_context(ucp_context_h ucpContext) { delete ucpContext; }

ucx_am_context::~ucx_am_context() {
  for (auto& [k, d] : am_desc_map_) d.release(mr_);
  for (auto& d : am_queue_) d.release(mr_);
  for (auto& r : conn_requests_) worker_->reject(std::move(r));
  connecting_.clear();
  conn_mgr_.clear();
}

ucx_am_context::scheduler ucx_am_context::get_scheduler() noexcept { return scheduler(this); }

ucs_status_t ucx_am_context::get_ucp_address(std::vector<std::byte>& address) const {
  address = worker_->address().serialize();
  return UCS_OK;
}

void ucx_am_context::attach_send_attr(const void* header_data, std::shared_ptr<const UcxSendAttr> attr) {
  if (!header_data || !attr) return;
  std::lock_guard lk(send_attr_mu_);
  send_attrs_[header_data] = std::move(attr);
  send_attr_count_.store(send_attrs_.size(), std::memory_order_release);
}
std::shared_ptr<const UcxSendAttr> ucx_am_context::take_send_attr(const void* header_data) {
  if (send_attr_count_.load(std::memory_order_acquire) == 0) return nullptr;
  std::lock_guard lk(send_attr_mu_);
  auto it = send_attrs_.find(header_data);
  if (it == send_attrs_.end()) return nullptr;
  auto out = std::move(it->second);
  send_attrs_.erase(it);
  send_attr_count_.store(send_attrs_.size(), std::memory_order_release);
  return out;
}

ucs_status_t ucx_am_context::register_ucx_memory(void* ptr, size_t size, void*& memh) {
  memh = nullptr;
  auto* cuda = dynamic_cast<UcxCudaMemoryResourceManager*>(&mr_);
  if (!cuda) return UCS_OK;  // host memory needs no registration with this transport
  const auto* reg = cuda->register_memory(ptr, size);
  if (!reg) return UCS_ERR_INVALID_ADDR;
  memh = const_cast<void*>(static_cast<const void*>(reg));
  return UCS_OK;
}

void ucx_am_context::unregister_ucx_memory(void* memh) {
  auto* cuda = dynamic_cast<UcxCudaMemoryResourceManager*>(&mr_);
  if (!cuda || !memh) return;
  cuda->unregister_memory(static_cast<const UcxCudaMemoryResourceManager::Registration*>(memh)->base);
}

// ---- queues ---------------------------------------------------------------------------
void ucx_am_context::schedule_local(operation_base* op) noexcept {
  op->next = nullptr;
  if (local_tail_) local_tail_->next = op;
  else local_head_ = op;
  local_tail_ = op;
}

void ucx_am_context::schedule_remote(operation_base* op) noexcept {
  operation_base* head = remote_head_.load(std::memory_order_relaxed);
  do {
    op->next = head;
  } while (!remote_head_.compare_exchange_weak(head, op, std::memory_order_release, std::memory_order_relaxed));
}

void ucx_am_context::acquire_remote_queued_items() noexcept {
  operation_base* list = remote_head_.exchange(nullptr, std::memory_order_acquire);
  // the stack is newest-first; reverse it to keep submission order
  operation_base* rev = nullptr;
  while (list) {
    operation_base* n = list->next;
    list->next = rev;
    rev = list;
    list = n;
  }
  while (rev) {
    operation_base* n = rev->next;
    schedule_local(rev);
    rev = n;
  }
}

void ucx_am_context::execute_pending_local() noexcept {
  // run what is queued now; work queued meanwhile waits for the next turn so the transport is not starved
  operation_base* head = local_head_;
  local_head_ = local_tail_ = nullptr;
  while (head) {
    operation_base* n = head->next;
    head->next = nullptr;
    head->execute(head);
    head = n;
  }
}

void ucx_am_context::schedule_timer(timer_op* op) noexcept {
  op->armed = true;
  timers_.emplace(op->due, op);
}

bool ucx_am_context::cancel_timer(timer_op* op) noexcept {
  if (!op->armed) return false;
  auto range = timers_.equal_range(op->due);
  for (auto it = range.first; it != range.second; ++it) {
    if (it->second == op) {
      timers_.erase(it);
      op->armed = false;
      return true;
    }
  }
  return false;
}

void ucx_am_context::watch_flag(flag_op* op) noexcept {
  op->armed = true;
  flag_ops_.push_back(op);
}

bool ucx_am_context::unwatch_flag(flag_op* op) noexcept {
  if (!op->armed) return false;
  for (auto& slot : flag_ops_) {
    if (slot == op) {
      slot = flag_ops_.back();
      flag_ops_.pop_back();
      op->armed = false;
      return true;
    }
  }
  return false;
}

void ucx_am_context::poll_flags() noexcept {
  for (size_t i = 0; i < flag_ops_.size();) {
    flag_op* op = flag_ops_[i];
    // an acquire load: what the writer stored before the word is visible once the value is seen
    if (__atomic_load_n(const_cast<const uint64_t*>(op->flag), __ATOMIC_ACQUIRE) >= op->at_least) {
      flag_ops_[i] = flag_ops_.back();
      flag_ops_.pop_back();
      op->armed = false;
      schedule_local(op);
    } else {
      ++i;
    }
  }
}

void ucx_am_context::update_timers() noexcept {
  if (timers_.empty()) return;
  // the clock as read by the transport's last progress() call: deadlines are milliseconds, one loop
  // iteration of staleness does not matter, and a clock read per iteration is saved
  const auto now = worker_->last_progress_time();
  while (!timers_.empty() && timers_.begin()->first <= now) {
    timer_op* op = timers_.begin()->second;
    timers_.erase(timers_.begin());
    op->armed = false;
    schedule_local(op);
  }
}

void ucx_am_context::push_cqe(const ucx_am_cqe_t& cqe) {
  if (cq_tail_ - cq_head_ >= kCompletionQueueEntryCount) acquire_completion_queue_items();
  cq_entries_[cq_tail_ % kCompletionQueueEntryCount] = cqe;
  ++cq_tail_;
}

// Completion entries carry a pointer to an operation_base whose execute() reads `res`.
void ucx_am_context::acquire_completion_queue_items() noexcept {
  while (cq_head_ != cq_tail_) {
    const ucx_am_cqe_t& e = cq_entries_[cq_head_ % kCompletionQueueEntryCount];
    ++cq_head_;
    auto* op = reinterpret_cast<operation_base*>(e.user_data);
    if (op) schedule_local(op);
  }
}

void ucx_am_context::park(parked_op*& head, parked_op*& tail, parked_op* op) noexcept {
  op->parked = true;
  op->next_parked = nullptr;
  op->prev_parked = tail;
  if (tail) tail->next_parked = op;
  else head = op;
  tail = op;
}

void ucx_am_context::unpark(parked_op*& head, parked_op*& tail, parked_op* op) noexcept {
  if (!op->parked) return;
  if (op->prev_parked) op->prev_parked->next_parked = op->next_parked;
  else head = op->next_parked;
  if (op->next_parked) op->next_parked->prev_parked = op->prev_parked;
  else tail = op->prev_parked;
  op->parked = false;
  op->prev_parked = op->next_parked = nullptr;
}

void ucx_am_context::wake_one(parked_op*& head, parked_op*& tail) noexcept {
  if (!head) return;
  parked_op* op = head;
  unpark(head, tail, op);
  op->queued = true;
  schedule_local(op);
}

void ucx_am_context::wake_all(parked_op*& head, parked_op*& tail) noexcept {
  while (head) wake_one(head, tail);
}

// ---- transport events -------------------------------------------------------------------
void ucx_am_context::on_am(transport::AmArrival&& a) {
  UcxAmDesc d;
  auto* conn = static_cast<UcxConnection*>(a.ep->user_data);
  d.conn_id = conn ? conn->id() : reinterpret_cast<conn_id_t>(a.ep);
  d.header = a.header;
  d.header_length = a.header_len;
  d.data = a.data;
  d.data_length = a.data_len;
  d.rndv = a.rndv;
  d.msg_id = a.msg_id;
  d.seg_count = a.seg_count;
  d.sender_mem_type = a.sender_mem_type;
  d.data_mem_type = a.data_mem_type;
  d.data_keep = std::move(a.data_keep);
  am_queue_.push_back(d);
  wake_one(recv_waiters_head_, recv_waiters_tail_);
}

void ucx_am_context::on_endpoint_error(transport::Endpoint* ep, int status) {
  auto* conn = static_cast<UcxConnection*>(ep->user_data);
  if (!conn) return;
  const conn_id_t id = conn->id();
  UCX_CTX_DEBUG << name_ << ": connection " << id << " (" << conn->peer_name() << ") failed: " << ucs_status_string(status);
  // messages that were queued from this peer stay readable; rendezvous ones can no longer complete
  if (conn_mgr_.get_connection(id)) {
    if (handle_errors_) {
      conn_mgr_.mark_failed(id, status);
      wake_one(error_waiters_head_, error_waiters_tail_);
    } else {
      conn->mark_failed(status);
      conn_mgr_.deactivate(id);
    }
  }
}

size_t ucx_am_context::stash_rndv_desc(UcxAmDesc&& d) {
  const size_t key = next_desc_key_++;
  am_desc_map_.emplace(key, d);
  return key;
}

const UcxAmDesc* ucx_am_context::view_pending_am_desc(size_t key) const {
  auto it = am_desc_map_.find(key);
  return it == am_desc_map_.end() ? nullptr : &it->second;
}

std::optional<UcxAmDesc> ucx_am_context::pop_pending_am_desc(size_t key) {
  auto it = am_desc_map_.find(key);
  if (it == am_desc_map_.end()) return std::nullopt;
  UcxAmDesc d = it->second;
  am_desc_map_.erase(it);
  return d;
}

void ucx_am_context::release_rndv_am_desc(size_t key) {
  // The descriptor map and the transport belong to the loop's thread. A caller on another
  // thread (an error path of a worker-pool continuation, say) hands the release over to it.
  if (running_ && std::this_thread::get_id() != io_thread_.load(std::memory_order_relaxed)) {
    struct release_op : operation_base {
      ucx_am_context* ctx;
      size_t key;
    };
    auto* op = new release_op();
    op->ctx = this;
    op->key = key;
    op->execute = [](operation_base* b) noexcept {
      auto* self = static_cast<release_op*>(b);
      self->ctx->release_rndv_am_desc(self->key);
      delete self;
    };
    schedule_remote(op);
    return;
  }
  auto d = pop_pending_am_desc(key);
  if (!d) return;
  if (auto* c = conn_mgr_.get_connection(d->conn_id)) c->release_rndv(*d);
  d->release(mr_);
}

// ---- listening / connections ---------------------------------------------------------------
int ucx_am_context::start_listening(const sockaddr* addr, socklen_t len) { return worker_->listen(addr, len); }
int ucx_am_context::start_listening(port_t port) { return worker_->listen(port); }
void ucx_am_context::stop_listening() {
  worker_->stop_listening();
  for (auto& r : conn_requests_) worker_->reject(std::move(r));
  conn_requests_.clear();
}

UcxConnection* ucx_am_context::new_connection() {
  connecting_.push_back(std::make_unique<UcxConnection>(*worker_, handle_errors_));
  return connecting_.back().get();
}

conn_id_t ucx_am_context::register_connection(UcxConnection* c) {
  for (auto it = connecting_.begin(); it != connecting_.end(); ++it) {
    if (it->get() == c) {
      auto owned = std::move(*it);
      connecting_.erase(it);
      return conn_mgr_.add_connection(std::move(owned));
    }
  }
  return 0;
}

void ucx_am_context::drop_connection(UcxConnection* c) {
  for (auto it = connecting_.begin(); it != connecting_.end(); ++it) {
    if (it->get() == c) {
      connecting_.erase(it);
      return;
    }
  }
}

// Reconnect a failed connection from its recorded "ip:port" peer name.
int ucx_am_context::reconnect(const ConnectionManager::FailedConnection& f, UcxCallback* cb, UcxConnection** out) {
  auto colon = f.peer_name.rfind(':');
  if (colon == std::string::npos) return UCS_ERR_INVALID_ADDR;
  sockaddr_in in{};
  in.sin_family = AF_INET;
  if (inet_pton(AF_INET, f.peer_name.substr(0, colon).c_str(), &in.sin_addr) != 1) return UCS_ERR_INVALID_ADDR;
  in.sin_port = htons(static_cast<uint16_t>(std::atoi(f.peer_name.c_str() + colon + 1)));
  UcxConnection* c = new_connection();
  int st = c->connect(nullptr, reinterpret_cast<sockaddr*>(&in), sizeof(in), cb);
  if (st != UCS_INPROGRESS) {
    drop_connection(c);
    return st;
  }
  *out = c;
  return UCS_INPROGRESS;
}

void ucx_am_context::reject_stale_requests() {
  const auto now = std::chrono::steady_clock::now();
  while (!conn_requests_.empty() && now - conn_requests_.front().arrival > conn_timeout_) {
    UCX_CTX_DEBUG << name_ << ": rejecting a connection request older than the connection timeout";
    worker_->reject(std::move(conn_requests_.front()));
    conn_requests_.pop_front();
  }
}

// ---- the loop ------------------------------------------------------------------------------
void ucx_am_context::run_loop(const std::function<bool()>& should_stop) {
  io_thread_.store(std::this_thread::get_id(), std::memory_order_relaxed);
  std::unique_ptr<OperationRAII> guard;
  if (device_ctx_) guard = (*device_ctx_)();  // the device stays current for the whole loop
  running_ = true;
  stopping_ = false;
  unsigned idle = 0;
  const bool spin_only = std::getenv("EUX_BUSY_POLL") != nullptr;
  while (!should_stop()) {
    const bool had_local = local_head_ != nullptr;
    execute_pending_local();
    acquire_completion_queue_items();
    update_timers();
    if (!flag_ops_.empty()) poll_flags();
    acquire_remote_queued_items();
    const int events = worker_->progress();
    if (!conn_requests_.empty()) reject_stale_requests();
    if (events == 0 && !had_local && local_head_ == nullptr) {
      if (++idle > 2000 && !spin_only) sched_yield();
    } else {
      idle = 0;
    }
  }
  teardown();
  running_ = false;
  io_thread_.store(std::thread::id{}, std::memory_order_relaxed);
}

// Stop requested: everything that is parked or queued completes with "done";
// operations submitted from other threads meanwhile are drained for a short grace period.
void ucx_am_context::teardown() {
  stopping_ = true;
  const auto deadline = clock_t::now() + std::chrono::milliseconds(200);
  for (int quiet = 0; quiet < 3 && clock_t::now() < deadline;) {
    wake_all(recv_waiters_head_, recv_waiters_tail_);
    wake_all(accept_waiters_head_, accept_waiters_tail_);
    wake_all(error_waiters_head_, error_waiters_tail_);
    while (!timers_.empty()) {
      timer_op* op = timers_.begin()->second;
      timers_.erase(timers_.begin());
      op->armed = false;
      schedule_local(op);
    }
    while (!flag_ops_.empty()) {
      flag_op* op = flag_ops_.back();
      flag_ops_.pop_back();
      op->armed = false;
      schedule_local(op);
    }
    acquire_remote_queued_items();
    acquire_completion_queue_items();
    const bool any = local_head_ != nullptr;
    execute_pending_local();
    worker_->progress();
    quiet = any ? 0 : quiet + 1;
  }
}

}  // namespace eux::ucxx
