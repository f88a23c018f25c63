#include "eux/ucxx/ucx_connection.hpp"

#include <cstdlib>

namespace eux::ucxx {

void UcxAmDesc::release(UcxMemoryResourceManager& mr) noexcept {
  try {
    if (header) mr.deallocate(ucx_memory_type::HOST, header, header_length);
    if (data && !data_keep) mr.deallocate(ucx_memory_type::HOST, data, data_length);
    data_keep.reset();
  } catch (...) {
  }
  header = data = nullptr;
}

UcxConnection::~UcxConnection() {
  if (ep_) {
    ep_->user_data = nullptr;
    worker_.destroy(ep_);
    ep_ = nullptr;
  }
}

int UcxConnection::connect(const sockaddr* src, const sockaddr* dst, socklen_t len, UcxCallback* cb) {
  int st = UCS_OK;
  ep_ = worker_.connect(dst, len, src, src ? len : 0, [this, cb](int s) {
    status_ = s == UCS_OK ? Status::kConnected : Status::kFailed;
    ucs_status_ = s;
    if (cb) (*cb)(s);
  }, &st);
  if (!ep_) {
    status_ = Status::kFailed;
    ucs_status_ = st;
    return st;
  }
  ep_->user_data = this;
  peer_name_ = ep_->peer_name();
  return UCS_INPROGRESS;
}

int UcxConnection::connect(const transport::WorkerAddress& addr, UcxCallback* cb) {
  int st = UCS_OK;
  ep_ = worker_.connect(addr, [this, cb](int s) {
    status_ = s == UCS_OK ? Status::kConnected : Status::kFailed;
    ucs_status_ = s;
    if (cb) (*cb)(s);
  }, &st);
  if (!ep_) {
    status_ = Status::kFailed;
    ucs_status_ = st;
    return st;
  }
  ep_->user_data = this;
  peer_name_ = ep_->peer_name();
  return UCS_INPROGRESS;
}

int UcxConnection::accept(transport::ConnRequest&& req) {
  int st = UCS_OK;
  ep_ = worker_.accept(std::move(req), &st);
  if (!ep_) {
    status_ = Status::kFailed;
    ucs_status_ = st;
    return st;
  }
  adopt(ep_);
  return UCS_OK;
}

void UcxConnection::adopt(transport::Endpoint* ep) {
  ep_ = ep;
  ep_->user_data = this;
  peer_name_ = ep_->peer_name();
  status_ = Status::kConnected;
}

int UcxConnection::send_am_data(const void* header, size_t header_len, const void* buffer, size_t length,
                                ucx_memory_type_t type, UcxCallback* cb, uint64_t* request_id, std::shared_ptr<const UcxSendAttr> attr) {
  if (!ep_ || status_ != Status::kConnected) return UCS_ERR_NOT_CONNECTED;
  ucx_buffer_t seg{const_cast<void*>(buffer), length};
  return worker_.am_send(ep_, header, header_len, &seg, length ? 1 : 0, type, false,
                         [cb](int s) { if (cb) (*cb)(s); }, request_id, std::move(attr));
}

int UcxConnection::send_am_iov_data(const void* header, size_t header_len, const ucx_buffer_t* iov, size_t count,
                                    ucx_memory_type_t type, UcxCallback* cb, uint64_t* request_id, std::shared_ptr<const UcxSendAttr> attr) {
  if (!ep_ || status_ != Status::kConnected) return UCS_ERR_NOT_CONNECTED;
  // scatter-gather sends always go by rendezvous, like the reference (ucx_connection.cpp:419)
  return worker_.am_send(ep_, header, header_len, iov, count, type, true, [cb](int s) { if (cb) (*cb)(s); }, request_id, std::move(attr));
}

int UcxConnection::recv_am_data(const UcxAmDesc& desc, void* buffer, size_t length, ucx_memory_type_t type, UcxCallback* cb,
                                std::shared_ptr<const UcxSendAttr> attr) {
  if (!ep_ || status_ != Status::kConnected) return UCS_ERR_NOT_CONNECTED;
  ucx_buffer_t seg{buffer, length};
  return worker_.rndv_recv(ep_, desc.msg_id, &seg, 1, type, [cb](int s) { if (cb) (*cb)(s); }, std::move(attr));
}

int UcxConnection::recv_am_iov_data(const UcxAmDesc& desc, const ucx_buffer_t* iov, size_t count, ucx_memory_type_t type,
                                    UcxCallback* cb, std::shared_ptr<const UcxSendAttr> attr) {
  if (!ep_ || status_ != Status::kConnected) return UCS_ERR_NOT_CONNECTED;
  return worker_.rndv_recv(ep_, desc.msg_id, iov, count, type, [cb](int s) { if (cb) (*cb)(s); }, std::move(attr));
}

bool UcxConnection::cancel_send(uint64_t request_id) { return ep_ ? worker_.cancel_send(ep_, request_id) : true; }
bool UcxConnection::cancel_recv(uint64_t msg_id) { return ep_ ? worker_.cancel_recv(ep_, msg_id) : true; }
void UcxConnection::release_rndv(const UcxAmDesc& desc) {
  if (ep_ && desc.rndv) worker_.rndv_discard(ep_, desc.msg_id);
}
std::vector<uint64_t> UcxConnection::rndv_segment_sizes(const UcxAmDesc& desc) const {
  return ep_ ? worker_.rndv_segment_sizes(ep_, desc.msg_id) : std::vector<uint64_t>{};
}

void UcxConnection::disconnect() {
  if (ep_ && (status_ == Status::kConnected || status_ == Status::kConnecting)) {
    status_ = Status::kDisconnecting;
    worker_.close(ep_, true);
  }
  status_ = Status::kClosed;
}

}  // namespace eux::ucxx
