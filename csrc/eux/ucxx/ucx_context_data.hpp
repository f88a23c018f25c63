// Ownership-aware wrappers around the C data model: UcxBuffer, UcxHeader,
// UcxBufferVec, UcxAmData, UcxAmIovec. Each is move-only, knows which memory
// resource manager and memory kind its bytes came from, whether it owns them,
// and optionally a release function that replaces deallocation (used to hand
// ownership back to a transport-owned receive buffer or to drop the Python
// owner of a DLPack tensor). Public surface follows the reference's
// ucx_context/ucx_context_data.hpp:45-986.
#pragma once

#include <functional>
#include <memory>
#include <numeric>
#include <stdexcept>
#include <utility>
#include <vector>

#include "eux/ucxx/ucx_context_def.h"
#include "eux/ucxx/ucx_memory_resource.hpp"
#include "eux/ucxx/ucx_send_attr.hpp"

namespace eux::ucxx {

using ucp_release_fn_t = std::function<void(void*)>;
using MrRef = std::reference_wrapper<UcxMemoryResourceManager>;

class UcxBufferVec;
class UcxAmData;

namespace detail {
// Give back one owned range: the release function wins over the memory resource.
inline void release_range(UcxMemoryResourceManager& mr, ucx_memory_type_t type, ucx_buffer_t& b,
                          const ucp_release_fn_t& fn) noexcept {
  if (!b.data) return;
  try {
    if (fn) fn(b.data);
    else mr.deallocate(type, b.data, b.size);
  } catch (...) {
  }
  b.data = nullptr;
  b.size = 0;
}
}  // namespace detail

class UcxBuffer {
 public:
  // allocate `size` bytes of `type`
  UcxBuffer(MrRef mr, ucx_memory_type_t type, size_t size, void* mem_h = nullptr, bool own_buffer = true,
            ucp_release_fn_t ucp_release_fn = nullptr)
      : mr_(mr), type_(type), buffer_{nullptr, size}, mem_h_(mem_h), own_buffer_(own_buffer),
        ucp_release_fn_(std::move(ucp_release_fn)) {
    if (own_buffer_ && size > 0) buffer_.data = mr_.get().allocate(type_, size);
  }
  // adopt or view existing bytes
  UcxBuffer(MrRef mr, ucx_memory_type_t type, void* data, size_t size, void* mem_h = nullptr, bool own_buffer = true,
            ucp_release_fn_t ucp_release_fn = nullptr)
      : mr_(mr), type_(type), buffer_{data, size}, mem_h_(mem_h), own_buffer_(own_buffer),
        ucp_release_fn_(std::move(ucp_release_fn)) {}
  UcxBuffer(MrRef mr, ucx_memory_type_t type, const ucx_buffer_t& buffer, void* mem_h = nullptr, bool own_buffer = true,
            ucp_release_fn_t ucp_release_fn = nullptr)
      : UcxBuffer(mr, type, buffer.data, buffer.size, mem_h, own_buffer, std::move(ucp_release_fn)) {}

  UcxBuffer(const UcxBuffer&) = delete;
  UcxBuffer& operator=(const UcxBuffer&) = delete;
  UcxBuffer(UcxBuffer&& o) noexcept
      : mr_(o.mr_), type_(o.type_), buffer_(std::exchange(o.buffer_, {nullptr, 0})), mem_h_(std::exchange(o.mem_h_, nullptr)),
        own_buffer_(std::exchange(o.own_buffer_, false)), ucp_release_fn_(std::move(o.ucp_release_fn_)), send_attr_(std::move(o.send_attr_)) {
    o.ucp_release_fn_ = nullptr;
  }
  UcxBuffer& operator=(UcxBuffer&& o) noexcept {
    if (this != &o) {
      reset();
      mr_ = o.mr_;
      type_ = o.type_;
      buffer_ = std::exchange(o.buffer_, {nullptr, 0});
      mem_h_ = std::exchange(o.mem_h_, nullptr);
      own_buffer_ = std::exchange(o.own_buffer_, false);
      ucp_release_fn_ = std::move(o.ucp_release_fn_);
      o.ucp_release_fn_ = nullptr;
      send_attr_ = std::move(o.send_attr_);
    }
    return *this;
  }
  ~UcxBuffer() { reset(); }

  // Optional remarks for the transport when this buffer is sent (a strided layout, an event that says when
  // the bytes are complete); see ucx_send_attr.hpp. size() stays the size of the message.
  void set_send_attr(std::shared_ptr<const UcxSendAttr> a) { send_attr_ = std::move(a); }
  const std::shared_ptr<const UcxSendAttr>& send_attr() const { return send_attr_; }

  ucx_buffer_t* get() { return &buffer_; }
  const ucx_buffer_t* get() const { return &buffer_; }
  void* data() { return buffer_.data; }
  const void* data() const { return buffer_.data; }
  size_t size() const { return buffer_.size; }
  ucx_memory_type_t type() const { return type_; }
  void* mem_h() const { return mem_h_; }
  bool own_buffer() const { return own_buffer_; }
  UcxMemoryResourceManager& mr() const { return mr_.get(); }

  // Give up ownership without freeing; the caller becomes responsible for the bytes.
  ucx_buffer_t release() {
    own_buffer_ = false;
    ucp_release_fn_ = nullptr;
    return std::exchange(buffer_, {nullptr, 0});
  }

  // Split into consecutive views (no copy). The views keep this buffer alive.
  UcxBufferVec to_buffer_vec(const std::vector<size_t>& sizes) &&;

 private:
  friend class UcxBufferVec;
  friend class UcxAmData;
  void reset() noexcept {
    if (own_buffer_) detail::release_range(mr_.get(), type_, buffer_, ucp_release_fn_);
    own_buffer_ = false;
  }
  MrRef mr_;
  ucx_memory_type_t type_;
  ucx_buffer_t buffer_;
  void* mem_h_;
  bool own_buffer_;
  ucp_release_fn_t ucp_release_fn_;
  std::shared_ptr<const UcxSendAttr> send_attr_;
};

// Active-message header bytes: always host memory.
class UcxHeader {
 public:
  explicit UcxHeader(MrRef mr, size_t size = 0, bool own_header = true) : mr_(mr), header_{nullptr, 0}, own_header_(own_header) {
    if (size > 0) {
      header_.data = mr_.get().allocate(ucx_memory_type::HOST, size);
      header_.size = size;
      own_header_ = true;
    }
  }
  UcxHeader(MrRef mr, ucx_header_t&& header, bool own_header = true)
      : mr_(mr), header_(std::exchange(header, {nullptr, 0})), own_header_(own_header) {}
  UcxHeader(MrRef mr, const ucx_header_t& header, bool own_header = false) : mr_(mr), header_(header), own_header_(own_header) {}
  UcxHeader(MrRef mr, void* data, size_t size, bool own_header = false) : mr_(mr), header_{data, size}, own_header_(own_header) {}
  // deep copy of another header
  UcxHeader(const UcxHeader& other, bool own_header) : mr_(other.mr_), header_(other.header_), own_header_(own_header) {
    if (own_header_ && other.header_.data && other.header_.size) {
      header_.data = mr_.get().allocate(ucx_memory_type::HOST, other.header_.size);
      mr_.get().memcpy(ucx_memory_type::HOST, header_.data, ucx_memory_type::HOST, other.header_.data, other.header_.size);
    }
  }
  UcxHeader(const UcxHeader&) = delete;
  UcxHeader& operator=(const UcxHeader&) = delete;
  UcxHeader(UcxHeader&& o) noexcept
      : mr_(o.mr_), header_(std::exchange(o.header_, {nullptr, 0})), own_header_(std::exchange(o.own_header_, false)) {}
  UcxHeader& operator=(UcxHeader&& o) noexcept {
    if (this != &o) {
      reset();
      mr_ = o.mr_;
      header_ = std::exchange(o.header_, {nullptr, 0});
      own_header_ = std::exchange(o.own_header_, false);
    }
    return *this;
  }
  ~UcxHeader() { reset(); }

  ucx_header_t* get() { return &header_; }
  const ucx_buffer_t* get() const { return &header_; }
  void* data() { return header_.data; }
  const void* data() const { return header_.data; }
  size_t size() const { return header_.size; }
  ucx_memory_type_t type() const { return ucx_memory_type::HOST; }
  bool own_buffer() const { return own_header_; }
  bool own_header() const { return own_header_; }
  UcxMemoryResourceManager& mr() const { return mr_.get(); }
  ucx_header_t release() {
    own_header_ = false;
    return std::exchange(header_, {nullptr, 0});
  }

 private:
  void reset() noexcept {
    if (own_header_) detail::release_range(mr_.get(), ucx_memory_type::HOST, header_, nullptr);
    own_header_ = false;
  }
  MrRef mr_;
  ucx_header_t header_;
  bool own_header_;
};

// N payload ranges of one memory kind: either N independent allocations, or N
// views over one backing UcxBuffer.
class UcxBufferVec {
 public:
  UcxBufferVec(MrRef mr, ucx_memory_type_t type, const std::vector<size_t>& sizes, void* mem_h = nullptr,
               bool own_buffer = true, ucp_release_fn_t ucp_release_fn = nullptr)
      : mr_(mr), type_(type), buffers_(sizes.size()), mem_h_(mem_h), own_buffer_(own_buffer),
        ucp_release_fn_(std::move(ucp_release_fn)) {
    for (size_t i = 0; i < sizes.size(); ++i) {
      buffers_[i].size = sizes[i];
      buffers_[i].data = (own_buffer_ && sizes[i]) ? mr_.get().allocate(type_, sizes[i]) : nullptr;
    }
  }
  UcxBufferVec(MrRef mr, ucx_memory_type_t type, std::vector<ucx_buffer_t>&& buffers, void* mem_h = nullptr,
               bool own_buffer = true, ucp_release_fn_t ucp_release_fn = nullptr)
      : mr_(mr), type_(type), buffers_(std::move(buffers)), mem_h_(mem_h), own_buffer_(own_buffer),
        ucp_release_fn_(std::move(ucp_release_fn)) {}
  UcxBufferVec(MrRef mr, ucx_memory_type_t type, const std::vector<ucx_buffer_t>& buffers, void* mem_h = nullptr,
               bool own_buffer = false, ucp_release_fn_t ucp_release_fn = nullptr)
      : mr_(mr), type_(type), buffers_(buffers), mem_h_(mem_h), own_buffer_(own_buffer),
        ucp_release_fn_(std::move(ucp_release_fn)) {}
  // take over independently allocated buffers (all of one kind, one manager)
  explicit UcxBufferVec(std::vector<UcxBuffer>&& buffers)
      : mr_(checked_front(buffers).mr_), type_(buffers.front().type_), mem_h_(buffers.front().mem_h_),
        own_buffer_(buffers.front().own_buffer_), ucp_release_fn_(std::move(buffers.front().ucp_release_fn_)) {
    buffers_.reserve(buffers.size());
    for (auto& b : buffers) {
      if (b.type_ != type_) throw std::invalid_argument("UcxBufferVec: mixed memory types");
      buffers_.push_back(b.release());
    }
    buffers.clear();
  }
  explicit UcxBufferVec(UcxBuffer&& buffer)
      : mr_(buffer.mr_), type_(buffer.type_), mem_h_(buffer.mem_h_), own_buffer_(buffer.own_buffer_),
        ucp_release_fn_(std::move(buffer.ucp_release_fn_)) {
    buffers_.push_back(buffer.release());
  }

  UcxBufferVec(const UcxBufferVec&) = delete;
  UcxBufferVec& operator=(const UcxBufferVec&) = delete;
  UcxBufferVec(UcxBufferVec&& o) noexcept
      : mr_(o.mr_), type_(o.type_), buffers_(std::move(o.buffers_)), mem_h_(std::exchange(o.mem_h_, nullptr)),
        own_buffer_(std::exchange(o.own_buffer_, false)), ucp_release_fn_(std::move(o.ucp_release_fn_)),
        backing_buffer_(std::move(o.backing_buffer_)), send_attr_(std::move(o.send_attr_)) {
    o.buffers_.clear();
    o.ucp_release_fn_ = nullptr;
  }
  UcxBufferVec& operator=(UcxBufferVec&& o) noexcept {
    if (this != &o) {
      reset();
      mr_ = o.mr_;
      type_ = o.type_;
      buffers_ = std::move(o.buffers_);
      o.buffers_.clear();
      mem_h_ = std::exchange(o.mem_h_, nullptr);
      own_buffer_ = std::exchange(o.own_buffer_, false);
      ucp_release_fn_ = std::move(o.ucp_release_fn_);
      o.ucp_release_fn_ = nullptr;
      backing_buffer_ = std::move(o.backing_buffer_);
      send_attr_ = std::move(o.send_attr_);
    }
    return *this;
  }
  ~UcxBufferVec() { reset(); }

  // As for UcxBuffer; of a vector only the event is looked at (every range is dense).
  void set_send_attr(std::shared_ptr<const UcxSendAttr> a) { send_attr_ = std::move(a); }
  const std::shared_ptr<const UcxSendAttr>& send_attr() const { return send_attr_; }

  std::vector<void*> data_ptrs() {
    std::vector<void*> out;
    out.reserve(buffers_.size());
    for (auto& b : buffers_) out.push_back(b.data);
    return out;
  }
  std::vector<const void*> data_ptrs() const {
    std::vector<const void*> out;
    out.reserve(buffers_.size());
    for (auto& b : buffers_) out.push_back(b.data);
    return out;
  }
  std::vector<size_t> data_sizes() const {
    std::vector<size_t> out;
    out.reserve(buffers_.size());
    for (auto& b : buffers_) out.push_back(b.size);
    return out;
  }
  size_t total_size() const {
    return std::accumulate(buffers_.begin(), buffers_.end(), size_t{0}, [](size_t a, const ucx_buffer_t& b) { return a + b.size; });
  }
  void* data() { return buffers_.data(); }
  const void* data() const { return buffers_.data(); }
  size_t size() const { return buffers_.size(); }
  bool empty() const { return buffers_.empty(); }
  auto begin() { return buffers_.begin(); }
  auto begin() const { return buffers_.begin(); }
  auto end() { return buffers_.end(); }
  auto end() const { return buffers_.end(); }
  ucx_buffer_t& operator[](size_t i) { return buffers_[i]; }
  const ucx_buffer_t& operator[](size_t i) const { return buffers_[i]; }
  ucx_buffer_t& at(size_t i) { return buffers_.at(i); }
  const ucx_buffer_t& at(size_t i) const { return buffers_.at(i); }
  std::vector<ucx_buffer_t>& buffers() { return buffers_; }
  const std::vector<ucx_buffer_t>& buffers() const { return buffers_; }
  ucx_memory_type_t type() const { return type_; }
  void* mem_h() const { return mem_h_; }
  bool own_buffer() const { return own_buffer_; }
  bool has_backing_buffer() const { return backing_buffer_ != nullptr; }
  UcxMemoryResourceManager& mr() const { return mr_.get(); }

  // Turn an independently allocated vector into individual buffers (ownership moves).
  std::vector<UcxBuffer> ExtractBuffers() && {
    if (backing_buffer_) throw std::logic_error("ExtractBuffers() needs independently allocated ranges, not views of one buffer");
    std::vector<UcxBuffer> out;
    out.reserve(buffers_.size());
    for (auto& b : buffers_) out.emplace_back(mr_, type_, b, mem_h_, own_buffer_, ucp_release_fn_);
    own_buffer_ = false;
    buffers_.clear();
    return out;
  }

 private:
  friend class UcxBuffer;
  static UcxBuffer& checked_front(std::vector<UcxBuffer>& v) {
    if (v.empty()) throw std::invalid_argument("UcxBufferVec: empty buffer list");
    return v.front();
  }
  UcxBufferVec(MrRef mr, ucx_memory_type_t type, std::vector<ucx_buffer_t>&& views, void* mem_h,
               std::unique_ptr<UcxBuffer>&& backing)
      : mr_(mr), type_(type), buffers_(std::move(views)), mem_h_(mem_h), own_buffer_(false), backing_buffer_(std::move(backing)) {}
  void reset() noexcept {
    if (own_buffer_)
      for (auto& b : buffers_) detail::release_range(mr_.get(), type_, b, ucp_release_fn_);
    own_buffer_ = false;
    buffers_.clear();
    backing_buffer_.reset();
  }
  MrRef mr_;
  ucx_memory_type_t type_;
  std::vector<ucx_buffer_t> buffers_;
  void* mem_h_;
  bool own_buffer_;
  ucp_release_fn_t ucp_release_fn_;
  std::unique_ptr<UcxBuffer> backing_buffer_;
  std::shared_ptr<const UcxSendAttr> send_attr_;
};

inline UcxBufferVec UcxBuffer::to_buffer_vec(const std::vector<size_t>& sizes) && {
  const size_t total = std::accumulate(sizes.begin(), sizes.end(), size_t{0});
  if (total > buffer_.size) throw std::length_error("to_buffer_vec: the chunks need more bytes than the buffer holds");
  std::vector<ucx_buffer_t> views;
  views.reserve(sizes.size());
  char* p = static_cast<char*>(buffer_.data);
  for (size_t n : sizes) {
    views.push_back({p, n});
    p += n;
  }
  MrRef mr = mr_;
  ucx_memory_type_t type = type_;
  void* memh = mem_h_;
  auto backing = std::make_unique<UcxBuffer>(std::move(*this));
  return UcxBufferVec(mr, type, std::move(views), memh, std::move(backing));
}

// One active message with a contiguous payload.
class UcxAmData {
 public:
  UcxAmData(MrRef mr, size_t header_size, size_t buffer_size, ucx_memory_type_t buffer_type, bool own_header = true,
            bool own_buffer = true, ucp_release_fn_t ucp_release_fn = nullptr)
      : mr_(mr), data_{}, own_header_(own_header), own_buffer_(own_buffer), ucp_release_fn_(std::move(ucp_release_fn)) {
    data_.buffer_type = buffer_type;
    if (header_size > 0 && own_header_) {
      data_.header.data = mr_.get().allocate(ucx_memory_type::HOST, header_size);
      data_.header.size = header_size;
    }
    data_.buffer.size = buffer_size;  // a non-owning message still says how much it expects
    if (buffer_size > 0 && own_buffer_) data_.buffer.data = mr_.get().allocate(buffer_type, buffer_size);
  }
  UcxAmData(MrRef mr, ucx_am_data_t&& data, bool own_header = true, bool own_buffer = true,
            ucp_release_fn_t ucp_release_fn = nullptr)
      : mr_(mr), data_(std::exchange(data, ucx_am_data_t{})), own_header_(own_header), own_buffer_(own_buffer),
        ucp_release_fn_(std::move(ucp_release_fn)) {}
  UcxAmData(MrRef mr, const ucx_am_data_t& data, bool own_header = false, bool own_buffer = false,
            ucp_release_fn_t ucp_release_fn = nullptr)
      : mr_(mr), data_(data), own_header_(own_header), own_buffer_(own_buffer), ucp_release_fn_(std::move(ucp_release_fn)) {}
  // assemble from a header and a buffer (both give up their bytes)
  UcxAmData(MrRef mr, UcxHeader&& header, UcxBuffer&& buffer)
      : mr_(mr), data_{}, own_header_(header.own_header()), own_buffer_(buffer.own_buffer()),
        ucp_release_fn_(std::move(buffer.ucp_release_fn_)) {
    data_.buffer_type = buffer.type();
    data_.mem_h = buffer.mem_h();
    data_.header = header.release();
    data_.buffer = buffer.release();
  }
  UcxAmData(const UcxAmData&) = delete;
  UcxAmData& operator=(const UcxAmData&) = delete;
  UcxAmData(UcxAmData&& o) noexcept
      : mr_(o.mr_), data_(std::exchange(o.data_, ucx_am_data_t{})), own_header_(std::exchange(o.own_header_, false)),
        own_buffer_(std::exchange(o.own_buffer_, false)), ucp_release_fn_(std::move(o.ucp_release_fn_)) {
    o.ucp_release_fn_ = nullptr;
  }
  UcxAmData& operator=(UcxAmData&& o) noexcept {
    if (this != &o) {
      reset();
      mr_ = o.mr_;
      data_ = std::exchange(o.data_, ucx_am_data_t{});
      own_header_ = std::exchange(o.own_header_, false);
      own_buffer_ = std::exchange(o.own_buffer_, false);
      ucp_release_fn_ = std::move(o.ucp_release_fn_);
      o.ucp_release_fn_ = nullptr;
    }
    return *this;
  }
  ~UcxAmData() { reset(); }

  ucx_am_data_t* get() { return &data_; }
  const ucx_am_data_t* get() const { return &data_; }
  bool owns_header() const { return own_header_; }
  bool own_buffer() const { return own_buffer_; }
  UcxMemoryResourceManager& mr() const { return mr_.get(); }
  // Only a message that does not yet have a release function accepts one.
  bool set_ucp_release_fn(ucp_release_fn_t&& fn) {
    if (ucp_release_fn_) return false;
    ucp_release_fn_ = std::move(fn);
    return true;
  }
  // Split into its two parts; ownership follows.
  UcxHeader move_header() {
    bool own = std::exchange(own_header_, false);
    return UcxHeader(mr_, std::exchange(data_.header, {nullptr, 0}), own);
  }
  UcxBuffer move_buffer() {
    bool own = std::exchange(own_buffer_, false);
    auto fn = std::move(ucp_release_fn_);
    ucp_release_fn_ = nullptr;
    return UcxBuffer(mr_, data_.buffer_type, std::exchange(data_.buffer, {nullptr, 0}), data_.mem_h, own, std::move(fn));
  }

 private:
  void reset() noexcept {
    if (own_header_) detail::release_range(mr_.get(), ucx_memory_type::HOST, data_.header, nullptr);
    if (own_buffer_) detail::release_range(mr_.get(), data_.buffer_type, data_.buffer, ucp_release_fn_);
    own_header_ = own_buffer_ = false;
  }
  MrRef mr_;
  ucx_am_data_t data_;
  bool own_header_;
  bool own_buffer_;
  ucp_release_fn_t ucp_release_fn_;
};

// One active message with a scatter-gather payload.
class UcxAmIovec {
 public:
  UcxAmIovec(MrRef mr, size_t header_size, const std::vector<size_t>& buffer_sizes, ucx_memory_type_t buffer_type,
             bool own_header = true, bool own_buffer = true)
      : mr_(mr), iovec_{}, own_header_(own_header), own_buffer_(own_buffer) {
    iovec_.buffer_type = buffer_type;
    if (header_size > 0 && own_header_) {
      iovec_.header.data = mr_.get().allocate(ucx_memory_type::HOST, header_size);
      iovec_.header.size = header_size;
    }
    iovec_.buffer_count = buffer_sizes.size();
    if (iovec_.buffer_count) {
      iovec_.buffer_vec = static_cast<ucx_buffer_t*>(
          mr_.get().allocate(ucx_memory_type::HOST, sizeof(ucx_buffer_t) * iovec_.buffer_count, alignof(ucx_buffer_t)));
      own_vec_ = true;
      for (size_t i = 0; i < iovec_.buffer_count; ++i) {
        iovec_.buffer_vec[i].size = buffer_sizes[i];
        iovec_.buffer_vec[i].data = (own_buffer_ && buffer_sizes[i]) ? mr_.get().allocate(buffer_type, buffer_sizes[i]) : nullptr;
      }
    }
  }
  UcxAmIovec(MrRef mr, ucx_am_iovec_t&& iovec, bool own_header = true, bool own_buffer = true)
      : mr_(mr), iovec_(std::exchange(iovec, ucx_am_iovec_t{})), own_header_(own_header), own_buffer_(own_buffer),
        own_vec_(own_buffer) {}
  UcxAmIovec(MrRef mr, const ucx_am_iovec_t& iovec, bool own_header = false, bool own_buffer = false)
      : mr_(mr), iovec_(iovec), own_header_(own_header), own_buffer_(own_buffer), own_vec_(false) {}
  // assemble from a header and a buffer vector: the element array is copied, the ranges are taken over
  UcxAmIovec(MrRef mr, UcxHeader&& header, UcxBufferVec&& vec)
      : mr_(mr), iovec_{}, own_header_(header.own_header()), own_buffer_(vec.own_buffer()) {
    iovec_.buffer_type = vec.type();
    iovec_.mem_h = vec.mem_h();
    iovec_.header = header.release();
    iovec_.buffer_count = vec.size();
    if (iovec_.buffer_count) {
      iovec_.buffer_vec = static_cast<ucx_buffer_t*>(
          mr_.get().allocate(ucx_memory_type::HOST, sizeof(ucx_buffer_t) * iovec_.buffer_count, alignof(ucx_buffer_t)));
      own_vec_ = true;
      for (size_t i = 0; i < iovec_.buffer_count; ++i) iovec_.buffer_vec[i] = vec[i];
    }
    keep_ = std::make_unique<UcxBufferVec>(std::move(vec));  // keeps a backing buffer / release function alive
    own_buffer_ = false;
  }
  UcxAmIovec(const UcxAmIovec&) = delete;
  UcxAmIovec& operator=(const UcxAmIovec&) = delete;
  UcxAmIovec(UcxAmIovec&& o) noexcept
      : mr_(o.mr_), iovec_(std::exchange(o.iovec_, ucx_am_iovec_t{})), own_header_(std::exchange(o.own_header_, false)),
        own_buffer_(std::exchange(o.own_buffer_, false)), own_vec_(std::exchange(o.own_vec_, false)), keep_(std::move(o.keep_)) {}
  UcxAmIovec& operator=(UcxAmIovec&& o) noexcept {
    if (this != &o) {
      reset();
      mr_ = o.mr_;
      iovec_ = std::exchange(o.iovec_, ucx_am_iovec_t{});
      own_header_ = std::exchange(o.own_header_, false);
      own_buffer_ = std::exchange(o.own_buffer_, false);
      own_vec_ = std::exchange(o.own_vec_, false);
      keep_ = std::move(o.keep_);
    }
    return *this;
  }
  ~UcxAmIovec() { reset(); }

  ucx_am_iovec_t* get() { return &iovec_; }
  const ucx_am_iovec_t* get() const { return &iovec_; }
  bool owns_header() const { return own_header_; }
  bool own_buffer() const { return own_buffer_; }
  UcxMemoryResourceManager& mr() const { return mr_.get(); }
  UcxHeader move_header() {
    bool own = std::exchange(own_header_, false);
    return UcxHeader(mr_, std::exchange(iovec_.header, {nullptr, 0}), own);
  }
  UcxBufferVec move_buffers() {
    if (keep_) {
      auto v = std::move(*keep_);
      keep_.reset();
      return v;
    }
    std::vector<ucx_buffer_t> ranges(iovec_.buffer_vec, iovec_.buffer_vec + iovec_.buffer_count);
    bool own = std::exchange(own_buffer_, false);
    return UcxBufferVec(mr_, iovec_.buffer_type, std::move(ranges), iovec_.mem_h, own);
  }

 private:
  void reset() noexcept {
    if (own_header_) detail::release_range(mr_.get(), ucx_memory_type::HOST, iovec_.header, nullptr);
    if (iovec_.buffer_vec) {
      if (own_buffer_)
        for (size_t i = 0; i < iovec_.buffer_count; ++i)
          detail::release_range(mr_.get(), iovec_.buffer_type, iovec_.buffer_vec[i], nullptr);
      if (own_vec_) {
        try {
          mr_.get().deallocate(ucx_memory_type::HOST, iovec_.buffer_vec, sizeof(ucx_buffer_t) * iovec_.buffer_count,
                               alignof(ucx_buffer_t));
        } catch (...) {
        }
      }
    }
    iovec_ = ucx_am_iovec_t{};
    own_header_ = own_buffer_ = own_vec_ = false;
    keep_.reset();
  }
  MrRef mr_;
  ucx_am_iovec_t iovec_;
  bool own_header_;
  bool own_buffer_;
  bool own_vec_ = false;
  std::unique_ptr<UcxBufferVec> keep_;
};

}  // namespace eux::ucxx
