// A pair of single-producer / single-consumer byte rings in a POSIX shared-memory segment: the
// control channel between two workers on the same host once their TCP handshake is done. The
// connecting side creates the segment and offers its name in the HELLO frame; the accepting side
// maps it (which only works on the same host), unlinks the name and says so in its reply; from
// then on both write their frames into the rings and poll them from their progress loop. The TCP
// socket stays open as the liveness signal. The reference gets the same effect from UCX's
// shared-memory transports (posix/sysv/cma) under ucp_am_send_nbx.
//
// Behind the rings the segment holds two pages of 64-bit flag words, one page per direction. A side
// whose worker drives a GPU registers them with CUDA, so that a kernel on its GPU can store a
// sequence number that the peer's *host* thread reads with a plain load: the completion signal of a
// pushed payload crosses process boundaries without a control frame. A second set of words per
// direction is written and read by the two host threads only (receive-ring credits).
#pragma once

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>

namespace eux::ucxx::transport {

struct alignas(64) ShmRing {
  std::atomic<uint64_t> head{0};  // consumer position
  char pad0[56];
  std::atomic<uint64_t> tail{0};  // producer position
  char pad1[56];
};

class ShmChannel {
 public:
  static constexpr uint32_t kMagic = 0x4d485345u;  // "ESHM"
  static constexpr size_t kRingBytes = size_t(2) << 20;
  static constexpr size_t kFlagWords = 512;          // device-written completion words per direction (one page)
  static constexpr size_t kHostWords = 512;          // host-written words per direction (credits and the like)

  // The offering side: creates a fresh segment; the name is what the peer needs to map it.
  static std::unique_ptr<ShmChannel> create(const std::string& name) {
    int fd = ::shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR | O_CLOEXEC, 0600);
    if (fd < 0) return nullptr;
    if (::ftruncate(fd, static_cast<off_t>(total_bytes())) != 0) {
      ::close(fd);
      ::shm_unlink(name.c_str());
      return nullptr;
    }
    auto ch = map(fd, name, true);
    ::close(fd);
    if (!ch) ::shm_unlink(name.c_str());
    return ch;
  }
  // The accepting side: maps an offered segment and removes its name.
  static std::unique_ptr<ShmChannel> open(const std::string& name) {
    int fd = ::shm_open(name.c_str(), O_RDWR | O_CLOEXEC, 0600);
    if (fd < 0) return nullptr;
    struct stat st{};
    // only a segment of this user's own making is mapped: its indices and flag words are taken as they are
    // afterwards, which is more than a stranger on the same host is trusted with (he keeps the socket)
    if (::fstat(fd, &st) != 0 || static_cast<size_t>(st.st_size) != total_bytes() || st.st_uid != ::geteuid()) {
      ::close(fd);
      return nullptr;
    }
    auto ch = map(fd, name, false);
    ::close(fd);
    if (ch && ch->hdr_->magic != kMagic) ch.reset();
    if (ch) ::shm_unlink(name.c_str());
    return ch;
  }
  ~ShmChannel() {
    if (base_) ::munmap(base_, total_bytes());
    if (creator_ && !name_.empty()) ::shm_unlink(name_.c_str());  // harmless when the peer already did
  }
  ShmChannel(const ShmChannel&) = delete;
  ShmChannel& operator=(const ShmChannel&) = delete;
  const std::string& name() const { return name_; }
  bool creator() const { return creator_; }  // this side made the segment (it is the side that connected)

  // Stream semantics, like a non-blocking socket: bytes moved, or -1 with errno = EAGAIN.
  ssize_t write(const void* data, size_t len) {
    ShmRing* r = out_ring();
    const uint64_t tail = r->tail.load(std::memory_order_relaxed);
    const uint64_t head = r->head.load(std::memory_order_acquire);
    const uint64_t used = tail - head;
    if (used > kRingBytes) {  // indices that no honest peer produces: the ring is not written through them
      errno = EIO;
      return -1;
    }
    const size_t room = kRingBytes - static_cast<size_t>(used);
    size_t n = len < room ? len : room;
    if (n == 0) {
      errno = EAGAIN;
      return -1;
    }
    char* buf = out_data();
    const size_t pos = static_cast<size_t>(tail % kRingBytes);
    const size_t first = n < kRingBytes - pos ? n : kRingBytes - pos;
    std::memcpy(buf + pos, data, first);
    if (n > first) std::memcpy(buf, static_cast<const char*>(data) + first, n - first);
    r->tail.store(tail + n, std::memory_order_release);
    return static_cast<ssize_t>(n);
  }
  ssize_t read(void* data, size_t len) {
    ShmRing* r = in_ring();
    const uint64_t head = r->head.load(std::memory_order_relaxed);
    const uint64_t tail = r->tail.load(std::memory_order_acquire);
    if (tail - head > kRingBytes) {  // see write()
      errno = EIO;
      return -1;
    }
    const size_t avail = static_cast<size_t>(tail - head);
    size_t n = len < avail ? len : avail;
    if (n == 0) {
      errno = EAGAIN;
      return -1;
    }
    const char* buf = in_data();
    const size_t pos = static_cast<size_t>(head % kRingBytes);
    const size_t first = n < kRingBytes - pos ? n : kRingBytes - pos;
    std::memcpy(data, buf + pos, first);
    if (n > first) std::memcpy(static_cast<char*>(data) + first, buf, n - first);
    r->head.store(head + n, std::memory_order_release);
    return static_cast<ssize_t>(n);
  }
  // ---- flag pages -------------------------------------------------------------------------
  // Words that this side's GPU writes and the peer's host reads / the other way round.
  volatile uint64_t* out_flags() { return flag_page(creator_ ? 0 : 1); }
  volatile uint64_t* in_flags() { return flag_page(creator_ ? 1 : 0); }
  // Words written by this side's host thread and read by the peer's / the other way round.
  std::atomic<uint64_t>* out_words() { return reinterpret_cast<std::atomic<uint64_t>*>(const_cast<uint64_t*>(flag_page(creator_ ? 2 : 3))); }
  std::atomic<uint64_t>* in_words() { return reinterpret_cast<std::atomic<uint64_t>*>(const_cast<uint64_t*>(flag_page(creator_ ? 3 : 2))); }
  // The page-aligned range that holds the device-written words of both directions (for cudaHostRegister).
  void* flag_area() { return base_ + flags_offset(); }
  static constexpr size_t flag_area_bytes() { return 2 * kPage; }

  bool readable() const {
    const ShmRing* r = const_cast<ShmChannel*>(this)->in_ring();
    return r->tail.load(std::memory_order_acquire) != r->head.load(std::memory_order_relaxed);
  }

 private:
  struct Header {
    uint32_t magic;
    uint32_t ring_bytes;
    char pad[56];
  };
  static constexpr size_t kPage = 4096;
  static_assert(kFlagWords * 8 == kPage && kHostWords * 8 == kPage);
  static size_t flags_offset() { return (sizeof(Header) + 2 * sizeof(ShmRing) + 2 * kRingBytes + kPage - 1) / kPage * kPage; }
  static size_t total_bytes() { return flags_offset() + 4 * kPage; }
  volatile uint64_t* flag_page(int i) { return reinterpret_cast<volatile uint64_t*>(base_ + flags_offset() + size_t(i) * kPage); }
  static std::unique_ptr<ShmChannel> map(int fd, const std::string& name, bool creator) {
    void* p = ::mmap(nullptr, total_bytes(), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    if (p == MAP_FAILED) return nullptr;
    auto ch = std::unique_ptr<ShmChannel>(new ShmChannel());
    ch->base_ = static_cast<char*>(p);
    ch->hdr_ = reinterpret_cast<Header*>(p);
    ch->name_ = name;
    ch->creator_ = creator;
    if (creator) {
      new (ch->ring(0)) ShmRing();
      new (ch->ring(1)) ShmRing();
      ch->hdr_->ring_bytes = static_cast<uint32_t>(kRingBytes);
      std::atomic_thread_fence(std::memory_order_release);
      ch->hdr_->magic = kMagic;
    }
    return ch;
  }
  ShmChannel() = default;
  ShmRing* ring(int i) { return reinterpret_cast<ShmRing*>(base_ + sizeof(Header) + i * sizeof(ShmRing)); }
  char* data(int i) { return base_ + sizeof(Header) + 2 * sizeof(ShmRing) + i * kRingBytes; }
  // ring 0 carries creator -> opener, ring 1 the other way
  ShmRing* out_ring() { return ring(creator_ ? 0 : 1); }
  ShmRing* in_ring() { return ring(creator_ ? 1 : 0); }
  char* out_data() { return data(creator_ ? 0 : 1); }
  const char* in_data() { return data(creator_ ? 1 : 0); }

  char* base_ = nullptr;
  Header* hdr_ = nullptr;
  std::string name_;
  bool creator_ = false;
};

}  // namespace eux::ucxx::transport
