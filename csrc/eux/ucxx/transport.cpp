#include "eux/ucxx/transport.hpp"

#include <arpa/inet.h>
#include <cuda_runtime_api.h>
#include <errno.h>
#include <fcntl.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/epoll.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/uio.h>
#include <sys/un.h>
#include <unistd.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <random>

#include "eux/ucxx/nvtx_range.hpp"
#include "eux/ucxx/ucx_context_logger.hpp"
#include "kernels/eux_kernels.h"

namespace eux::ucxx::transport {

namespace {

int set_nonblocking(int fd) {
  int fl = fcntl(fd, F_GETFL, 0);
  return fl < 0 ? -1 : fcntl(fd, F_SETFL, fl | O_NONBLOCK);
}
void tune_socket(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  int big = 4 << 20;
  setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &big, sizeof(big));
  setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &big, sizeof(big));
}
std::string sockaddr_to_string(const sockaddr* sa) {
  char buf[INET6_ADDRSTRLEN] = {0};
  if (sa->sa_family == AF_INET) {
    auto* in = reinterpret_cast<const sockaddr_in*>(sa);
    inet_ntop(AF_INET, &in->sin_addr, buf, sizeof(buf));
    return std::string(buf) + ":" + std::to_string(ntohs(in->sin_port));
  }
  if (sa->sa_family == AF_INET6) {
    auto* in6 = reinterpret_cast<const sockaddr_in6*>(sa);
    inet_ntop(AF_INET6, &in6->sin6_addr, buf, sizeof(buf));
    return std::string(buf) + ":" + std::to_string(ntohs(in6->sin6_port));
  }
  return "unknown";
}
std::string peer_of(int fd) {
  sockaddr_storage ss{};
  socklen_t len = sizeof(ss);
  if (getpeername(fd, reinterpret_cast<sockaddr*>(&ss), &len) != 0) return "unknown";
  return sockaddr_to_string(reinterpret_cast<sockaddr*>(&ss));
}
uint64_t random_uid() {
  std::random_device rd;
  return (uint64_t(rd()) << 32) ^ rd() ^ (uint64_t(getpid()) << 17);
}
bool is_device_type(ucx_memory_type_t t) { return t == ucx_memory_type::CUDA || t == ucx_memory_type::CUDA_MANAGED; }

// Large pushes of every worker of this process that target memory through one GPU leave through one
// stream per device, in the order in which they were asked for. Two workers (a runtime's client and server
// side) that push in the same direction at the same time would otherwise share the link, and the transfer
// that the peer is waiting for would take twice as long; one after the other, each runs at the full rate
// and the first is done in half the time.
std::mutex g_bulk_mu;
std::unordered_map<int, cudaStream_t> g_bulk_streams;
cudaStream_t bulk_stream_for(int device) {
  std::lock_guard lk(g_bulk_mu);
  auto it = g_bulk_streams.find(device);
  if (it != g_bulk_streams.end()) return it->second;
  cudaStream_t st = nullptr;
  int prev = -1;
  cudaGetDevice(&prev);
  if (cudaSetDevice(device) != cudaSuccess || cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess) {
    cudaGetLastError();
    st = nullptr;
  }
  if (prev >= 0 && prev != device) cudaSetDevice(prev);
  if (st) g_bulk_streams.emplace(device, st);  // lives as long as the process
  return st;
}

// Workers alive in this process, by their random uid. A peer is "this process" only when the uid it
// presented in the handshake is found here: a pid alone says nothing (two containers, pid namespaces
// or hosts routinely share one), and it arrives from the wire.
std::mutex g_live_mu;
std::unordered_map<uint64_t, int> g_live_uids;
void live_add(uint64_t uid) {
  std::lock_guard lk(g_live_mu);
  ++g_live_uids[uid];
}
void live_remove(uint64_t uid) {
  std::lock_guard lk(g_live_mu);
  auto it = g_live_uids.find(uid);
  if (it != g_live_uids.end() && --it->second <= 0) g_live_uids.erase(it);
}
bool live_has(uint64_t uid) {
  std::lock_guard lk(g_live_mu);
  return g_live_uids.count(uid) != 0;
}

// Limits on what a frame may claim. One frame from an unauthenticated socket must not be able to make
// the receiver buffer or allocate without bound.
constexpr size_t kMaxSegCount = 4096;                // scatter-gather segments per message
constexpr uint64_t kFdListenerTag = 0xfffffffeu;     // epoll tag of the Unix socket on which descriptor channels are accepted
// Device regions announced in an RTS: one per allocation that the payload touches. A sender that does
// not say how many (status 0) describes one per segment.
inline size_t rts_region_count(const FrameHeader& fh) {
  if (!(fh.flags & kFlagDeviceRegions)) return 0;
  return fh.status > 0 ? static_cast<size_t>(fh.status) : static_cast<size_t>(fh.seg_count);
}
constexpr size_t kMinInlineCap = size_t(16) << 20;   // inline payloads: the larger of this and the eager limit

// Device channel geometry. The shared flag page of a direction (512 words) is split: the first 256 words
// signal pushed rendezvous payloads (the receiver picks the word), the next kEagerSlots the eager ring's slots.
constexpr uint32_t kPushWords = 256;
constexpr uint32_t kEagerSlots = 32;                 // one bit each in a 64-bit free mask
constexpr uint32_t kEagerSlotBytesMax = 1 << 20;     // largest slot
constexpr uint32_t kEagerRunMax = 16;                // an eager payload may take up to this many consecutive slots (half the ring)
constexpr uint32_t kEagerRunSizing = 4;              // a payload at the limit takes this many slots, as far as the largest slot allows
constexpr uint32_t kEagerBatchBytes = 64 << 10;      // eager payloads up to here share one launch per pass; larger ones get a launch of several CTAs
// Slot size for a worker whose eager limit is `limit`: a quarter of it (a payload at the limit takes a run of
// kEagerRunSizing slots), at least 4 KiB and at most kEagerSlotBytesMax, a power of two. A limit above four of
// the largest slots keeps that slot size and lets a payload take a longer run, up to kEagerRunMax.
inline uint32_t eager_slot_bytes(size_t limit) {
  uint32_t b = 4096;
  while (size_t(b) * kEagerRunSizing < limit && b < kEagerSlotBytesMax) b <<= 1;
  return b;
}
// The longest run a ring of these slots takes: rings of smaller slots were sized for a smaller limit and keep it.
inline uint32_t eager_run_max(uint32_t slot_bytes) { return slot_bytes < kEagerSlotBytesMax ? kEagerRunSizing : kEagerRunMax; }
constexpr uint32_t kEagerWordBase = kPushWords;
static_assert(kEagerWordBase + kEagerSlots <= ShmChannel::kFlagWords);
constexpr auto kEagerArrivalTimeout = std::chrono::seconds(10);
constexpr auto kHeldSendTimeout = std::chrono::seconds(60);   // how long an announcement waits for its payload's producer

// HELLO / HELLO_ACK body: u64 client id, then the worker address (fixed 60-byte form)
constexpr size_t kAddrWire = 4 + 4 + 2 + 2 + 4 + 4 + 8 + 32;

void put_addr(char* p, const WorkerAddress& a) {
  std::memcpy(p, &a.magic, 4);
  std::memcpy(p + 4, &a.ipv4, 4);
  std::memcpy(p + 8, &a.port, 2);
  std::memcpy(p + 10, &a.reserved, 2);
  std::memcpy(p + 12, &a.pid, 4);
  std::memcpy(p + 16, &a.device, 4);
  std::memcpy(p + 20, &a.uid, 8);
  std::memcpy(p + 28, a.name, 32);
}
bool get_addr(const char* p, size_t n, WorkerAddress* a) {
  if (n < kAddrWire) return false;
  std::memcpy(&a->magic, p, 4);
  std::memcpy(&a->ipv4, p + 4, 4);
  std::memcpy(&a->port, p + 8, 2);
  std::memcpy(&a->reserved, p + 10, 2);
  std::memcpy(&a->pid, p + 12, 4);
  std::memcpy(&a->device, p + 16, 4);
  std::memcpy(&a->uid, p + 20, 8);
  std::memcpy(a->name, p + 28, 32);
  a->name[31] = 0;
  return a->magic == WorkerAddress{}.magic;
}

}  // namespace

std::vector<std::byte> WorkerAddress::serialize() const {
  std::vector<std::byte> out(kAddrWire);
  put_addr(reinterpret_cast<char*>(out.data()), *this);
  return out;
}
bool WorkerAddress::parse(const std::byte* p, size_t n, WorkerAddress* out) {
  return get_addr(reinterpret_cast<const char*>(p), n, out);
}

// ---------------------------------------------------------------------------
// construction / listeners
// ---------------------------------------------------------------------------
Worker::Worker(UcxMemoryResourceManager& mr, const WorkerOptions& opt) : mr_(mr), opt_(opt) {
  cuda_mr_ = dynamic_cast<UcxCudaMemoryResourceManager*>(&mr_);
  if (const char* e = std::getenv("EUX_EAGER_LIMIT")) opt_.eager_limit = std::strtoull(e, nullptr, 10);
  if (const char* e = std::getenv("UCX_RNDV_THRESH")) {
    // honoured for parity with the reference's test environment (ucx_am_connection_test.cpp:70-71)
    char* end = nullptr;
    unsigned long long v = std::strtoull(e, &end, 10);
    if (end != e && v > 0) opt_.eager_limit = v;
  }
  if (const char* e = std::getenv("EUX_SHM")) opt_.use_shm = e[0] != '0';
  if (const char* e = std::getenv("EUX_DEV_EAGER_LIMIT")) opt_.dev_eager_limit = std::strtoull(e, nullptr, 10);
  if (const char* e = std::getenv("EUX_PUSH_THRESH")) opt_.push_threshold = std::strtoull(e, nullptr, 10);
  if (opt_.dev_eager_limit > size_t(kEagerSlotBytesMax) * kEagerRunMax) opt_.dev_eager_limit = size_t(kEagerSlotBytesMax) * kEagerRunMax;
  epfd_ = epoll_create1(EPOLL_CLOEXEC);
  if (epfd_ < 0) throw std::system_error(errno, std::generic_category(), "epoll_create1");
  addr_.pid = static_cast<uint32_t>(getpid());
  addr_.device = opt_.device;
  addr_.uid = random_uid();
  live_add(addr_.uid);
  std::strncpy(addr_.name, opt_.name.c_str(), sizeof(addr_.name) - 1);
  if (cuda_mr_ && opt_.use_shm) open_fd_listener();
  // implicit listener: makes the worker reachable through its address blob. Nobody is authenticated on it,
  // so it listens on the loopback interface unless the worker is told to advertise another address
  // (EUX_ADVERTISE_IP: workers on several hosts), and then on all interfaces.
  sockaddr_in in{};
  in.sin_family = AF_INET;
  in.sin_addr.s_addr = htonl(std::getenv("EUX_ADVERTISE_IP") ? INADDR_ANY : INADDR_LOOPBACK);
  in.sin_port = 0;
  if (listen(reinterpret_cast<sockaddr*>(&in), sizeof(in)) == UCS_OK) {
    listeners_.back().implicit = true;
    sockaddr_in bound{};
    socklen_t len = sizeof(bound);
    getsockname(listeners_.back().fd, reinterpret_cast<sockaddr*>(&bound), &len);
    addr_.port = ntohs(bound.sin_port);
    addr_.ipv4 = htonl(INADDR_LOOPBACK);
    if (const char* ip = std::getenv("EUX_ADVERTISE_IP")) {
      in_addr a{};
      if (inet_pton(AF_INET, ip, &a) == 1) addr_.ipv4 = a.s_addr;
    }
  }
}

Worker::~Worker() {
  live_remove(addr_.uid);
  for (auto& [p, ep] : eps_) teardown_device_channel(p);
  for (auto& [p, ep] : eps_) close_fd_channel(p);
  if (fd_listen_ >= 0) {
    ::close(fd_listen_);
    ::unlink(fd_path_.c_str());
  }
  for (auto& [p, ep] : eps_)
    if (ep->fd_ >= 0) ::close(ep->fd_);
  for (auto& l : listeners_)
    if (l.fd >= 0) ::close(l.fd);
  for (auto& h : hellos_) ::close(h.fd);
  if (epfd_ >= 0) ::close(epfd_);
  if (device_ready_) {
    if (stream_) cudaStreamSynchronize(static_cast<cudaStream_t>(stream_));
    if (stream_) cudaStreamDestroy(static_cast<cudaStream_t>(stream_));
    if (flag_host_) cudaFreeHost(flag_host_);
    if (counter_dev_) cudaFree(counter_dev_);
  }
}

int Worker::listen(const sockaddr* addr, socklen_t len) {
  int fd = ::socket(addr->sa_family, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) return UCS_ERR_IO_ERROR;
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  if (::bind(fd, addr, len) != 0 || ::listen(fd, 256) != 0 || set_nonblocking(fd) != 0) {
    int e = errno;
    ::close(fd);
    return e == EADDRINUSE ? UCS_ERR_BUSY : UCS_ERR_IO_ERROR;
  }
  epoll_event ev{};
  ev.events = EPOLLIN;
  ev.data.u64 = (uint64_t(1) << 63) | uint64_t(listeners_.size());
  if (epoll_ctl(epfd_, EPOLL_CTL_ADD, fd, &ev) != 0) {
    ::close(fd);
    return UCS_ERR_IO_ERROR;
  }
  listeners_.push_back({fd, false});
  return UCS_OK;
}

int Worker::listen(uint16_t port) {
  sockaddr_in in{};
  in.sin_family = AF_INET;
  in.sin_addr.s_addr = htonl(INADDR_ANY);
  in.sin_port = htons(port);
  return listen(reinterpret_cast<sockaddr*>(&in), sizeof(in));
}

void Worker::stop_listening() {
  for (auto& l : listeners_) {
    if (l.implicit || l.fd < 0) continue;
    epoll_ctl(epfd_, EPOLL_CTL_DEL, l.fd, nullptr);
    ::close(l.fd);
    l.fd = -1;
  }
}

Endpoint* Worker::new_endpoint(int fd) {
  auto ep = std::make_unique<Endpoint>();
  ep->worker_ = this;
  ep->fd_ = fd;
  Endpoint* raw = ep.get();
  eps_.emplace(raw, std::move(ep));
  epoll_event ev{};
  ev.events = EPOLLIN | EPOLLOUT | EPOLLRDHUP | EPOLLET;
  ev.data.ptr = raw;
  epoll_ctl(epfd_, EPOLL_CTL_ADD, fd, &ev);
  return raw;
}

Endpoint* Worker::connect(const sockaddr* dst, socklen_t len, const sockaddr* src, socklen_t src_len, Completion done,
                          int* status) {
  int fd = ::socket(dst->sa_family, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) {
    *status = UCS_ERR_IO_ERROR;
    return nullptr;
  }
  if (src && src_len && ::bind(fd, src, src_len) != 0) {
    ::close(fd);
    *status = UCS_ERR_INVALID_ADDR;
    return nullptr;
  }
  set_nonblocking(fd);
  tune_socket(fd);
  int rc = ::connect(fd, dst, len);
  if (rc != 0 && errno != EINPROGRESS) {
    int e = errno;
    ::close(fd);
    *status = (e == ENETUNREACH || e == EHOSTUNREACH) ? UCS_ERR_UNREACHABLE : UCS_ERR_IO_ERROR;
    return nullptr;
  }
  Endpoint* ep = new_endpoint(fd);
  ep->peer_name_ = sockaddr_to_string(dst);
  ep->state_ = Endpoint::State::kConnecting;
  ep->on_connected_ = std::move(done);
  *status = UCS_INPROGRESS;
  return ep;
}

Endpoint* Worker::connect(const WorkerAddress& addr, Completion done, int* status) {
  sockaddr_in in{};
  in.sin_family = AF_INET;
  in.sin_addr.s_addr = addr.ipv4;
  in.sin_port = htons(addr.port);
  return connect(reinterpret_cast<sockaddr*>(&in), sizeof(in), nullptr, 0, std::move(done), status);
}

constexpr size_t kShmNameWire = 48;

void Worker::send_hello(Endpoint* ep, uint8_t type, uint8_t flags, const std::string& shm_name) {
  Endpoint::SendItem it;
  FrameHeader fh;
  fh.type = type;
  fh.flags = flags;
  const bool offer = (flags & kFlagShmOffer) && !shm_name.empty() && shm_name.size() < kShmNameWire;
  fh.header_len = 8 + kAddrWire + (offer ? kShmNameWire : 0);
  it.owned.assign(sizeof(fh) + fh.header_len, 0);
  std::memcpy(it.owned.data(), &fh, sizeof(fh));
  std::memcpy(it.owned.data() + sizeof(fh), &opt_.client_id, 8);
  put_addr(it.owned.data() + sizeof(fh) + 8, addr_);
  if (offer) std::memcpy(it.owned.data() + sizeof(fh) + 8 + kAddrWire, shm_name.data(), shm_name.size());
  it.switch_to_shm = type == kHelloAck && (flags & kFlagShmAccept);
  enqueue(ep, std::move(it));
}

void Worker::activate_shm(Endpoint* ep) {
  if (!ep->shm_ || ep->shm_active_) return;
  ep->shm_active_ = true;
  shm_eps_.push_back(ep);
  if (ep->shm_->creator()) connect_fd_channel(ep);  // before anything below is announced to the peer
  setup_device_channel(ep);
}

// Socket-like I/O on whichever channel the endpoint uses.
ssize_t Worker::io_read(Endpoint* ep, void* buf, size_t n) {
  return ep->shm_active_ ? ep->shm_->read(buf, n) : ::read(ep->fd_, buf, n);
}
ssize_t Worker::io_readv(Endpoint* ep, const iovec* iov, int cnt) {
  if (!ep->shm_active_) return ::readv(ep->fd_, iov, cnt);
  ssize_t total = 0;
  for (int i = 0; i < cnt; ++i) {
    ssize_t n = ep->shm_->read(iov[i].iov_base, iov[i].iov_len);
    if (n < 0 && errno == EIO && total == 0) return -1;  // a ring with impossible indices: the connection ends
    if (n < 0) break;
    total += n;
    if (static_cast<size_t>(n) < iov[i].iov_len) break;
  }
  if (total == 0) {
    errno = EAGAIN;
    return -1;
  }
  return total;
}
ssize_t Worker::io_writev(Endpoint* ep, const iovec* iov, int cnt) {
  if (!ep->shm_active_) {
    // sendmsg, not writev: a peer that has gone away must end as EPIPE here, not as a SIGPIPE for the whole
    // process (a library cannot count on the application ignoring that signal)
    msghdr mh{};
    mh.msg_iov = const_cast<iovec*>(iov);
    mh.msg_iovlen = static_cast<size_t>(cnt);
    return ::sendmsg(ep->fd_, &mh, MSG_NOSIGNAL);
  }
  ssize_t total = 0;
  for (int i = 0; i < cnt; ++i) {
    ssize_t n = ep->shm_->write(iov[i].iov_base, iov[i].iov_len);
    if (n < 0 && errno == EIO && total == 0) return -1;
    if (n < 0) break;
    total += n;
    if (static_cast<size_t>(n) < iov[i].iov_len) break;
  }
  if (total == 0) {
    errno = EAGAIN;
    return -1;
  }
  return total;
}

Endpoint* Worker::accept(ConnRequest&& req, int* status) {
  if (req.fd < 0) {
    *status = UCS_ERR_INVALID_PARAM;
    return nullptr;
  }
  Endpoint* ep = new_endpoint(req.fd);
  req.fd = -1;
  ep->peer_name_ = req.peer_name;
  ep->remote_.addr = req.remote;
  ep->remote_.name_str = req.worker_name;
  ep->remote_client_id_ = req.client_id;
  ep->state_ = Endpoint::State::kConnected;
  ep->rbuf_ = std::move(req.pending);
  if (opt_.use_shm && !req.shm_name.empty()) ep->shm_ = ShmChannel::open(req.shm_name);  // null on another host
  send_hello(ep, kHelloAck, ep->shm_ ? kFlagShmAccept : 0);
  *status = UCS_OK;
  if (!ep->rbuf_.empty()) reparse_.push_back(ep);  // frames that came in right behind the HELLO
  return ep;
}

void Worker::reject(ConnRequest&& req) {
  if (req.fd >= 0) ::close(req.fd);
  req.fd = -1;
}

void Worker::accept_pending(Listener& l) {
  for (;;) {
    sockaddr_storage ss{};
    socklen_t len = sizeof(ss);
    int fd = ::accept4(l.fd, reinterpret_cast<sockaddr*>(&ss), &len, SOCK_NONBLOCK | SOCK_CLOEXEC);
    if (fd < 0) return;
    tune_socket(fd);
    hellos_.push_back({fd, l.implicit, sockaddr_to_string(reinterpret_cast<sockaddr*>(&ss)), {}, std::chrono::steady_clock::now()});
  }
}

// Accepted sockets are read until their HELLO frame is complete.
void Worker::poll_hellos() {
  for (auto it = hellos_.begin(); it != hellos_.end();) {
    char tmp[512];
    bool dead = false;
    for (;;) {
      ssize_t n = ::read(it->fd, tmp, sizeof(tmp));
      if (n > 0) {
        it->buf.insert(it->buf.end(), tmp, tmp + n);
        if (it->buf.size() >= sizeof(FrameHeader)) {
          FrameHeader peek;
          std::memcpy(&peek, it->buf.data(), sizeof(peek));
          if (peek.magic != kFrameMagic || it->buf.size() >= sizeof(FrameHeader) + peek.header_len) break;
        }
        continue;
      }
      if (n == 0 || (errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR)) dead = true;
      break;
    }
    size_t need = sizeof(FrameHeader) + 8 + kAddrWire;
    if (it->buf.size() >= sizeof(FrameHeader)) {
      FrameHeader peek;
      std::memcpy(&peek, it->buf.data(), sizeof(peek));
      if (peek.magic == kFrameMagic && peek.header_len >= 8 + kAddrWire && peek.header_len <= 8 + kAddrWire + kShmNameWire)
        need = sizeof(FrameHeader) + peek.header_len;
    }
    if (!dead && it->buf.size() < need) {
      if (std::chrono::steady_clock::now() - it->since > std::chrono::seconds(5)) dead = true;
      else {
        ++it;
        continue;
      }
    }
    if (!dead) {
      FrameHeader fh;
      std::memcpy(&fh, it->buf.data(), sizeof(fh));
      ConnRequest req;
      if (fh.magic != kFrameMagic || fh.type != kHello ||
          !get_addr(it->buf.data() + sizeof(fh) + 8, it->buf.size() - sizeof(fh) - 8, &req.remote)) {
        dead = true;
      } else {
        std::memcpy(&req.client_id, it->buf.data() + sizeof(fh), 8);
        if ((fh.flags & kFlagShmOffer) && fh.header_len >= 8 + kAddrWire + kShmNameWire) {
          const char* nm = it->buf.data() + sizeof(fh) + 8 + kAddrWire;
          req.shm_name.assign(nm, strnlen(nm, kShmNameWire - 1));
        }
        req.fd = it->fd;
        req.peer_name = it->peer;
        req.worker_name = req.remote.name;
        req.arrival = std::chrono::steady_clock::now();
        req.pending.assign(it->buf.begin() + need, it->buf.end());
        if (it->implicit) {
          int st;
          Endpoint* ep = accept(std::move(req), &st);
          if (ep) {
            ep->auto_accepted_ = true;
            if (on_auto_accept) on_auto_accept(ep);
          }
        } else if (on_conn_request) {
          on_conn_request(std::move(req));
        } else {
          ::close(req.fd);
        }
      }
    }
    if (dead) ::close(it->fd);
    it = hellos_.erase(it);
  }
}

// ---------------------------------------------------------------------------
// progress loop, socket I/O
// ---------------------------------------------------------------------------
int Worker::progress() {
  int handled = 0;
  if (!pull_batch_.empty()) flush_pull_batch();  // pulls posted by the context since the last pass
  if (!reparse_.empty()) {
    auto list = std::move(reparse_);
    reparse_.clear();
    for (Endpoint* ep : list)
      if (eps_.count(ep) && ep->state_ == Endpoint::State::kConnected) parse_frames(ep);
  }
  // The sockets are looked at on every call while any endpoint still talks through one. Once all of them
  // use the rings, a socket only reports a new connection or a peer that went away, and the system
  // call is made every few microseconds instead.
  epoll_event evs[64];
  int n = 0;
  const auto now = std::chrono::steady_clock::now();
  last_progress_ = now;
  if (eps_.size() > shm_eps_.size() || now - last_epoll_ >= std::chrono::microseconds(5)) {
    last_epoll_ = now;
    n = epoll_wait(epfd_, evs, 64, 0);
  }
  for (int i = 0; i < n; ++i) {
    ++handled;
    if (evs[i].data.u64 >> 63) {
      size_t idx = static_cast<size_t>(evs[i].data.u64 & 0xffffffffu);
      if (idx == kFdListenerTag) {
        accept_fd_channels();
        continue;
      }
      if (idx < listeners_.size() && listeners_[idx].fd >= 0) accept_pending(listeners_[idx]);
      continue;
    }
    Endpoint* ep = static_cast<Endpoint*>(evs[i].data.ptr);
    if (!eps_.count(ep)) continue;
    if (ep->state_ == Endpoint::State::kClosed || ep->state_ == Endpoint::State::kFailed) continue;
    if (evs[i].events & (EPOLLERR | EPOLLHUP)) {
      int err = 0;
      socklen_t len = sizeof(err);
      getsockopt(ep->fd_, SOL_SOCKET, SO_ERROR, &err, &len);
      if (ep->state_ == Endpoint::State::kConnecting) {
        fail(ep, (err == ENETUNREACH || err == EHOSTUNREACH || err == ETIMEDOUT) ? UCS_ERR_UNREACHABLE : UCS_ERR_NOT_CONNECTED);
        continue;
      }
      if (!(evs[i].events & EPOLLIN)) {
        fail(ep, UCS_ERR_CONNECTION_RESET);
        continue;
      }
    }
    if (evs[i].events & EPOLLOUT) handle_writable(ep);
    if (ep->state_ == Endpoint::State::kFailed || ep->state_ == Endpoint::State::kClosed) continue;
    if (evs[i].events & (EPOLLIN | EPOLLRDHUP)) {
      handle_readable(ep);
      if (ep->shm_active_ && eps_.count(ep) && ep->state_ == Endpoint::State::kConnected && ep->fd_ >= 0) {
        // the frames travel through the rings; the socket only tells us when the peer is gone
        char probe;
        ssize_t r = ::recv(ep->fd_, &probe, 1, MSG_PEEK | MSG_DONTWAIT);
        if (r == 0 || (r < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR)) fail(ep, UCS_ERR_CONNECTION_RESET);
      }
    }
  }
  // rings are polled: nothing wakes epoll when a peer writes into shared memory
  for (size_t i = 0; i < shm_eps_.size();) {
    Endpoint* ep = shm_eps_[i];
    if (!eps_.count(ep) || !ep->shm_active_ || ep->state_ == Endpoint::State::kFailed || ep->state_ == Endpoint::State::kClosed) {
      shm_eps_[i] = shm_eps_.back();
      shm_eps_.pop_back();
      continue;
    }
    if (ep->shm_->readable()) {
      ++handled;
      handle_readable(ep);
    }
    if (eps_.count(ep) && ep->state_ == Endpoint::State::kConnected && !ep->sendq_.empty()) flush(ep);
    ++i;
  }
  if (!hellos_.empty()) poll_hellos();
  if (!awaiting_ring_.empty()) {
    for (size_t i = 0; i < awaiting_ring_.size();) {
      Endpoint* ep = awaiting_ring_[i];
      const bool alive = eps_.count(ep) && ep->state_ == Endpoint::State::kConnected && ep->await_dev_ring_;
      if (alive && now <= ep->dev_ring_deadline_) {
        ++i;
        continue;
      }
      awaiting_ring_[i] = awaiting_ring_.back();
      awaiting_ring_.pop_back();
      if (alive) finish_connect(ep);  // the peer stayed silent: go on without its ring
    }
  }
  if (!pull_batch_.empty()) flush_pull_batch();
  if (!held_sends_.empty()) poll_held_sends();
  drain_slot_releases();
  if (!device_ops_.empty() || !eager_waits_.empty() || !push_waits_.empty()) poll_device();
  if (!graveyard_.empty()) {
    for (Endpoint* ep : graveyard_) eps_.erase(ep);
    graveyard_.clear();
  }
  return handled;
}

void Worker::fail(Endpoint* ep, int status) {
  if (ep->state_ == Endpoint::State::kFailed || ep->state_ == Endpoint::State::kClosed) return;
  const bool was_connecting = ep->state_ == Endpoint::State::kConnecting || ep->state_ == Endpoint::State::kHelloSent || ep->await_dev_ring_;
  ep->await_dev_ring_ = false;
  ep->state_ = Endpoint::State::kFailed;
  if (ep->fd_ >= 0) {
    epoll_ctl(epfd_, EPOLL_CTL_DEL, ep->fd_, nullptr);
    ::close(ep->fd_);
    ep->fd_ = -1;
  }
  teardown_device_channel(ep);
  close_fd_channel(ep);
  std::erase_if(held_sends_, [ep](const HeldSend& h) { return h.ep == ep; });
  ep->shm_active_ = false;
  ep->shm_.reset();
  // every operation in flight ends with the endpoint's status
  std::vector<Completion> cbs;
  for (auto& it : ep->sendq_)
    if (it.done) cbs.push_back(std::move(it.done));
  ep->sendq_.clear();
  for (auto& [id, ps] : ep->pending_sends_)
    if (ps.done) cbs.push_back(std::move(ps.done));
  ep->pending_sends_.clear();
  for (auto& [id, pr] : ep->pending_recvs_)
    if (pr.done) cbs.push_back(std::move(pr.done));
  ep->pending_recvs_.clear();
  ep->rts_.clear();
  for (auto& d : device_ops_)
    if (d.ep == ep) d.ep = nullptr;  // the kernel still finishes; nobody is told
  Completion connected = std::move(ep->on_connected_);
  ep->on_connected_ = nullptr;
  for (auto& cb : cbs) cb(status);
  if (was_connecting && connected) connected(status);
  else if (on_ep_error) on_ep_error(ep, status);
}

void Worker::close(Endpoint* ep, bool notify_peer) {
  if (!eps_.count(ep)) return;
  if (ep->state_ == Endpoint::State::kConnected && notify_peer && ep->fd_ >= 0) {
    FrameHeader fh;
    fh.type = kClose;
    // best effort, blocking for at most the socket buffer: the frame is 40 bytes
    if (ep->shm_active_) (void)ep->shm_->write(&fh, sizeof(fh));
    else (void)!::send(ep->fd_, &fh, sizeof(fh), MSG_NOSIGNAL);
  }
  if (ep->fd_ >= 0) {
    epoll_ctl(epfd_, EPOLL_CTL_DEL, ep->fd_, nullptr);
    ::shutdown(ep->fd_, SHUT_RDWR);
    ::close(ep->fd_);
    ep->fd_ = -1;
  }
  teardown_device_channel(ep);
  close_fd_channel(ep);
  std::erase_if(held_sends_, [ep](const HeldSend& h) { return h.ep == ep; });
  ep->shm_active_ = false;
  ep->shm_.reset();
  if (ep->state_ != Endpoint::State::kFailed) {
    ep->state_ = Endpoint::State::kClosed;
    std::vector<Completion> cbs;
    for (auto& it : ep->sendq_)
      if (it.done) cbs.push_back(std::move(it.done));
    ep->sendq_.clear();
    for (auto& [id, ps] : ep->pending_sends_)
      if (ps.done) cbs.push_back(std::move(ps.done));
    for (auto& [id, pr] : ep->pending_recvs_)
      if (pr.done) cbs.push_back(std::move(pr.done));
    ep->pending_sends_.clear();
    ep->pending_recvs_.clear();
    for (auto& d : device_ops_)
      if (d.ep == ep) d.ep = nullptr;
    for (auto& cb : cbs) cb(UCS_ERR_CANCELED);
  }
}

void Worker::destroy(Endpoint* ep) {
  if (!eps_.count(ep)) return;
  close(ep, false);
  for (auto& d : device_ops_)
    if (d.ep == ep) d.ep = nullptr;
  graveyard_.push_back(ep);
}

namespace {
std::mutex g_fault_mu;
std::shared_ptr<FaultHook> g_fault_hook;  // null when no test has installed one
std::atomic<bool> g_fault_on{false};
}  // namespace

bool is_live_local_uid(uint64_t uid) { return live_has(uid); }

namespace {
std::atomic<ConsumerEventHook> g_consumer_event_hook{nullptr};
struct SlotRelease {  // slots waiting for the consumer's queued GPU work before they go back to the sender
  void* event;
  int device;
  std::shared_ptr<ShmChannel> shm;
  uint64_t mask;
};
std::mutex g_slot_release_mu;
std::vector<SlotRelease> g_slot_releases;
std::atomic<size_t> g_slot_release_count{0};

void* record_consumer_event(int device) {
  void* ev = nullptr;
  if (auto hook = g_consumer_event_hook.load(std::memory_order_acquire))
    if (hook(device, &ev) == kConsumerEvent) return ev;
  return nullptr;
}
}  // namespace

void set_consumer_event_hook(ConsumerEventHook hook) { g_consumer_event_hook.store(hook, std::memory_order_release); }

// Any worker of the process hands back the slots whose consumers have finished (the entry owns what it touches).
void Worker::drain_slot_releases() {
  if (g_slot_release_count.load(std::memory_order_acquire) == 0) return;
  std::unique_lock lk(g_slot_release_mu, std::try_to_lock);
  if (!lk.owns_lock()) return;
  for (size_t i = 0; i < g_slot_releases.size();) {
    auto& r = g_slot_releases[i];
    if (cudaEventQuery(static_cast<cudaEvent_t>(r.event)) == cudaErrorNotReady) {
      ++i;
      continue;
    }
    cudaGetLastError();
    cudaEventDestroy(static_cast<cudaEvent_t>(r.event));
    r.shm->out_words()[0].fetch_or(r.mask, std::memory_order_release);
    if (i + 1 != g_slot_releases.size()) g_slot_releases[i] = std::move(g_slot_releases.back());
    g_slot_releases.pop_back();
  }
  g_slot_release_count.store(g_slot_releases.size(), std::memory_order_release);
}

void set_fault_hook(FaultHook hook) {
  std::lock_guard lk(g_fault_mu);
  g_fault_hook = hook ? std::make_shared<FaultHook>(std::move(hook)) : nullptr;
  g_fault_on.store(g_fault_hook != nullptr, std::memory_order_release);
}

void Worker::enqueue(Endpoint* ep, Endpoint::SendItem&& item) {
  if (g_fault_on.load(std::memory_order_acquire) && item.owned.size() >= sizeof(FrameHeader)) {
    std::shared_ptr<FaultHook> hook;
    {
      std::lock_guard lk(g_fault_mu);
      hook = g_fault_hook;
    }
    FrameHeader fh;
    std::memcpy(&fh, item.owned.data(), sizeof(fh));
    if (hook && (*hook)(opt_.name, fh.type, fh.msg_id)) {
      if (item.done) item.done(UCS_OK);  // lost on the wire: the sender cannot tell
      return;
    }
  }
  ep->sendq_.push_back(std::move(item));
  if (ep->state_ == Endpoint::State::kConnected || ep->state_ == Endpoint::State::kHelloSent) flush(ep);
}

void Worker::send_control(Endpoint* ep, uint8_t type, uint8_t flags, uint64_t msg_id, int32_t status) {
  Endpoint::SendItem it;
  FrameHeader fh;
  fh.type = type;
  fh.flags = flags;
  fh.msg_id = msg_id;
  fh.status = status;
  it.owned.resize(sizeof(fh));
  std::memcpy(it.owned.data(), &fh, sizeof(fh));
  enqueue(ep, std::move(it));
}

// Write as much of the send queue as the socket takes.
void Worker::flush(Endpoint* ep) {
  while (!ep->sendq_.empty() && ep->fd_ >= 0) {
    auto& it = ep->sendq_.front();
    iovec iov[16];
    int cnt = 0;
    if (it.owned_off < it.owned.size()) {
      iov[cnt].iov_base = it.owned.data() + it.owned_off;
      iov[cnt].iov_len = it.owned.size() - it.owned_off;
      ++cnt;
    }
    for (size_t s = it.seg_idx; s < it.segs.size() && cnt < 16; ++s) {
      size_t off = (s == it.seg_idx) ? it.seg_off : 0;
      if (it.segs[s].size == off) continue;
      iov[cnt].iov_base = static_cast<char*>(it.segs[s].data) + off;
      iov[cnt].iov_len = it.segs[s].size - off;
      ++cnt;
    }
    if (cnt == 0) {
      Completion done = std::move(it.done);
      ep->sendq_.pop_front();
      if (done) done(UCS_OK);
      continue;
    }
    ssize_t n = io_writev(ep, iov, cnt);
    if (n < 0) {
      if (errno == EAGAIN || errno == EWOULDBLOCK) return;  // EPOLLOUT (edge) or the ring poll will call us again
      if (errno == EINTR) continue;
      fail(ep, UCS_ERR_CONNECTION_RESET);
      return;
    }
    size_t left = static_cast<size_t>(n);
    size_t take = std::min(left, it.owned.size() - it.owned_off);
    it.owned_off += take;
    left -= take;
    while (left > 0 && it.seg_idx < it.segs.size()) {
      size_t avail = it.segs[it.seg_idx].size - it.seg_off;
      size_t t = std::min(avail, left);
      it.seg_off += t;
      left -= t;
      if (it.seg_off == it.segs[it.seg_idx].size) {
        ++it.seg_idx;
        it.seg_off = 0;
      }
    }
    while (it.seg_idx < it.segs.size() && it.segs[it.seg_idx].size == 0) ++it.seg_idx;
    if (it.owned_off == it.owned.size() && it.seg_idx >= it.segs.size()) {
      Completion done = std::move(it.done);
      const bool to_shm = it.switch_to_shm;
      ep->sendq_.pop_front();
      if (to_shm) activate_shm(ep);  // the accepting reply is on the wire: everything after it uses the rings
      if (done) done(UCS_OK);
    }
  }
}

void Worker::handle_writable(Endpoint* ep) {
  if (ep->state_ == Endpoint::State::kConnecting) {
    int err = 0;
    socklen_t len = sizeof(err);
    getsockopt(ep->fd_, SOL_SOCKET, SO_ERROR, &err, &len);
    if (err != 0) {
      fail(ep, (err == ENETUNREACH || err == EHOSTUNREACH || err == ETIMEDOUT) ? UCS_ERR_UNREACHABLE : UCS_ERR_NOT_CONNECTED);
      return;
    }
    ep->state_ = Endpoint::State::kHelloSent;
    if (opt_.use_shm) {
      static std::atomic<uint64_t> counter{0};
      std::random_device rd;
      char name[kShmNameWire];
      std::snprintf(name, sizeof(name), "/eux-%d-%llx-%08x", (int)getpid(),
                    (unsigned long long)counter.fetch_add(1), (unsigned)rd());
      ep->shm_ = ShmChannel::create(name);
    }
    send_hello(ep, kHello, ep->shm_ ? kFlagShmOffer : 0, ep->shm_ ? ep->shm_->name() : std::string());
    return;
  }
  flush(ep);
}

void Worker::handle_readable(Endpoint* ep) {
  for (;;) {
    if (ep->fd_ < 0) return;
    if (ep->direct_active_) {
      // payload of a DATA frame goes straight into the posted receive buffers
      auto pit = ep->pending_recvs_.find(ep->direct_msg_);
      if (pit == ep->pending_recvs_.end()) {  // cancelled meanwhile: drain into a scratch buffer
        char sink[65536];
        ssize_t n = io_read(ep, sink, std::min(sizeof(sink), ep->direct_left_));
        if (n > 0) {
          ep->direct_left_ -= static_cast<size_t>(n);
          if (ep->direct_left_ == 0) ep->direct_active_ = false;
          continue;
        }
        if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) return;
        if (n < 0 && errno == EINTR) continue;
        fail(ep, UCS_ERR_CONNECTION_RESET);
        return;
      }
      auto& pr = pit->second;
      while (ep->direct_seg_ < pr.segs.size() && pr.segs[ep->direct_seg_].size == ep->direct_off_) {
        ++ep->direct_seg_;
        ep->direct_off_ = 0;
      }
      iovec iov[16];
      int cnt = 0;
      size_t budget = ep->direct_left_;
      for (size_t s = ep->direct_seg_; s < pr.segs.size() && cnt < 16 && budget > 0; ++s) {
        size_t off = (s == ep->direct_seg_) ? ep->direct_off_ : 0;
        size_t len = std::min(pr.segs[s].size - off, budget);
        if (!len) continue;
        iov[cnt].iov_base = static_cast<char*>(pr.segs[s].data) + off;
        iov[cnt].iov_len = len;
        budget -= len;
        ++cnt;
      }
      if (cnt == 0) {  // the posted buffers are smaller than the payload: fail it, drain the rest
        Completion done = std::move(pr.done);
        ep->pending_recvs_.erase(pit);
        if (done) done(UCS_ERR_MESSAGE_TRUNCATED);
        continue;
      }
      ssize_t n = io_readv(ep, iov, cnt);
      if (n <= 0) {
        if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) return;
        if (n < 0 && errno == EINTR) continue;
        fail(ep, UCS_ERR_CONNECTION_RESET);
        return;
      }
      size_t left = static_cast<size_t>(n);
      ep->direct_left_ -= left;
      while (left > 0) {
        size_t avail = pr.segs[ep->direct_seg_].size - ep->direct_off_;
        size_t t = std::min(avail, left);
        ep->direct_off_ += t;
        left -= t;
        if (ep->direct_off_ == pr.segs[ep->direct_seg_].size) {
          ++ep->direct_seg_;
          ep->direct_off_ = 0;
        }
      }
      if (ep->direct_left_ == 0) {
        ep->direct_active_ = false;
        Endpoint::PendingRecv fin = std::move(pr);
        ep->pending_recvs_.erase(pit);
        int st = ep->direct_total_ == fin.total ? UCS_OK : UCS_ERR_MESSAGE_TRUNCATED;
        if (st != UCS_OK) ++stats_.truncated;
        if (fin.bounce && st == UCS_OK) {  // staged through host memory: scatter into the device destinations
          try {
            const char* src = static_cast<const char*>(fin.bounce.get());
            for (auto& d : fin.dev_dsts) {
              mr_.memcpy(fin.mem_type, d.data, ucx_memory_type::HOST, src, d.size);
              src += d.size;
            }
          } catch (...) {
            st = UCS_ERR_IO_ERROR;
          }
        }
        if (fin.done) fin.done(st);
      }
      continue;
    }
    // frame headers and small bodies are buffered
    if (ep->rpos_ > 0 && ep->rpos_ == ep->rbuf_.size()) {
      ep->rbuf_.clear();
      ep->rpos_ = 0;
    }
    char tmp[65536];
    ssize_t n = io_read(ep, tmp, sizeof(tmp));
    if (n > 0) {
      ep->rbuf_.insert(ep->rbuf_.end(), tmp, tmp + n);
      if (!parse_frames(ep)) return;
      continue;
    }
    if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) return;
    if (n < 0 && errno == EINTR) continue;
    fail(ep, n == 0 ? UCS_ERR_CONNECTION_RESET : UCS_ERR_IO_ERROR);
    return;
  }
}

// ---------------------------------------------------------------------------
// frame parsing
// ---------------------------------------------------------------------------
// Consumes complete frames from ep->rbuf_. Returns false when the endpoint died.
bool Worker::parse_frames(Endpoint* ep) {
  for (;;) {
    if (ep->state_ == Endpoint::State::kFailed || ep->state_ == Endpoint::State::kClosed) return false;
    if (ep->direct_active_) return true;  // the rest of the stream belongs to a posted receive
    const size_t avail = ep->rbuf_.size() - ep->rpos_;
    if (avail < sizeof(FrameHeader)) break;
    FrameHeader fh;
    std::memcpy(&fh, ep->rbuf_.data() + ep->rpos_, sizeof(fh));
    if (fh.magic != kFrameMagic) {
      fail(ep, UCS_ERR_IO_ERROR);
      return false;
    }
    const size_t inline_cap = std::max(opt_.eager_limit, kMinInlineCap);
    if (fh.header_len > kMaxHeaderLen || fh.seg_count > kMaxSegCount || (fh.type == kAmEager && fh.payload_len > inline_cap)) {
      UCX_CONN_ERROR << "frame from " << ep->peer_name_ << " refused: header " << fh.header_len << " B, " << fh.seg_count
                     << " segments, inline payload " << (fh.type == kAmEager ? fh.payload_len : 0) << " B";
      ++stats_.frames_refused;
      fail(ep, UCS_ERR_IO_ERROR);
      return false;
    }
    size_t meta = fh.header_len;
    if (fh.type == kAmRts) {
      const size_t nreg = rts_region_count(fh);
      if (nreg > kMaxSegCount) {
        UCX_CONN_ERROR << "frame from " << ep->peer_name_ << " refused: " << nreg << " device regions";
        ++stats_.frames_refused;
        fail(ep, UCS_ERR_IO_ERROR);
        return false;
      }
      meta += size_t(fh.seg_count) * 8 + nreg * sizeof(PeerRegionDesc) + ((fh.flags & kFlagLayout) ? sizeof(WireLayout) : 0);
    }
    if (fh.type == kAmDevEager) meta += 8;  // the flag value that the payload's arrival will carry
    size_t body = meta + (fh.type == kAmEager ? fh.payload_len : 0);
    if (avail < sizeof(fh) + body) break;  // wait for the rest (eager bodies are small)
    const char* b = ep->rbuf_.data() + ep->rpos_ + sizeof(fh);
    ep->rpos_ += sizeof(fh) + body;
    dispatch_frame(ep, fh, b);
  }
  if (ep->rpos_ > 0 && !ep->direct_active_) {
    ep->rbuf_.erase(ep->rbuf_.begin(), ep->rbuf_.begin() + ep->rpos_);
    ep->rpos_ = 0;
  }
  return ep->state_ != Endpoint::State::kFailed && ep->state_ != Endpoint::State::kClosed;
}

void Worker::dispatch_frame(Endpoint* ep, const FrameHeader& fh, const char* body) {
  switch (fh.type) {
    case kHelloAck: {
      if (fh.header_len >= 8 + kAddrWire) {
        std::memcpy(&ep->remote_client_id_, body, 8);
        get_addr(body + 8, fh.header_len - 8, &ep->remote_.addr);
        ep->remote_.name_str = ep->remote_.addr.name;
      }
      if (ep->shm_) {
        if (fh.flags & kFlagShmAccept) activate_shm(ep);  // the peer mapped it: both directions switch here
        else ep->shm_.reset();                            // another host, or the peer does not want it
      }
      if (ep->state_ == Endpoint::State::kHelloSent) {
        ep->state_ = Endpoint::State::kConnected;
        // Two GPU workers on one host: the caller learns "connected" once the peer has said where its
        // device receive ring is (it follows the HELLO_ACK through the rings), or after a short wait.
        if (ep->shm_active_ && opt_.device >= 0 && cuda_mr_ && ep->remote_.addr.device >= 0 && ep->on_connected_) {
          ep->await_dev_ring_ = true;
          ep->dev_ring_deadline_ = std::chrono::steady_clock::now() + std::chrono::seconds(3);
          awaiting_ring_.push_back(ep);
        } else {
          finish_connect(ep);
        }
        if (eps_.count(ep) && ep->state_ == Endpoint::State::kConnected) flush(ep);
      }
      break;
    }
    case kAmEager: {
      AmArrival a;
      a.ep = ep;
      a.header_len = fh.header_len;
      a.header = fh.header_len ? mr_.allocate(ucx_memory_type::HOST, fh.header_len) : nullptr;
      if (fh.header_len) std::memcpy(a.header, body, fh.header_len);
      a.data_len = fh.payload_len;
      a.data = fh.payload_len ? mr_.allocate(ucx_memory_type::HOST, fh.payload_len) : nullptr;
      if (fh.payload_len) std::memcpy(a.data, body + fh.header_len, fh.payload_len);
      a.sender_mem_type = static_cast<ucx_memory_type_t>(fh.mem_type);
      a.msg_id = fh.msg_id;
      if (on_am) on_am(std::move(a));
      else {
        if (a.header) mr_.deallocate(ucx_memory_type::HOST, a.header, a.header_len);
        if (a.data) mr_.deallocate(ucx_memory_type::HOST, a.data, a.data_len);
      }
      break;
    }
    case kAmRts: {
      nvtx_mark("eux.transport.rts_received");
      Endpoint::RtsInfo info;
      info.payload_len = fh.payload_len;
      info.mem_type = static_cast<ucx_memory_type_t>(fh.mem_type);
      info.push_ok = (fh.flags & kFlagPushOk) != 0;
      const char* p = body + fh.header_len;
      info.seg_sizes.resize(fh.seg_count);
      if (fh.seg_count) std::memcpy(info.seg_sizes.data(), p, size_t(fh.seg_count) * 8);
      p += size_t(fh.seg_count) * 8;
      uint64_t seg_sum = 0;
      for (uint64_t sz : info.seg_sizes) seg_sum += sz;
      if (fh.seg_count && seg_sum != fh.payload_len) {
        UCX_CONN_ERROR << "RTS from " << ep->peer_name_ << " refused: segment sizes add up to " << seg_sum << ", payload is " << fh.payload_len;
        ++stats_.frames_refused;
        fail(ep, UCS_ERR_IO_ERROR);
        break;
      }
      if ((fh.flags & kFlagDeviceRegions) && !peer_is_local(ep)) ++stats_.regions_ignored;
      if ((fh.flags & kFlagDeviceRegions) && peer_is_local(ep)) {
        // Device regions are addresses and handles of the sender's process: they mean something only
        // when the handshake showed that the sender runs on this host. From anyone else they are
        // ignored and the payload takes the staged host protocol.
        info.regions.resize(rts_region_count(fh));
        std::memcpy(info.regions.data(), p, info.regions.size() * sizeof(PeerRegionDesc));
        uint64_t reg_sum = 0;
        for (auto& r : info.regions) reg_sum += r.length;
        if (fh.flags & kFlagLayout) {
          // a strided view inside the one region: what the layout says must lie inside it and add up to the payload
          std::memcpy(&info.layout, p + info.regions.size() * sizeof(PeerRegionDesc), sizeof(WireLayout));
          SendHint chk;
          chk.ndim = info.layout.ndim;
          chk.elem_size = info.layout.elem_size;
          chk.src_dtype = info.layout.src_dtype;
          chk.dst_dtype = info.layout.dst_dtype;
          std::memcpy(chk.shape, info.layout.shape, sizeof(chk.shape));
          std::memcpy(chk.stride, info.layout.stride, sizeof(chk.stride));
          chk.span_bytes = info.layout.span_bytes;
          chk.dense_bytes = fh.payload_len;
          info.has_layout = info.regions.size() == 1 && info.layout.ndim > 0 && chk.layout_valid() && reg_sum == info.layout.span_bytes;
          if (!info.has_layout) info.regions.clear();  // the sender packs it and it takes the staged way
        } else if (reg_sum != fh.payload_len) {
          info.regions.clear();
        }
      }
      ep->rts_[fh.msg_id] = std::move(info);
      AmArrival a;
      a.ep = ep;
      a.header_len = fh.header_len;
      a.header = fh.header_len ? mr_.allocate(ucx_memory_type::HOST, fh.header_len) : nullptr;
      if (fh.header_len) std::memcpy(a.header, body, fh.header_len);
      a.data_len = fh.payload_len;
      a.rndv = true;
      a.msg_id = fh.msg_id;
      a.seg_count = fh.seg_count > 1 ? fh.seg_count : 0;
      a.sender_mem_type = static_cast<ucx_memory_type_t>(fh.mem_type);
      if (on_am) on_am(std::move(a));
      else if (a.header) mr_.deallocate(ucx_memory_type::HOST, a.header, a.header_len);
      break;
    }
    case kRndvCts:
      if (fh.flags & kFlagPush) on_push_cts(ep, fh, body);
      else start_data_send(ep, fh.msg_id, (fh.flags & kFlagStage) != 0);
      break;
    case kDevRing: on_dev_ring(ep, fh, body); break;
    case kAmDevEager: on_dev_eager(ep, fh, body); break;
    case kRndvData: {
      auto pit = ep->pending_recvs_.find(fh.msg_id);
      ep->direct_active_ = true;
      ep->direct_msg_ = fh.msg_id;
      ep->direct_seg_ = 0;
      ep->direct_off_ = 0;
      ep->direct_left_ = fh.payload_len;
      ep->direct_total_ = fh.payload_len;
      // bytes of the payload that are already in the buffer
      size_t have = std::min<size_t>(ep->rbuf_.size() - ep->rpos_, ep->direct_left_);
      if (pit != ep->pending_recvs_.end()) {
        auto& pr = pit->second;
        const char* src = ep->rbuf_.data() + ep->rpos_;
        size_t left = have;
        while (left > 0 && ep->direct_seg_ < pr.segs.size()) {
          size_t room = pr.segs[ep->direct_seg_].size - ep->direct_off_;
          size_t t = std::min(room, left);
          std::memcpy(static_cast<char*>(pr.segs[ep->direct_seg_].data) + ep->direct_off_, src, t);
          src += t;
          left -= t;
          ep->direct_off_ += t;
          if (ep->direct_off_ == pr.segs[ep->direct_seg_].size) {
            ++ep->direct_seg_;
            ep->direct_off_ = 0;
          }
        }
      }
      ep->rpos_ += have;
      ep->direct_left_ -= have;
      if (ep->direct_left_ == 0) {
        ep->direct_active_ = false;
        if (pit != ep->pending_recvs_.end()) {
          Endpoint::PendingRecv fin = std::move(pit->second);
          ep->pending_recvs_.erase(pit);
          int st = fh.payload_len == fin.total ? UCS_OK : UCS_ERR_MESSAGE_TRUNCATED;
          if (st != UCS_OK) ++stats_.truncated;
          if (fin.bounce && st == UCS_OK) {
            try {
              const char* src = static_cast<const char*>(fin.bounce.get());
              for (auto& d : fin.dev_dsts) {
                mr_.memcpy(fin.mem_type, d.data, ucx_memory_type::HOST, src, d.size);
                src += d.size;
              }
            } catch (...) {
              st = UCS_ERR_IO_ERROR;
            }
          }
          if (fin.done) fin.done(st);
        }
      } else {
        // the buffered bytes are used up; continue reading straight from the socket
        ep->rbuf_.clear();
        ep->rpos_ = 0;
      }
      break;
    }
    case kRndvFin: {
      // receiver -> sender: the payload was pulled (or refused); sender -> receiver: the send was withdrawn
      // Both sides number their messages from 1: a FIN that comes from the *sender* of a message (it
      // withdrew the send, or cannot push it) must not be mistaken for the answer to this side's own
      // message of the same number.
      auto it = (fh.flags & kFlagFromSender) ? ep->pending_sends_.end() : ep->pending_sends_.find(fh.msg_id);
      if (it != ep->pending_sends_.end()) {
        Completion c = std::move(it->second.done);
        ep->pending_sends_.erase(it);
        if (c) c(fh.status);
        break;
      }
      ep->rts_.erase(fh.msg_id);
      for (auto pw = push_waits_.begin(); pw != push_waits_.end(); ++pw) {
        if (pw->ep != ep || pw->msg_id != fh.msg_id) continue;
        // the sender could not push after all (or withdrew the send): take the other roads
        PushWait w = std::move(*pw);
        push_waits_.erase(pw);
        if (ep->push_inflight_) --ep->push_inflight_;
        if (fh.status == UCS_ERR_UNSUPPORTED) {
          w.info.push_ok = false;
          ep->rts_[w.msg_id] = std::move(w.info);
          int st = rndv_recv(ep, w.msg_id, w.segs.data(), w.segs.size(), ucx_memory_type::CUDA, w.done, w.ready);
          if (st != UCS_INPROGRESS && w.done) w.done(st);
        } else if (w.done) {
          w.done(fh.status);
        }
        return;
      }
      auto pr = ep->pending_recvs_.find(fh.msg_id);
      if (pr != ep->pending_recvs_.end() && fh.status != UCS_OK) {
        Completion c = std::move(pr->second.done);
        ep->pending_recvs_.erase(pr);
        if (c) c(fh.status);
      }
      break;
    }
    case kClose: fail(ep, UCS_ERR_CONNECTION_RESET); break;
    default: break;
  }
}

// ---------------------------------------------------------------------------
// active message send / rendezvous
// ---------------------------------------------------------------------------
int Worker::am_send(Endpoint* ep, const void* header, size_t header_len, const ucx_buffer_t* segs, size_t seg_count,
                    ucx_memory_type_t mem_type, bool force_rndv, Completion done, uint64_t* msg_id_out,
                    std::shared_ptr<const SendHint> hint) {
  if (!eps_.count(ep) || ep->state_ != Endpoint::State::kConnected) return UCS_ERR_NOT_CONNECTED;
  // What the receiving side would refuse (and close the connection over) is not sent in the first place: the
  // caller gets the error at once and the connection stays.
  if (header_len > kMaxHeaderLen || seg_count > kMaxSegCount) return UCS_ERR_EXCEEDS_LIMIT;
  size_t total = 0;
  for (size_t i = 0; i < seg_count; ++i) total += segs[i].size;
  const bool device = is_device_type(mem_type);
  if (device) nvtx_mark("eux.transport.am_send_device");
  if (!device || total == 0) hint.reset();  // remarks are about device payloads
  bool strided = hint && hint->ndim > 0;
  if (strided && (seg_count != 1 || hint->dense_bytes != total || !hint->layout_valid())) return UCS_ERR_INVALID_PARAM;
  const bool rndv = total > 0 && (force_rndv || device || seg_count > 1 || total >= opt_.eager_limit);
  const uint64_t id = ep->next_msg_id_++;
  if (msg_id_out) *msg_id_out = id;
  // A payload whose producer is still running does not go out eagerly: the eager kernel would have to wait for
  // the producer on this worker's stream, and every other transfer of the worker behind it. It is announced
  // instead, once the producer is done (below), and nothing else waits.
  const bool producer_running = hint && hint->ready_event && cudaEventQuery(static_cast<cudaEvent_t>(hint->ready_event)) == cudaErrorNotReady;
  if (!producer_running) cudaGetLastError();
  if (device && !force_rndv && !producer_running && seg_count == 1 && total > 0 && total <= opt_.dev_eager_limit && ep->tx_ring_ && ep->out_flags_dev_) {
    int st = dev_eager_send(ep, header, header_len, segs[0], mem_type, id, done, hint);
    if (st != UCS_ERR_NO_RESOURCE) return st;  // no free slot right now: the rendezvous takes it
  }
  // A strided view travels as it lies when the peer can gather it out of this process's memory: one
  // exportable allocation under its span, peer on this host. Otherwise it is packed here first, by the
  // same kernel, and the dense copy travels.
  ucx_buffer_t packed_seg{};
  std::shared_ptr<void> packed;
  std::vector<PeerRegionDesc> regions;
  if (strided) {
    bool fused = false;
    if (cuda_mr_ && peer_is_local(ep)) {
      ucx_buffer_t span{segs[0].data, hint->span_bytes};
      fused = export_for_peer(ep, &span, 1, hint->span_bytes, &regions) && regions.size() == 1 && (regions[0].exportable || peer_is_this_process(ep));
      if (!fused) regions.clear();
    }
    if (!fused) {
      if (hint->ready_event && ensure_device()) cudaStreamWaitEvent(static_cast<cudaStream_t>(stream_), static_cast<cudaEvent_t>(hint->ready_event), 0);
      packed = pack_local(*hint, segs[0].data);
      if (!packed) return UCS_ERR_NO_MEMORY;
      packed_seg = {packed.get(), total};
      segs = &packed_seg;
      hint.reset();  // dense and complete from here on
      strided = false;
    }
  }
  FrameHeader fh;
  fh.header_len = static_cast<uint32_t>(header_len);
  fh.payload_len = total;
  fh.msg_id = id;
  fh.mem_type = static_cast<uint32_t>(mem_type);
  Endpoint::SendItem it;
  if (!rndv) {
    fh.type = kAmEager;
    const bool copy = total <= opt_.send_copy_limit;
    it.owned.resize(sizeof(fh) + header_len + (copy ? total : 0));
    std::memcpy(it.owned.data(), &fh, sizeof(fh));
    if (header_len) std::memcpy(it.owned.data() + sizeof(fh), header, header_len);
    if (copy) {
      char* p = it.owned.data() + sizeof(fh) + header_len;
      for (size_t i = 0; i < seg_count; ++i) {
        if (segs[i].size) std::memcpy(p, segs[i].data, segs[i].size);
        p += segs[i].size;
      }
      enqueue(ep, std::move(it));
      return ep->state_ == Endpoint::State::kConnected ? UCS_OK : UCS_ERR_CONNECTION_RESET;
    }
    it.segs.assign(segs, segs + seg_count);
    it.done = std::move(done);
    enqueue(ep, std::move(it));
    return UCS_INPROGRESS;
  }
  // rendezvous: announce, keep the user's ranges until CTS or FIN
  fh.type = kAmRts;
  fh.seg_count = static_cast<uint32_t>(seg_count);
  if (strided) {
    fh.flags |= kFlagDeviceRegions | kFlagLayout;
    fh.status = 1;
  } else if (device && cuda_mr_ && peer_is_local(ep)) {
    const bool ok = export_for_peer(ep, segs, seg_count, total, &regions);
    if (ok) {
      fh.flags |= kFlagDeviceRegions;
      fh.status = static_cast<int32_t>(regions.size());  // one per allocation touched, which may be more than the segments
    }
    if (ok && ep->out_flags_dev_ && opt_.push_threshold && total >= opt_.push_threshold) fh.flags |= kFlagPushOk;
  }
  it.owned.resize(sizeof(fh) + header_len + seg_count * 8 + regions.size() * sizeof(PeerRegionDesc) + (strided ? sizeof(WireLayout) : 0));
  char* p = it.owned.data();
  std::memcpy(p, &fh, sizeof(fh));
  p += sizeof(fh);
  if (header_len) std::memcpy(p, header, header_len);
  p += header_len;
  for (size_t i = 0; i < seg_count; ++i) {
    uint64_t sz = segs[i].size;
    std::memcpy(p, &sz, 8);
    p += 8;
  }
  if (!regions.empty()) std::memcpy(p, regions.data(), regions.size() * sizeof(PeerRegionDesc));
  p += regions.size() * sizeof(PeerRegionDesc);
  if (strided) {
    WireLayout l;
    l.ndim = hint->ndim;
    l.elem_size = static_cast<uint16_t>(hint->elem_size);
    l.src_dtype = hint->src_dtype;
    l.dst_dtype = hint->dst_dtype;
    std::memcpy(l.shape, hint->shape, sizeof(l.shape));
    std::memcpy(l.stride, hint->stride, sizeof(l.stride));
    l.span_bytes = hint->span_bytes;
    std::memcpy(p, &l, sizeof(l));
  }
  Endpoint::PendingSend ps;
  ps.segs.assign(segs, segs + seg_count);
  ps.mem_type = mem_type;
  ps.done = std::move(done);
  if (strided) ps.layout = hint;
  ps.keep = packed;
  ep->pending_sends_.emplace(id, std::move(ps));
  // The peer (or this worker's staging copy) reads the memory as soon as it hears of it: the announcement
  // waits until the producer is done. The sending thread does not.
  if (hint && hint->ready_event && cudaEventQuery(static_cast<cudaEvent_t>(hint->ready_event)) == cudaErrorNotReady) {
    held_sends_.push_back({ep, std::move(hint), std::move(it), id, std::chrono::steady_clock::now() + kHeldSendTimeout});
    ++stats_.sends_held;
    return UCS_INPROGRESS;
  }
  cudaGetLastError();
  enqueue(ep, std::move(it));
  return UCS_INPROGRESS;
}

void Worker::poll_held_sends() {
  for (auto it = held_sends_.begin(); it != held_sends_.end();) {
    if (cudaEventQuery(static_cast<cudaEvent_t>(it->hint->ready_event)) == cudaErrorNotReady) {
      if (it->msg_id && last_progress_ > it->deadline) {
        // the producer never finished: the send ends with an error instead of waiting for ever
        HeldSend h = std::move(*it);
        it = held_sends_.erase(it);
        UCX_CONN_ERROR << opt_.name << ": a device payload's producer did not finish in time; the send is dropped";
        if (eps_.count(h.ep)) {
          auto ps = h.ep->pending_sends_.find(h.msg_id);
          if (ps != h.ep->pending_sends_.end()) {
            Completion done = std::move(ps->second.done);
            h.ep->pending_sends_.erase(ps);
            if (done) done(UCS_ERR_TIMED_OUT);
          }
        }
        continue;
      }
      ++it;
      continue;
    }
    cudaGetLastError();  // done, or failed: either way nothing more to wait for (a failed producer shows in the data's consumer)
    HeldSend h = std::move(*it);
    it = held_sends_.erase(it);
    if (eps_.count(h.ep) && h.ep->state_ == Endpoint::State::kConnected) enqueue(h.ep, std::move(h.item));
  }
}

// The kernel's description of a gather from a WireLayout. Elements travel as opaque units: 1, 2 and 4 bytes
// as such, 8 and 16 as two or four 4-byte units under one more innermost dimension.
void Worker::fill_gather(eux_xfer_desc* d, const WireLayout& l) {
  const int64_t words = l.elem_size > 4 ? l.elem_size / 4 : 1;
  const int unit_dtype = l.elem_size == 1 ? EUX_DT_BYTES : (l.elem_size == 2 ? EUX_DT_F16 : EUX_DT_F32);
  d->src_dtype = d->dst_dtype = unit_dtype;
  d->op = EUX_OP_NONE;
  if (l.src_dtype != l.dst_dtype) {  // converted on the way (the layout was checked: both are floating-point types of the kernel)
    d->src_dtype = l.src_dtype;
    d->dst_dtype = l.dst_dtype;
    // a dense row-major source takes the vectorised kernel; anything else the element-wise one
    bool dense = true;
    int64_t expect = 1;
    for (int i = l.ndim - 1; i >= 0 && dense; --i) {
      dense = l.shape[i] == 1 || l.stride[i] == expect;
      expect *= l.shape[i];
    }
    if (dense) {
      uint64_t n = 1;
      for (int i = 0; i < l.ndim; ++i) n *= static_cast<uint64_t>(l.shape[i]);
      d->ndim = 0;
      d->n_elems = n;
      return;
    }
  }
  uint64_t n = 1;
  int nd = 0;
  for (int i = 0; i < l.ndim; ++i) {
    d->shape[nd] = l.shape[i];
    d->stride[nd] = l.stride[i] * words;
    n *= static_cast<uint64_t>(l.shape[i]);
    ++nd;
  }
  if (words > 1) {
    d->shape[nd] = words;
    d->stride[nd] = 1;
    n *= static_cast<uint64_t>(words);
    ++nd;
  }
  d->ndim = nd;
  d->n_elems = n;
}

std::shared_ptr<void> Worker::pack_local(const SendHint& h, const void* src) {
  if (!ensure_device()) return nullptr;
  if (h.elem_size > 4 && h.ndim >= kSendAttrMaxDims) return nullptr;
  void* tmp = nullptr;
  try {
    tmp = mr_.allocate(ucx_memory_type::CUDA, h.dense_bytes);
  } catch (...) {
    return nullptr;
  }
  UcxMemoryResourceManager* mr = &mr_;
  const size_t bytes = h.dense_bytes;
  std::shared_ptr<void> out(tmp, [mr, bytes](void* p) {
    try {
      mr->deallocate(ucx_memory_type::CUDA, p, bytes);
    } catch (...) {
    }
  });
  WireLayout l;
  l.ndim = h.ndim;
  l.elem_size = static_cast<uint16_t>(h.elem_size);
  l.src_dtype = h.src_dtype;
  l.dst_dtype = h.dst_dtype;
  std::memcpy(l.shape, h.shape, sizeof(l.shape));
  std::memcpy(l.stride, h.stride, sizeof(l.stride));
  eux_xfer_desc d{};
  d.src = src;
  d.dst = tmp;
  fill_gather(&d, l);
  flush_pull_batch();
  if (eux_xfer_launch(&d, counter_dev_, 0, stream_) != 0) return nullptr;
  ++stats_.kernel_launches;
  ++stats_.device_packs;
  if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream_)) != cudaSuccess) return nullptr;
  return out;
}

// CTS arrived: stream the payload as one DATA frame.
void Worker::start_data_send(Endpoint* ep, uint64_t msg_id, bool staged) {
  auto pit = ep->pending_sends_.find(msg_id);
  if (pit == ep->pending_sends_.end()) return;
  Endpoint::PendingSend ps = std::move(pit->second);
  ep->pending_sends_.erase(pit);
  size_t total = 0;
  for (auto& s : ps.segs) total += s.size;
  FrameHeader fh;
  fh.type = kRndvData;
  fh.msg_id = msg_id;
  fh.payload_len = total;
  Endpoint::SendItem it;
  it.owned.resize(sizeof(fh));
  std::memcpy(it.owned.data(), &fh, sizeof(fh));
  if (is_device_type(ps.mem_type)) {
    // device payload that the receiver cannot map: stage it through host memory
    (void)staged;
    if (ps.layout) {
      // ... and a strided one is made dense on the device first
      ps.keep = pack_local(*ps.layout, ps.segs[0].data);
      if (!ps.keep) {
        if (ps.done) ps.done(UCS_ERR_NO_MEMORY);
        return;
      }
      ps.segs[0].data = ps.keep.get();
      ps.layout.reset();
    }
    std::shared_ptr<void> bounce(std::malloc(total ? total : 1), std::free);
    try {
      char* dst = static_cast<char*>(bounce.get());
      for (auto& s : ps.segs) {
        mr_.memcpy(ucx_memory_type::HOST, dst, ps.mem_type, s.data, s.size);
        dst += s.size;
      }
    } catch (...) {
      if (ps.done) ps.done(UCS_ERR_IO_ERROR);
      return;
    }
    it.segs.push_back({bounce.get(), total});
    it.keep = bounce;
  } else {
    it.segs = std::move(ps.segs);
  }
  it.done = std::move(ps.done);
  enqueue(ep, std::move(it));
}

std::vector<uint64_t> Worker::rndv_segment_sizes(Endpoint* ep, uint64_t msg_id) const {
  auto e = eps_.find(ep);
  if (e == eps_.end()) return {};
  auto it = ep->rts_.find(msg_id);
  return it == ep->rts_.end() ? std::vector<uint64_t>{} : it->second.seg_sizes;
}

int Worker::rndv_recv(Endpoint* ep, uint64_t msg_id, const ucx_buffer_t* segs, size_t seg_count, ucx_memory_type_t mem_type,
                      Completion done, std::shared_ptr<const SendHint> ready) {
  if (ready && !ready->ready_event) ready.reset();
  if (!eps_.count(ep) || ep->state_ != Endpoint::State::kConnected) return UCS_ERR_NOT_CONNECTED;
  auto rit = ep->rts_.find(msg_id);
  if (rit == ep->rts_.end()) return UCS_ERR_NO_MESSAGE;
  Endpoint::RtsInfo info = std::move(rit->second);
  ep->rts_.erase(rit);
  size_t room = 0;
  for (size_t i = 0; i < seg_count; ++i) room += segs[i].size;
  if (room < info.payload_len) {
    send_control(ep, kRndvFin, 0, msg_id, UCS_ERR_MESSAGE_TRUNCATED);
    return UCS_ERR_MESSAGE_TRUNCATED;
  }
  const bool dst_device = is_device_type(mem_type);
  if (info.push_ok && !info.has_layout && dst_device && !info.regions.empty() && ep->shm_active_ && opt_.push_threshold) {
    int st = request_push(ep, msg_id, info, segs, seg_count, done, ready);
    if (st == UCS_INPROGRESS) return st;  // otherwise: pull it
  }
  if (!info.regions.empty() && dst_device) {
    int st = device_pull(ep, msg_id, info, segs, seg_count, done, ready);
    if (st == UCS_INPROGRESS || st == UCS_OK) {
      ++stats_.device_pulls;
      return st;
    }
    note_staged(ep, "the sender's memory could not be mapped, or no flag slot or launch was to be had");
  } else if (dst_device && is_device_type(info.mem_type)) {
    note_staged(ep, "the sender announced no usable device regions (allocation not exportable, or peer not shown to be on this host)");
  }
  Endpoint::PendingRecv pr;
  pr.mem_type = mem_type;
  pr.total = info.payload_len;
  pr.done = std::move(done);
  if (dst_device) {
    pr.bounce = std::shared_ptr<void>(std::malloc(info.payload_len ? info.payload_len : 1), std::free);
    pr.segs.push_back({pr.bounce.get(), static_cast<size_t>(info.payload_len)});
    size_t left = info.payload_len;
    for (size_t i = 0; i < seg_count && left > 0; ++i) {
      size_t t = std::min<size_t>(segs[i].size, left);
      pr.dev_dsts.push_back({segs[i].data, t});
      left -= t;
    }
  } else {
    pr.segs.assign(segs, segs + seg_count);
  }
  ep->pending_recvs_.emplace(msg_id, std::move(pr));
  send_control(ep, kRndvCts, is_device_type(info.mem_type) ? kFlagStage : 0, msg_id);
  return UCS_INPROGRESS;
}

// A device payload that goes device -> host -> wire -> host -> device is a silent factor of ten or
// more: say so, once per endpoint, at a level the default logger shows.
void Worker::note_staged(Endpoint* ep, const char* why) {
  ++stats_.device_staged;
  nvtx_mark("eux.transport.device_staged");
  if (ep->staged_logged_) return;
  ep->staged_logged_ = true;
  UCX_CONN_ERROR << opt_.name << ": device payload from " << ep->remote_.name_str << " (" << ep->peer_name_
                 << ") is staged through host memory: " << why << " (reported once per endpoint)";
}

void Worker::rndv_discard(Endpoint* ep, uint64_t msg_id) {
  if (!eps_.count(ep)) return;
  if (ep->rts_.erase(msg_id) && ep->state_ == Endpoint::State::kConnected)
    send_control(ep, kRndvFin, 0, msg_id, UCS_ERR_CANCELED);
}

// A send can be withdrawn while it waits for the receiver (RTS sent, no CTS yet)
// or while its frame has not started to go out. Once bytes of the frame are on
// the wire the user's memory is in use and the send runs to completion.
bool Worker::cancel_send(Endpoint* ep, uint64_t msg_id) {
  if (!eps_.count(ep)) return true;
  auto it = ep->pending_sends_.find(msg_id);
  if (it != ep->pending_sends_.end()) {
    ep->pending_sends_.erase(it);
    // an announcement that still waits for its payload's producer never leaves: the peer never hears of the message
    const size_t held = std::erase_if(held_sends_, [ep, msg_id](const HeldSend& h) { return h.ep == ep && h.msg_id == msg_id; });
    if (!held && ep->state_ == Endpoint::State::kConnected) send_control(ep, kRndvFin, kFlagFromSender, msg_id, UCS_ERR_CANCELED);
    return true;
  }
  for (auto s = ep->sendq_.begin(); s != ep->sendq_.end(); ++s) {
    FrameHeader fh;
    if (s->owned.size() < sizeof(fh)) continue;
    std::memcpy(&fh, s->owned.data(), sizeof(fh));
    if (fh.msg_id != msg_id || (fh.type != kAmEager && fh.type != kRndvData)) continue;
    if (s->owned_off == 0 && fh.type == kAmEager) {
      ep->sendq_.erase(s);
      return true;
    }
    return false;
  }
  return true;  // nothing in flight under that id
}

// A posted host receive can be withdrawn at any time (bytes that still arrive are
// drained and dropped). A device pull cannot: its kernel is writing the buffer.
bool Worker::cancel_recv(Endpoint* ep, uint64_t msg_id) {
  if (!eps_.count(ep)) return true;
  for (auto& d : device_ops_)
    if (d.ep == ep && d.msg_id == msg_id && d.send_fin) return false;
  for (auto& w : push_waits_)
    if (w.ep == ep && w.msg_id == msg_id) return false;  // the peer's kernel may be writing the buffers
  ep->pending_recvs_.erase(msg_id);
  return true;
}

// ---------------------------------------------------------------------------
// device data plane
// ---------------------------------------------------------------------------
void Worker::finish_connect(Endpoint* ep) {
  ep->await_dev_ring_ = false;
  Completion c = std::move(ep->on_connected_);
  ep->on_connected_ = nullptr;
  if (c && ep->state_ == Endpoint::State::kConnected) c(UCS_OK);
}

// The peer presented the uid of a worker that lives in this process (and this process's pid).
bool Worker::peer_is_this_process(const Endpoint* ep) const {
  return ep->remote_.addr.pid == addr_.pid && live_has(ep->remote_.addr.uid);
}
// Same host, shown by the handshake: the peer mapped the shared-memory channel that this side created
// (or the other way round), which only a process on this host can do; or it is this very process.
bool Worker::peer_is_local(const Endpoint* ep) const { return ep->shm_active_ || peer_is_this_process(ep); }

bool Worker::ensure_device() {
  if (device_ready_) return true;
  if (device_failed_ || opt_.device < 0) return false;
  cudaStream_t st = nullptr;
  if (cudaSetDevice(opt_.device) != cudaSuccess || cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess) {
    cudaGetLastError();
    device_failed_ = true;
    return false;
  }
  void *h = nullptr, *d = nullptr, *c = nullptr;
  if (eux_host_alloc_mapped(&h, &d, 4096) != 0 || cudaMalloc(&c, 256) != cudaSuccess || cudaMemsetAsync(c, 0, 256, st) != cudaSuccess ||
      cudaStreamSynchronize(st) != cudaSuccess) {
    cudaGetLastError();
    device_failed_ = true;
    return false;
  }
  if (int rc = eux_xfer_preload(); rc != 0) UCX_CONN_WARN << opt_.name << ": transfer kernels could not be loaded ahead of use: " << eux_error_string(rc);
  stream_ = st;
  flag_host_ = static_cast<uint64_t*>(h);
  flag_dev_ = static_cast<uint64_t*>(d);
  counter_dev_ = static_cast<uint32_t*>(c);
  device_ready_ = true;
  return true;
}

// Receiver-driven pull: map the sender's regions and copy them into the posted
// device segments with the transfer kernel; the last launch publishes a sequence
// number in pinned host memory that poll_device() watches.
int Worker::device_pull(Endpoint* ep, uint64_t msg_id, Endpoint::RtsInfo& info, const ucx_buffer_t* segs, size_t seg_count,
                        Completion& done, const std::shared_ptr<const SendHint>& ready) {
  if (!cuda_mr_ || !ensure_device()) return UCS_ERR_UNSUPPORTED;
  // the destination may still be in use by work queued before it was handed out: this worker's kernels come after it
  if (ready) cudaStreamWaitEvent(static_cast<cudaStream_t>(stream_), static_cast<cudaEvent_t>(ready->ready_event), 0);
  NvtxRange range("eux.transport.device_pull");
  std::vector<void*> srcs(info.regions.size());
  for (size_t i = 0; i < info.regions.size(); ++i) {
    srcs[i] = import_from_peer(ep, info.regions[i]);
    if (!srcs[i]) return UCS_ERR_UNSUPPORTED;
  }
  if (device_ops_.size() + 2 >= kFlagSlots) return UCS_ERR_UNSUPPORTED;  // every transfer in flight owns a flag slot
  if (info.has_layout) {
    // a strided view: gather it straight out of the sender's memory into the (one, dense) destination
    if (seg_count == 0 || segs[0].size < info.payload_len || (info.layout.elem_size > 4 && info.layout.ndim >= kSendAttrMaxDims)) return UCS_ERR_UNSUPPORTED;
    const uint64_t seq = ++device_seq_;
    eux_xfer_desc d{};
    d.src = srcs[0];
    d.dst = segs[0].data;
    fill_gather(&d, info.layout);
    d.flag = flag_dev_ + seq % kFlagSlots;
    d.flag_value = seq;
    flush_pull_batch();
    const int rc = eux_xfer_launch(&d, counter_dev_, 0, stream_);
    if (rc != 0) {
      --device_seq_;
      UCX_CONN_ERROR << "gather kernel launch failed: " << eux_error_string(rc);
      return UCS_ERR_UNSUPPORTED;
    }
    ++stats_.kernel_launches;
    ++stats_.device_gathers;
    device_ops_.push_back({seq, ep, msg_id, std::move(done), true, ready});
    return UCS_INPROGRESS;
  }
  // walk source regions and destination segments together
  size_t si = 0, so = 0, di = 0, dof = 0;
  struct Piece {
    const char* s;
    char* d;
    size_t n;
  };
  std::vector<Piece> pieces;
  while (si < srcs.size() && di < seg_count) {
    size_t sl = info.regions[si].length - so, dl = segs[di].size - dof;
    size_t n = std::min(sl, dl);
    if (n) pieces.push_back({static_cast<const char*>(srcs[si]) + so, static_cast<char*>(segs[di].data) + dof, n});
    so += n;
    dof += n;
    if (so == info.regions[si].length) ++si, so = 0;
    if (dof == segs[di].size) ++di, dof = 0;
  }
  if (pieces.empty()) {
    send_control(ep, kRndvFin, 0, msg_id, UCS_OK);
    return UCS_OK;
  }
  const uint64_t seq = ++device_seq_;
  uint64_t* const flag = flag_dev_ + seq % kFlagSlots;
  if (pieces.size() == 1 && pieces[0].n <= kBatchMaxBytes) {
    // a small message: it leaves with the others of this pass in one launch
    pull_batch_.push_back({pieces[0].s, pieces[0].d, pieces[0].n, flag, seq});
    device_ops_.push_back({seq, ep, msg_id, std::move(done), true, ready});
    if (pull_batch_.size() == EUX_PULL_BATCH_MAX) flush_pull_batch();
    return UCS_INPROGRESS;
  }
  flush_pull_batch();  // launches stay in the order of their sequence numbers
  for (size_t i = 0; i < pieces.size(); ++i) {
    eux_xfer_desc d{};
    d.src = pieces[i].s;
    d.dst = pieces[i].d;
    d.n_elems = pieces[i].n;
    d.src_dtype = d.dst_dtype = EUX_DT_BYTES;
    d.op = EUX_OP_NONE;
    if (i + 1 == pieces.size()) {
      d.flag = flag;
      d.flag_value = seq;
    }
    int rc = eux_xfer_launch(&d, counter_dev_, 0, stream_);
    if (rc != 0) {
      UCX_CONN_ERROR << "transfer kernel launch failed: " << eux_error_string(rc);
      return UCS_ERR_IO_ERROR;
    }
    ++stats_.kernel_launches;
  }
  device_ops_.push_back({seq, ep, msg_id, std::move(done), true, ready});
  return UCS_INPROGRESS;
}

// One launch for all the small pulls collected since the last call. If the launch fails, those
// transfers end with an error at both sides.
void Worker::flush_pull_batch() {
  if (pull_batch_.empty()) return;
  NvtxRange range("eux.transport.device_pull_batch");
  const int rc = eux_xfer_pull_batch_launch(pull_batch_.data(), static_cast<int>(pull_batch_.size()), stream_);
  if (rc == 0) ++stats_.kernel_launches;
  if (rc != 0) {
    UCX_CONN_ERROR << "batched transfer kernel launch failed: " << eux_error_string(rc);
    const uint64_t first = pull_batch_.front().flag_value, last = pull_batch_.back().flag_value;
    std::vector<DeviceOp> failed;
    for (auto it = device_ops_.begin(); it != device_ops_.end();) {
      if (it->seq >= first && it->seq <= last) {
        failed.push_back(std::move(*it));
        it = device_ops_.erase(it);
      } else {
        ++it;
      }
    }
    pull_batch_.clear();
    for (auto& op : failed) {
      if (op.ep && eps_.count(op.ep) && op.ep->state_ == Endpoint::State::kConnected)
        send_control(op.ep, kRndvFin, 0, op.msg_id, UCS_ERR_IO_ERROR);
      if (op.done) op.done(UCS_ERR_IO_ERROR);
    }
    return;
  }
  pull_batch_.clear();
}

void Worker::poll_device() {
  // Every transfer in flight owns its flag word, and transfers run on two streams (the worker's own and
  // the device's stream for large pushes), so they finish in any order: each is looked at on its own.
  for (size_t i = 0; i < device_ops_.size();) {
    const uint64_t seq = device_ops_[i].seq;
    if (*static_cast<volatile uint64_t*>(flag_host_ + seq % kFlagSlots) != seq) {
      ++i;
      continue;
    }
    std::atomic_thread_fence(std::memory_order_acquire);
    DeviceOp op = std::move(device_ops_[i]);
    device_ops_.erase(device_ops_.begin() + static_cast<std::ptrdiff_t>(i));
    if (op.send_fin && op.ep && eps_.count(op.ep) && op.ep->state_ == Endpoint::State::kConnected)
      send_control(op.ep, kRndvFin, 0, op.msg_id, UCS_OK);
    if (op.done) op.done(UCS_OK);  // may start new transfers: they are appended and looked at in this pass too
  }
  // payloads that peers push: small ones into ring slots, large ones into posted buffers. The peer's
  // kernel stores the flag word (in the shared page) after its data stores; this thread reads it.
  if (!eager_waits_.empty()) {
    const auto now = last_progress_;
    for (auto it = eager_waits_.begin(); it != eager_waits_.end();) {
      const bool arrived = it->shm->in_flags()[kEagerWordBase + it->slot] == it->seq;
      if (arrived) {
        std::atomic_thread_fence(std::memory_order_acquire);
        EagerWait w = std::move(*it);
        it = eager_waits_.erase(it);
        ++stats_.device_eager_recv;
        nvtx_mark("eux.transport.device_eager_arrived");
        if (on_am && w.ep) on_am(std::move(w.arrival));
        else if (w.arrival.header) mr_.deallocate(ucx_memory_type::HOST, w.arrival.header, w.arrival.header_len);
        continue;  // the slot goes back when the arrival's keep-alive token is dropped
      }
      if (now > it->deadline) {
        UCX_CONN_ERROR << opt_.name << ": the payload of an eager device message (slot " << it->slot << ") never arrived; dropped";
        if (it->arrival.header) mr_.deallocate(ucx_memory_type::HOST, it->arrival.header, it->arrival.header_len);
        it = eager_waits_.erase(it);
        continue;
      }
      ++it;
    }
  }
  if (!push_waits_.empty()) {
    const auto now = last_progress_;
    for (auto it = push_waits_.begin(); it != push_waits_.end();) {
      const bool arrived = it->shm->in_flags()[it->word] == it->value;
      if (!arrived && now <= it->deadline) {
        ++it;
        continue;
      }
      std::atomic_thread_fence(std::memory_order_acquire);
      PushWait w = std::move(*it);
      it = push_waits_.erase(it);
      if (w.ep && eps_.count(w.ep) && w.ep->push_inflight_) --w.ep->push_inflight_;
      if (arrived) nvtx_mark("eux.transport.device_push_arrived");
      if (arrived) ++stats_.device_push_recv;
      else UCX_CONN_ERROR << opt_.name << ": a pushed payload (message " << w.msg_id << ") did not arrive in time";
      if (w.done) w.done(arrived ? UCS_OK : UCS_ERR_TIMED_OUT);
    }
  }
}

// ---------------------------------------------------------------------------
// device channel: flag pages registered with CUDA, eager receive rings, pushed rendezvous
// ---------------------------------------------------------------------------
Endpoint::DevRing::~DevRing() {
  try {
    if (mr && base) mr->deallocate(ucx_memory_type::CUDA, base, bytes);
  } catch (...) {
  }
}

// ---- file-descriptor channel ---------------------------------------------------------------------
// A cuMemCreate allocation is shared between processes as a POSIX file descriptor, and a descriptor
// travels only as ancillary data of a Unix socket. Every worker that manages device memory listens on a
// socket in /dev/shm named after its random id; the side that connected an endpoint (and so knows the
// peer's id from the handshake) connects to it once the shared-memory channel has shown that both are on
// one host, and says which endpoint it belongs to. From then on either side sends
// {allocation number, size} + descriptor the first time it announces memory of that allocation, always
// before the frame that refers to it, so the receiver finds the descriptor waiting when it reads the frame.
namespace {
constexpr uint32_t kFdMagic = 0x44465845u;  // "EXFD"
struct FdMsg {
  uint32_t magic = kFdMagic;
  uint32_t kind = 0;  // 0: hello (a = the connecting worker's id), 1: descriptor (a = allocation number, b = size)
  uint64_t a = 0, b = 0;
};
std::string fd_path_of(uint64_t uid) {
  char buf[64];
  std::snprintf(buf, sizeof(buf), "/dev/shm/eux-fd-%016llx", static_cast<unsigned long long>(uid));
  return buf;
}
bool fill_unix_addr(const std::string& path, sockaddr_un* un) {
  if (path.size() >= sizeof(un->sun_path)) return false;
  un->sun_family = AF_UNIX;
  std::memcpy(un->sun_path, path.c_str(), path.size() + 1);
  return true;
}
}  // namespace

void Worker::open_fd_listener() {
  sockaddr_un un{};
  fd_path_ = fd_path_of(addr_.uid);
  if (!fill_unix_addr(fd_path_, &un)) return;
  int fd = ::socket(AF_UNIX, SOCK_SEQPACKET | SOCK_CLOEXEC | SOCK_NONBLOCK, 0);
  if (fd < 0) return;
  ::unlink(fd_path_.c_str());
  epoll_event ev{};
  ev.events = EPOLLIN;
  ev.data.u64 = (uint64_t(1) << 63) | kFdListenerTag;
  // only this user may connect: what travels here are handles to device memory
  if (::bind(fd, reinterpret_cast<sockaddr*>(&un), sizeof(un)) != 0 || ::chmod(fd_path_.c_str(), 0600) != 0 || ::listen(fd, 64) != 0 ||
      epoll_ctl(epfd_, EPOLL_CTL_ADD, fd, &ev) != 0) {
    ::close(fd);
    ::unlink(fd_path_.c_str());
    return;
  }
  fd_listen_ = fd;
}

void Worker::accept_fd_channels() {
  if (fd_listen_ < 0) return;
  for (;;) {
    int fd = ::accept4(fd_listen_, nullptr, nullptr, SOCK_CLOEXEC | SOCK_NONBLOCK);
    if (fd < 0) return;
    // who is at the other end, as the kernel knows it: a process of this user, and (below) the very process
    // whose worker the hello names
    ucred cred{};
    socklen_t cred_len = sizeof(cred);
    if (getsockopt(fd, SOL_SOCKET, SO_PEERCRED, &cred, &cred_len) != 0 || cred.uid != geteuid()) {
      ::close(fd);
      continue;
    }
    // the peer wrote its hello right after connect(): it is there, or about to be
    FdMsg m{};
    ssize_t n = -1;
    for (int tries = 0; tries < 50; ++tries) {
      n = ::recv(fd, &m, sizeof(m), 0);
      if (n >= 0 || (errno != EAGAIN && errno != EWOULDBLOCK)) break;
      pollfd pf{fd, POLLIN, 0};
      ::poll(&pf, 1, 1);
    }
    Endpoint* owner = nullptr;
    if (n == ssize_t(sizeof(m)) && m.magic == kFdMagic && m.kind == 0)
      for (auto& [p, ep] : eps_)
        if (p->shm_active_ && p->fd_chan_ < 0 && p->remote_.addr.uid == m.a && !p->shm_->creator() &&
            (cred.pid == 0 || static_cast<uint32_t>(cred.pid) == p->remote_.addr.pid))  // pid 0: the peer lives in a pid namespace that this one cannot see into
          owner = p;
    if (!owner) {
      ::close(fd);
      continue;
    }
    owner->fd_chan_ = fd;
  }
}

void Worker::connect_fd_channel(Endpoint* ep) {
  if (!cuda_mr_ || ep->fd_chan_ >= 0 || peer_is_this_process(ep)) return;
  sockaddr_un un{};
  if (!fill_unix_addr(fd_path_of(ep->remote_.addr.uid), &un)) return;
  int fd = ::socket(AF_UNIX, SOCK_SEQPACKET | SOCK_CLOEXEC, 0);
  if (fd < 0) return;
  // a local connect: done at once, or refused (the peer manages no device memory, or shares no /dev/shm)
  FdMsg hello;
  hello.a = addr_.uid;
  if (::connect(fd, reinterpret_cast<sockaddr*>(&un), sizeof(un)) != 0 || ::send(fd, &hello, sizeof(hello), MSG_NOSIGNAL) != ssize_t(sizeof(hello)) ||
      set_nonblocking(fd) != 0) {
    ::close(fd);
    return;
  }
  ep->fd_chan_ = fd;
}

void Worker::close_fd_channel(Endpoint* ep) {
  if (ep->fd_chan_ >= 0) {
    ::close(ep->fd_chan_);
    ep->fd_chan_ = -1;
  }
  ep->vmm_sent_.clear();
  // mappings of the peer's allocations go with the endpoint, unless another endpoint of this worker talks
  // to the same peer worker (its transfers may be using them)
  if (cuda_mr_ && ep->remote_.addr.uid) {
    bool shared = false;
    for (auto& [p, other] : eps_) shared = shared || (p != ep && p->remote_.addr.uid == ep->remote_.addr.uid && p->state_ == Endpoint::State::kConnected);
    if (!shared) cuda_mr_->release_vmm_of(ep->remote_.addr.uid);
  }
}

bool Worker::send_vmm_fd(Endpoint* ep, const PeerRegionDesc& d) {
  PeerVmmRef ref;
  std::memcpy(&ref, d.handle, sizeof(ref));
  if (ep->vmm_sent_.count(ref.id)) return true;
  if (ep->fd_chan_ < 0) accept_fd_channels();
  if (ep->fd_chan_ < 0) return false;
  const int fd = cuda_mr_->export_vmm_fd(d);
  if (fd < 0) return false;
  FdMsg m;
  m.kind = 1;
  m.a = ref.id;
  m.b = ref.size;
  iovec iov{&m, sizeof(m)};
  alignas(cmsghdr) char ctl[CMSG_SPACE(sizeof(int))] = {};
  msghdr mh{};
  mh.msg_iov = &iov;
  mh.msg_iovlen = 1;
  mh.msg_control = ctl;
  mh.msg_controllen = sizeof(ctl);
  cmsghdr* c = CMSG_FIRSTHDR(&mh);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
  const ssize_t n = ::sendmsg(ep->fd_chan_, &mh, MSG_NOSIGNAL | MSG_DONTWAIT);
  ::close(fd);
  if (n != ssize_t(sizeof(m))) return false;  // the socket's buffer is full: this message is staged, the next one tries again
  ep->vmm_sent_.insert(ref.id);
  ++stats_.vmm_fds_sent;
  return true;
}

void Worker::drain_fd_channel(Endpoint* ep) {
  if (ep->fd_chan_ < 0) accept_fd_channels();
  if (ep->fd_chan_ < 0 || !cuda_mr_) return;
  for (;;) {
    FdMsg m{};
    iovec iov{&m, sizeof(m)};
    alignas(cmsghdr) char ctl[CMSG_SPACE(4 * sizeof(int))] = {};
    msghdr mh{};
    mh.msg_iov = &iov;
    mh.msg_iovlen = 1;
    mh.msg_control = ctl;
    mh.msg_controllen = sizeof(ctl);
    const ssize_t n = ::recvmsg(ep->fd_chan_, &mh, MSG_DONTWAIT | MSG_CMSG_CLOEXEC);
    if (n <= 0) return;
    std::vector<int> fds;
    for (cmsghdr* c = CMSG_FIRSTHDR(&mh); c; c = CMSG_NXTHDR(&mh, c)) {
      if (c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) continue;
      const size_t cnt = (c->cmsg_len - CMSG_LEN(0)) / sizeof(int);
      for (size_t i = 0; i < cnt; ++i) {
        int fd;
        std::memcpy(&fd, CMSG_DATA(c) + i * sizeof(int), sizeof(int));
        fds.push_back(fd);
      }
    }
    if (n == ssize_t(sizeof(m)) && m.magic == kFdMagic && m.kind == 1 && fds.size() == 1 && ensure_device()) {
      if (cuda_mr_->import_vmm(ep->remote_.addr.uid, PeerVmmRef{m.a, m.b}, fds[0])) ++stats_.vmm_fds_recv;
      else UCX_CONN_WARN << opt_.name << ": an allocation of " << m.b << " bytes offered by " << ep->peer_name_ << " could not be mapped";
    }
    for (int fd : fds) ::close(fd);
  }
}

bool Worker::export_for_peer(Endpoint* ep, const ucx_buffer_t* segs, size_t seg_count, uint64_t limit, std::vector<PeerRegionDesc>* out) {
  out->clear();
  uint64_t left = limit;
  for (size_t i = 0; i < seg_count && left > 0; ++i) {
    const uint64_t n = std::min<uint64_t>(segs[i].size, left);
    if (n == 0) continue;
    if (!cuda_mr_->export_regions(segs[i].data, n, out) || out->size() > kMaxSegCount) {
      out->clear();
      return false;
    }
    left -= n;
  }
  if (left != 0 || out->empty()) {
    out->clear();
    return false;
  }
  if (!peer_is_this_process(ep))
    for (auto& d : *out)
      if (d.kind == kRegionVmm && !send_vmm_fd(ep, d)) {
        out->clear();
        return false;
      }
  return true;
}

void* Worker::import_from_peer(Endpoint* ep, const PeerRegionDesc& d) {
  const bool same = peer_is_this_process(ep);
  void* p = cuda_mr_->import_region(d, same, ep->remote_.addr.uid);
  if (!p && !same && d.kind == kRegionVmm) {
    drain_fd_channel(ep);  // its descriptor was sent ahead of the frame that named it
    p = cuda_mr_->import_region(d, same, ep->remote_.addr.uid);
  }
  return p;
}

// Runs once per endpoint, when its shared-memory channel becomes active (so the peer is on this host)
// and this worker drives a GPU: registers the channel's flag pages with CUDA, allocates the receive ring
// for small device payloads and tells the peer where it is.
void Worker::setup_device_channel(Endpoint* ep) {
  if (ep->dev_tried_ || opt_.device < 0 || !cuda_mr_ || !ep->shm_) return;
  ep->dev_tried_ = true;
  // Whatever comes of the set-up, the peer is told (a ring, or "none"): a connecting peer holds its
  // "connected" back until it knows, so that its first message already finds the fast paths.
  PeerRegionDesc d;
  uint32_t geo[2] = {0, 0};
  auto announce = [&] {
    FrameHeader fh;
    fh.type = kDevRing;
    fh.header_len = sizeof(PeerRegionDesc) + 8;
    Endpoint::SendItem it;
    it.owned.resize(sizeof(fh) + fh.header_len);
    std::memcpy(it.owned.data(), &fh, sizeof(fh));
    std::memcpy(it.owned.data() + sizeof(fh), &d, sizeof(d));
    std::memcpy(it.owned.data() + sizeof(fh) + sizeof(d), geo, 8);
    enqueue(ep, std::move(it));
  };
  if ((!opt_.dev_eager_limit && !opt_.push_threshold) || !ensure_device()) {
    announce();
    return;
  }
  if (cudaHostRegister(ep->shm_->flag_area(), ShmChannel::flag_area_bytes(), cudaHostRegisterMapped | cudaHostRegisterPortable) != cudaSuccess) {
    cudaGetLastError();
    UCX_CONN_WARN << opt_.name << ": the shared flag page could not be registered with CUDA; device payloads will be pulled";
    announce();
    return;
  }
  ep->flags_registered_ = true;
  void* dev = nullptr;
  if (cudaHostGetDevicePointer(&dev, const_cast<uint64_t*>(ep->shm_->out_flags()), 0) != cudaSuccess || !dev) {
    cudaGetLastError();
    announce();
    return;
  }
  ep->out_flags_dev_ = static_cast<uint64_t*>(dev);
  if (opt_.dev_eager_limit) {
    // the ring: kEagerSlots slots, allocated from the pooled (already exportable) device memory
    auto ring = std::make_shared<Endpoint::DevRing>();
    try {
      ring->slot_bytes = eager_slot_bytes(opt_.dev_eager_limit);
      ring->bytes = size_t(kEagerSlots) * ring->slot_bytes;
      ring->base = mr_.allocate(ucx_memory_type::CUDA, ring->bytes);
      ring->mr = &mr_;
      if (cuda_mr_->export_region(ring->base, ring->bytes, &d)) {
        ep->rx_ring_ = std::move(ring);
        geo[0] = kEagerSlots;
        geo[1] = ep->rx_ring_->slot_bytes;
      }
    } catch (...) {
    }
  }
  announce();
}

// The peer's ring: map it and mark every slot free.
void Worker::on_dev_ring(Endpoint* ep, const FrameHeader& fh, const char* body) {
  // a connect that was held back for this frame completes now, whatever the frame says
  struct Release {
    Worker* w;
    Endpoint* ep;
    ~Release() { w->finish_connect(ep); }
  } release{this, ep};
  if (ep->fd_chan_ < 0) accept_fd_channels();  // the peer connected it before it sent this frame
  if (fh.header_len < sizeof(PeerRegionDesc) + 8 || !cuda_mr_ || !peer_is_local(ep) || !ep->out_flags_dev_) return;
  PeerRegionDesc d;
  uint32_t geo[2];
  std::memcpy(&d, body, sizeof(d));
  std::memcpy(geo, body + sizeof(d), 8);
  if (geo[0] == 0 || geo[0] > 64 || geo[1] == 0 || geo[1] > kEagerSlotBytesMax || uint64_t(geo[0]) * geo[1] != d.length) return;
  void* p = cuda_mr_->import_region(d, peer_is_this_process(ep));
  if (!p) return;
  ep->tx_ring_ = static_cast<char*>(p);
  ep->tx_slots_ = geo[0];
  ep->tx_slot_bytes_ = geo[1];
  ep->tx_free_ = geo[0] == 64 ? ~uint64_t(0) : ((uint64_t(1) << geo[0]) - 1);
}

// Before the shared segment is unmapped nothing on the GPU may still write into its flag page.
void Worker::teardown_device_channel(Endpoint* ep) {
  for (auto it = eager_waits_.begin(); it != eager_waits_.end();) {
    if (it->ep != ep) {
      ++it;
      continue;
    }
    if (it->arrival.header) mr_.deallocate(ucx_memory_type::HOST, it->arrival.header, it->arrival.header_len);
    it = eager_waits_.erase(it);
  }
  std::vector<Completion> cbs;
  for (auto it = push_waits_.begin(); it != push_waits_.end();) {
    if (it->ep != ep) {
      ++it;
      continue;
    }
    if (it->done) cbs.push_back(std::move(it->done));
    it = push_waits_.erase(it);
  }
  ep->push_inflight_ = 0;
  ep->tx_ring_ = nullptr;
  ep->tx_free_ = 0;
  ep->out_flags_dev_ = nullptr;
  if (ep->flags_registered_ && ep->shm_) {
    if (stream_) cudaStreamSynchronize(static_cast<cudaStream_t>(stream_));  // kernels of this worker that target the page (bounded)
    if (bulk_used_)
      if (cudaStream_t b = bulk_stream_for(opt_.device)) cudaStreamSynchronize(b);
    cudaHostUnregister(ep->shm_->flag_area());
    cudaGetLastError();
    ep->flags_registered_ = false;
  }
  ep->rx_ring_.reset();  // slots still held by the application keep the ring alive through their tokens
  for (auto& cb : cbs) cb(UCS_ERR_CONNECTION_RESET);
}

// Small device payload: one CTA of the next batched launch stores it into a free slot of the peer's ring,
// then raises the slot's flag in the shared page (the peer's host polls it) and this worker's own
// completion word. The active-message header travels at once through the control ring.
int Worker::dev_eager_send(Endpoint* ep, const void* header, size_t header_len, const ucx_buffer_t& seg, ucx_memory_type_t mem_type,
                           uint64_t msg_id, Completion& done, const std::shared_ptr<const SendHint>& hint) {
  if (!ensure_device() || device_ops_.size() + 2 >= kFlagSlots) return UCS_ERR_NO_RESOURCE;
  const uint32_t run = seg.size ? static_cast<uint32_t>((seg.size + ep->tx_slot_bytes_ - 1) / ep->tx_slot_bytes_) : 1;
  if (run > eager_run_max(ep->tx_slot_bytes_) || run > ep->tx_slots_) return UCS_ERR_NO_RESOURCE;
  const bool strided = hint && hint->ndim > 0;
  if (strided && hint->elem_size > 4 && hint->ndim >= kSendAttrMaxDims) return UCS_ERR_NO_RESOURCE;
  ep->tx_free_ |= ep->shm_->in_words()[0].exchange(0, std::memory_order_acquire);  // slots the peer has handed back
  if (!ep->tx_free_) return UCS_ERR_NO_RESOURCE;
  // the lowest run of `run` consecutive free slots
  uint64_t starts = ep->tx_free_;
  for (uint32_t i = 1; i < run; ++i) starts &= ep->tx_free_ >> i;
  if (ep->tx_slots_ < 64) starts &= (uint64_t(1) << (ep->tx_slots_ - run + 1)) - 1;
  if (!starts) return UCS_ERR_NO_RESOURCE;
  const uint32_t slot = static_cast<uint32_t>(__builtin_ctzll(starts));
  const uint64_t run_mask = ((run == 64 ? ~uint64_t(0) : (uint64_t(1) << run) - 1)) << slot;
  ep->tx_free_ &= ~run_mask;
  const uint64_t value = ++ep->tx_seq_;
  const uint64_t seq = ++device_seq_;
  eux_pull_item item{};
  item.src = seg.data;
  item.dst = ep->tx_ring_ + size_t(slot) * ep->tx_slot_bytes_;
  item.nbytes = seg.size;
  item.flag = ep->out_flags_dev_ + kEagerWordBase + slot;
  item.flag_value = value;
  item.flag2 = flag_dev_ + seq % kFlagSlots;
  item.flag2_value = seq;
  // this worker's kernel reads the payload: it is ordered after the producer on the device
  if (seg.size && hint && hint->ready_event) cudaStreamWaitEvent(static_cast<cudaStream_t>(stream_), static_cast<cudaEvent_t>(hint->ready_event), 0);
  if (seg.size && (strided || seg.size > kEagerBatchBytes)) {
    // gathered on its way into the slot, or too much for one CTA: a launch of its own
    eux_xfer_desc d{};
    d.src = seg.data;
    d.dst = item.dst;
    if (strided) {
      WireLayout l;
      l.ndim = hint->ndim;
      l.elem_size = static_cast<uint16_t>(hint->elem_size);
      l.src_dtype = hint->src_dtype;
      l.dst_dtype = hint->dst_dtype;
      std::memcpy(l.shape, hint->shape, sizeof(l.shape));
      std::memcpy(l.stride, hint->stride, sizeof(l.stride));
      fill_gather(&d, l);
    } else {
      d.n_elems = seg.size;
      d.src_dtype = d.dst_dtype = EUX_DT_BYTES;
      d.op = EUX_OP_NONE;
    }
    d.flag = item.flag;
    d.flag_value = item.flag_value;
    d.flag2 = item.flag2;
    d.flag2_value = item.flag2_value;
    flush_pull_batch();
    if (eux_xfer_launch(&d, counter_dev_, 0, stream_) != 0) {
      --device_seq_;
      --ep->tx_seq_;
      ep->tx_free_ |= run_mask;
      return UCS_ERR_NO_RESOURCE;
    }
    ++stats_.kernel_launches;
    if (strided) ++stats_.device_gathers;
    device_ops_.push_back({seq, ep, msg_id, std::move(done), false, hint});
  } else if (seg.size) {
    pull_batch_.push_back(item);
    device_ops_.push_back({seq, ep, msg_id, std::move(done), false, hint});
    if (pull_batch_.size() == EUX_PULL_BATCH_MAX) flush_pull_batch();
  } else {
    --device_seq_;
  }
  FrameHeader fh;
  fh.type = kAmDevEager;
  fh.header_len = static_cast<uint32_t>(header_len);
  fh.payload_len = seg.size;
  fh.msg_id = msg_id;
  fh.mem_type = static_cast<uint32_t>(mem_type);
  fh.status = static_cast<int32_t>(slot | (run << 8));  // first slot, and how many the payload takes
  Endpoint::SendItem it;
  it.owned.resize(sizeof(fh) + header_len + 8);
  std::memcpy(it.owned.data(), &fh, sizeof(fh));
  if (header_len) std::memcpy(it.owned.data() + sizeof(fh), header, header_len);
  std::memcpy(it.owned.data() + sizeof(fh) + header_len, &value, 8);
  enqueue(ep, std::move(it));
  ++stats_.device_eager_sent;
  nvtx_mark("eux.transport.device_eager_send");
  return ep->state_ == Endpoint::State::kConnected ? UCS_INPROGRESS : UCS_ERR_CONNECTION_RESET;
}

void Worker::on_dev_eager(Endpoint* ep, const FrameHeader& fh, const char* body) {
  const uint32_t slot = static_cast<uint32_t>(fh.status) & 0xffu, run = (static_cast<uint32_t>(fh.status) >> 8) & 0xffu;
  if (!ep->rx_ring_ || !ep->shm_ || run == 0 || run > eager_run_max(ep->rx_ring_->slot_bytes) || slot + run > kEagerSlots ||
      fh.payload_len > uint64_t(run) * ep->rx_ring_->slot_bytes) {
    UCX_CONN_ERROR << opt_.name << ": eager device frame from " << ep->peer_name_ << " names a slot this worker never offered";
    ++stats_.frames_refused;
    fail(ep, UCS_ERR_IO_ERROR);
    return;
  }
  EagerWait w;
  w.ep = ep;
  w.shm = ep->shm_;
  w.ring = ep->rx_ring_;
  w.slot = slot;
  std::memcpy(&w.seq, body + fh.header_len, 8);
  w.deadline = std::chrono::steady_clock::now() + kEagerArrivalTimeout;
  AmArrival& a = w.arrival;
  a.ep = ep;
  a.header_len = fh.header_len;
  a.header = fh.header_len ? mr_.allocate(ucx_memory_type::HOST, fh.header_len) : nullptr;
  if (fh.header_len) std::memcpy(a.header, body, fh.header_len);
  a.data = static_cast<char*>(w.ring->base) + size_t(slot) * w.ring->slot_bytes;
  a.data_len = fh.payload_len;
  a.msg_id = fh.msg_id;
  a.sender_mem_type = static_cast<ucx_memory_type_t>(fh.mem_type);
  a.data_mem_type = ucx_memory_type::CUDA;
  // Dropping the token hands the slot back: a bit in the word the sender's host thread collects. It
  // may be dropped on any thread, long after the endpoint is gone: it owns what it touches.
  struct SlotToken {
    std::shared_ptr<ShmChannel> shm;
    std::shared_ptr<Endpoint::DevRing> ring;
    uint64_t mask;  // the slots of the payload's run
    int device;
    SlotToken(std::shared_ptr<ShmChannel> s, std::shared_ptr<Endpoint::DevRing> r, uint64_t m, int dev)
        : shm(std::move(s)), ring(std::move(r)), mask(m), device(dev) {}
    SlotToken(const SlotToken&) = delete;  // exactly one object stands for the slots: its end hands them back
    SlotToken& operator=(const SlotToken&) = delete;
    ~SlotToken() {
      // ... once the GPU work that the application queued to read them has run (see set_consumer_event_hook)
      if (void* ev = record_consumer_event(device)) {
        std::lock_guard lk(g_slot_release_mu);
        g_slot_releases.push_back({ev, device, shm, mask});
        g_slot_release_count.store(g_slot_releases.size(), std::memory_order_release);
      } else {
        shm->out_words()[0].fetch_or(mask, std::memory_order_release);
      }
    }
  };
  a.data_keep = std::make_shared<SlotToken>(w.shm, w.ring, ((uint64_t(1) << run) - 1) << slot, opt_.device);
  eager_waits_.push_back(std::move(w));
}

// Receiver side of a pushed rendezvous: answer the RTS with the posted buffers' regions and the flag word
// the sender's kernel shall raise when the bytes are in place.
int Worker::request_push(Endpoint* ep, uint64_t msg_id, Endpoint::RtsInfo& info, const ucx_buffer_t* segs, size_t seg_count,
                         Completion& done, const std::shared_ptr<const SendHint>& ready) {
  if (!cuda_mr_ || ep->push_inflight_ + 1 >= kPushWords || seg_count > kMaxSegCount) return UCS_ERR_UNSUPPORTED;
  std::vector<PeerRegionDesc> regions;
  if (!export_for_peer(ep, segs, seg_count, info.payload_len, &regions)) return UCS_ERR_UNSUPPORTED;
  uint64_t room = 0;
  for (auto& d : regions) {
    if (!d.exportable) return UCS_ERR_UNSUPPORTED;
    room += d.length;
  }
  if (room != info.payload_len || regions.empty()) return UCS_ERR_UNSUPPORTED;
  const uint64_t value = ++ep->push_seq_;
  const uint32_t word = static_cast<uint32_t>(value % kPushWords);
  ++ep->push_inflight_;
  FrameHeader fh;
  fh.type = kRndvCts;
  fh.flags = kFlagPush;
  fh.msg_id = msg_id;
  fh.seg_count = static_cast<uint32_t>(regions.size());
  fh.header_len = static_cast<uint32_t>(regions.size() * sizeof(PeerRegionDesc));
  fh.payload_len = value;
  fh.status = static_cast<int32_t>(word);
  Endpoint::SendItem it;
  it.owned.resize(sizeof(fh) + fh.header_len);
  std::memcpy(it.owned.data(), &fh, sizeof(fh));
  std::memcpy(it.owned.data() + sizeof(fh), regions.data(), fh.header_len);
  PushWait w;
  w.ep = ep;
  w.shm = ep->shm_;
  w.msg_id = msg_id;
  w.word = word;
  w.value = value;
  w.done = std::move(done);
  w.segs.assign(segs, segs + seg_count);
  // a bound that no healthy transfer comes near: 30 s plus a second per GiB
  w.deadline = std::chrono::steady_clock::now() + std::chrono::seconds(30 + (info.payload_len >> 30));
  w.info = std::move(info);
  w.ready = ready;
  push_waits_.push_back(std::move(w));
  // the peer writes as soon as it is asked to: it is asked once the buffers may be written
  if (ready && cudaEventQuery(static_cast<cudaEvent_t>(ready->ready_event)) == cudaErrorNotReady) {
    held_sends_.push_back({ep, ready, std::move(it), 0, {}});  // bounded by the push wait's own deadline
    ++stats_.sends_held;
    return UCS_INPROGRESS;
  }
  cudaGetLastError();
  enqueue(ep, std::move(it));
  nvtx_mark("eux.transport.cts_push_sent");
  return UCS_INPROGRESS;
}

// Sender side: CTS(push) arrived. Map the receiver's regions and copy the payload into them with the
// transfer kernel; the last launch raises the receiver's flag word and this worker's own.
void Worker::on_push_cts(Endpoint* ep, const FrameHeader& fh, const char* body) {
  auto pit = ep->pending_sends_.find(fh.msg_id);
  if (pit == ep->pending_sends_.end()) return;  // withdrawn meanwhile; the FIN(cancelled) is on its way
  const uint32_t word = static_cast<uint32_t>(fh.status);
  auto refuse = [&] { send_control(ep, kRndvFin, kFlagFromSender, fh.msg_id, UCS_ERR_UNSUPPORTED); };  // the send stays pending: the receiver pulls
  if (!peer_is_local(ep) || !ep->out_flags_dev_ || !cuda_mr_ || word >= kPushWords || fh.seg_count == 0 ||
      fh.header_len != size_t(fh.seg_count) * sizeof(PeerRegionDesc) || !ensure_device() || device_ops_.size() + 2 >= kFlagSlots) {
    refuse();
    return;
  }
  std::vector<PeerRegionDesc> regions(fh.seg_count);
  std::memcpy(regions.data(), body, fh.header_len);
  std::vector<char*> dsts(regions.size());
  uint64_t room = 0;
  for (size_t i = 0; i < regions.size(); ++i) {
    dsts[i] = static_cast<char*>(import_from_peer(ep, regions[i]));
    if (!dsts[i]) {
      refuse();
      return;
    }
    room += regions[i].length;
  }
  auto& ps = pit->second;
  uint64_t total = 0;
  for (auto& sgm : ps.segs) total += sgm.size;
  if (room < total) {
    refuse();
    return;
  }
  NvtxRange range("eux.transport.device_push");
  // walk source segments and destination regions together
  std::vector<std::pair<const void*, void*>> ptrs;
  std::vector<size_t> lens;
  size_t si = 0, so = 0, di = 0, dof = 0;
  while (si < ps.segs.size() && di < regions.size()) {
    const size_t sl = ps.segs[si].size - so, dl = regions[di].length - dof;
    const size_t n = std::min(sl, dl);
    if (n) {
      ptrs.emplace_back(static_cast<const char*>(ps.segs[si].data) + so, dsts[di] + dof);
      lens.push_back(n);
    }
    so += n;
    dof += n;
    if (so == ps.segs[si].size) ++si, so = 0;
    if (dof == regions[di].length) ++di, dof = 0;
  }
  const uint64_t seq = ++device_seq_;
  flush_pull_batch();  // launches stay in the order of their sequence numbers
  int rc = launch_pieces(ptrs, lens, ep->out_flags_dev_ + word, fh.payload_len, flag_dev_ + seq % kFlagSlots, seq);
  if (rc != 0) {
    --device_seq_;
    UCX_CONN_ERROR << "transfer kernel launch failed: " << eux_error_string(rc);
    refuse();
    return;
  }
  Endpoint::PendingSend sent = std::move(ps);
  ep->pending_sends_.erase(pit);
  device_ops_.push_back({seq, ep, fh.msg_id, std::move(sent.done), false});
  ++stats_.device_pushes;
}

int Worker::launch_pieces(const std::vector<std::pair<const void*, void*>>& ptrs, const std::vector<size_t>& lens, uint64_t* flag,
                          uint64_t flag_value, uint64_t* flag2, uint64_t flag2_value) {
  // the process-wide stream of this device (see bulk_stream_for), with a last-CTA counter of its own: the
  // worker's other transfers run beside these on the worker's stream
  cudaStream_t bulk = bulk_stream_for(opt_.device);
  void* const st = bulk ? static_cast<void*>(bulk) : stream_;
  uint32_t* const counter = bulk ? counter_dev_ + 16 : counter_dev_;
  bulk_used_ = bulk_used_ || bulk != nullptr;
  for (size_t i = 0; i < ptrs.size(); ++i) {
    eux_xfer_desc d{};
    d.src = ptrs[i].first;
    d.dst = ptrs[i].second;
    d.n_elems = lens[i];
    d.src_dtype = d.dst_dtype = EUX_DT_BYTES;
    d.op = EUX_OP_NONE;
    if (i + 1 == ptrs.size()) {
      d.flag = flag;
      d.flag_value = flag_value;
      d.flag2 = flag2;
      d.flag2_value = flag2_value;
    }
    int rc = eux_xfer_launch(&d, counter, 0, st);
    if (rc != 0) return rc;
    ++stats_.kernel_launches;
  }
  return 0;
}

void Worker::update_interest(Endpoint*) {}

}  // namespace eux::ucxx::transport
