// The transport against a peer that does not play by the rules: a raw TCP socket that speaks the
// frame format by hand. Everything here is host-side; no GPU is touched.
//   * frames that claim absurd sizes fail the endpoint instead of growing buffers;
//   * device regions announced by a peer that never proved it runs on this host are ignored, even
//     when the descriptor carries this process's own pid and a made-up address (the payload then
//     takes the staged host protocol);
//   * a DATA frame shorter than the posted receive ends it with MESSAGE_TRUNCATED;
//   * import_region() uses a raw address only on the caller's say-so and only after the driver
//     confirmed the range.
#include <arpa/inet.h>
#include <sys/socket.h>
#include <unistd.h>

#include <chrono>
#include <sys/stat.h>
#include <sys/un.h>
#include <cstdlib>
#include <cstring>
#include <thread>

#include "check.hpp"
#include "eux/ucxx/cuda/ucx_cuda_memory_manager.hpp"
#include "eux/ucxx/transport.hpp"

using namespace eux::ucxx;
namespace tr = eux::ucxx::transport;

namespace {

struct RawPeer {
  int fd = -1;
  explicit RawPeer(uint16_t port) {
    fd = ::socket(AF_INET, SOCK_STREAM, 0);
    sockaddr_in in{};
    in.sin_family = AF_INET;
    in.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
    in.sin_port = htons(port);
    CHECK(::connect(fd, reinterpret_cast<sockaddr*>(&in), sizeof(in)) == 0);
  }
  ~RawPeer() {
    if (fd >= 0) ::close(fd);
  }
  void send_all(const void* p, size_t n) {
    const char* c = static_cast<const char*>(p);
    while (n) {
      ssize_t w = ::send(fd, c, n, MSG_NOSIGNAL);
      if (w <= 0) return;  // the worker may already have closed the socket on us
      c += w;
      n -= size_t(w);
    }
  }
  // HELLO without a shared-memory offer, presenting `pid` and `uid` as its own
  void hello(uint32_t pid, uint64_t uid) {
    tr::WorkerAddress a;
    a.pid = pid;
    a.uid = uid;
    a.device = 0;
    std::strncpy(a.name, "raw_peer", sizeof(a.name) - 1);
    auto addr = a.serialize();
    tr::FrameHeader fh;
    fh.type = tr::kHello;
    fh.header_len = uint32_t(8 + addr.size());
    uint64_t client_id = 7;
    send_all(&fh, sizeof(fh));
    send_all(&client_id, 8);
    send_all(addr.data(), addr.size());
  }
  // reads frames until one of `type` arrives (or ~2 s pass); returns its header
  bool wait_frame(uint8_t type, tr::FrameHeader* out) {
    timeval tv{0, 100000};
    setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    for (int tries = 0; tries < 40; ++tries) {
      tr::FrameHeader fh;
      size_t got = 0;
      while (got < sizeof(fh)) {
        ssize_t r = ::recv(fd, reinterpret_cast<char*>(&fh) + got, sizeof(fh) - got, 0);
        if (r <= 0) break;
        got += size_t(r);
      }
      if (got < sizeof(fh)) continue;
      std::vector<char> body(fh.header_len);
      size_t b = 0;
      while (b < body.size()) {
        ssize_t r = ::recv(fd, body.data() + b, body.size() - b, 0);
        if (r <= 0) break;
        b += size_t(r);
      }
      if (fh.type == type) {
        *out = fh;
        return true;
      }
    }
    return false;
  }
};

template <class Pred>
bool spin(tr::Worker& w, Pred done, int ms = 3000) {
  auto end = std::chrono::steady_clock::now() + std::chrono::milliseconds(ms);
  while (std::chrono::steady_clock::now() < end) {
    w.progress();
    if (done()) return true;
    std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
  return false;
}

struct Harness {
  DefaultUcxMemoryResourceManager mr;
  tr::Worker w;
  tr::Endpoint* ep = nullptr;
  int ep_error = 0;
  std::vector<tr::AmArrival> arrivals;
  Harness() : w(mr, [] {
    tr::WorkerOptions o;
    o.name = "victim";
    return o;
  }()) {
    w.on_auto_accept = [this](tr::Endpoint* e) { ep = e; };
    w.on_ep_error = [this](tr::Endpoint*, int st) { ep_error = st; };
    w.on_am = [this](tr::AmArrival&& a) { arrivals.push_back(std::move(a)); };
  }
  void free_arrivals() {
    for (auto& a : arrivals) {
      if (a.header) mr.deallocate(ucx_memory_type::HOST, a.header, a.header_len);
      if (a.data) mr.deallocate(ucx_memory_type::HOST, a.data, a.data_len);
    }
    arrivals.clear();
  }
};

}  // namespace

EUX_TEST(oversized_header_fails_the_endpoint) {
  Harness h;
  RawPeer peer(h.w.address().port);
  peer.hello(1, 1);
  CHECK(spin(h.w, [&] { return h.ep != nullptr; }));
  tr::FrameHeader fh;
  fh.type = tr::kAmEager;
  fh.header_len = 0x7fffffffu;  // 2 GiB of "header"
  fh.msg_id = 1;
  peer.send_all(&fh, sizeof(fh));
  CHECK(spin(h.w, [&] { return h.ep_error != 0; }));
  CHECK_EQ(h.w.stats().frames_refused, uint64_t(1));
  CHECK(h.arrivals.empty());
}

EUX_TEST(oversized_inline_payload_and_segment_count_are_refused) {
  {
    Harness h;
    RawPeer peer(h.w.address().port);
    peer.hello(1, 1);
    CHECK(spin(h.w, [&] { return h.ep != nullptr; }));
    tr::FrameHeader fh;
    fh.type = tr::kAmEager;
    fh.header_len = 8;
    fh.payload_len = uint64_t(1) << 60;  // an "inline" exabyte
    peer.send_all(&fh, sizeof(fh));
    CHECK(spin(h.w, [&] { return h.ep_error != 0; }));
    CHECK_EQ(h.w.stats().frames_refused, uint64_t(1));
  }
  {
    Harness h;
    RawPeer peer(h.w.address().port);
    peer.hello(1, 1);
    CHECK(spin(h.w, [&] { return h.ep != nullptr; }));
    tr::FrameHeader fh;
    fh.type = tr::kAmRts;
    fh.header_len = 8;
    fh.seg_count = 0x40000000u;  // times 104 bytes of descriptors each
    fh.flags = tr::kFlagDeviceRegions;
    fh.payload_len = 64;
    peer.send_all(&fh, sizeof(fh));
    CHECK(spin(h.w, [&] { return h.ep_error != 0; }));
    CHECK_EQ(h.w.stats().frames_refused, uint64_t(1));
  }
}

EUX_TEST(rts_whose_segments_do_not_add_up_is_refused) {
  Harness h;
  RawPeer peer(h.w.address().port);
  peer.hello(1, 1);
  CHECK(spin(h.w, [&] { return h.ep != nullptr; }));
  tr::FrameHeader fh;
  fh.type = tr::kAmRts;
  fh.header_len = 8;
  fh.seg_count = 2;
  fh.payload_len = 4096;
  fh.msg_id = 1;
  uint64_t hdr = 0, sizes[2] = {100, 200};
  peer.send_all(&fh, sizeof(fh));
  peer.send_all(&hdr, 8);
  peer.send_all(sizes, sizeof(sizes));
  CHECK(spin(h.w, [&] { return h.ep_error != 0; }));
  CHECK(h.arrivals.empty());
}

// The peer claims this process's pid (two containers often share one) and a live-looking address,
// but it never mapped a shared-memory channel and its uid is nobody's here.
EUX_TEST(forged_device_regions_are_ignored_and_the_payload_is_staged) {
  Harness h;
  RawPeer peer(h.w.address().port);
  peer.hello(uint32_t(getpid()), 0x1234567890abcdefull);
  CHECK(spin(h.w, [&] { return h.ep != nullptr; }));
  constexpr size_t kLen = 4096;
  tr::FrameHeader fh;
  fh.type = tr::kAmRts;
  fh.flags = tr::kFlagDeviceRegions;
  fh.header_len = 8;
  fh.seg_count = 1;
  fh.payload_len = kLen;
  fh.msg_id = 5;
  fh.mem_type = uint32_t(ucx_memory_type::CUDA);
  uint64_t hdr = 42, size = kLen;
  PeerRegionDesc d;
  d.pid = uint32_t(getpid());
  d.device = 0;
  d.base = 0x7f00dead0000ull;  // means nothing in this process
  d.offset = 0;
  d.length = kLen;
  d.exportable = 1;
  std::memset(d.handle, 0xab, sizeof(d.handle));
  peer.send_all(&fh, sizeof(fh));
  peer.send_all(&hdr, 8);
  peer.send_all(&size, 8);
  peer.send_all(&d, sizeof(d));
  CHECK(spin(h.w, [&] { return !h.arrivals.empty(); }));
  CHECK(h.arrivals[0].rndv);
  CHECK_EQ(h.w.stats().regions_ignored, uint64_t(1));
  // the receive is posted; with no regions left the worker asks for the bytes through the host protocol
  std::vector<char> dst(kLen, 0);
  ucx_buffer_t seg{dst.data(), dst.size()};
  int result = 1;
  int st = h.w.rndv_recv(h.ep, 5, &seg, 1, ucx_memory_type::HOST, [&](int s) { result = s; });
  CHECK_EQ(st, int(UCS_INPROGRESS));
  tr::FrameHeader cts;
  std::thread pump([&] { spin(h.w, [&] { return result != 1; }, 4000); });
  CHECK(peer.wait_frame(tr::kRndvCts, &cts));
  CHECK_EQ(cts.msg_id, uint64_t(5));
  CHECK(cts.flags & tr::kFlagStage);
  std::vector<char> payload(kLen);
  for (size_t i = 0; i < kLen; ++i) payload[i] = char(i * 7);
  tr::FrameHeader data;
  data.type = tr::kRndvData;
  data.msg_id = 5;
  data.payload_len = kLen;
  peer.send_all(&data, sizeof(data));
  peer.send_all(payload.data(), payload.size());
  pump.join();
  CHECK_EQ(result, int(UCS_OK));
  CHECK(std::memcmp(dst.data(), payload.data(), kLen) == 0);
  CHECK_EQ(h.w.stats().device_pulls, uint64_t(0));
  h.free_arrivals();
}

EUX_TEST(layout_of_a_strided_payload_is_checked_before_a_kernel_sees_it) {
  UcxSendAttr a;
  CHECK(a.layout_valid());  // dense
  a.ndim = 2;
  a.elem_size = 4;
  a.shape[0] = 70, a.shape[1] = 300;
  a.stride[0] = 1, a.stride[1] = 70;   // a transposed 300 x 70 matrix
  a.span_bytes = 300 * 70 * 4;
  a.dense_bytes = 300 * 70 * 4;
  CHECK(a.layout_valid());
  CHECK_EQ(a.elements(), uint64_t(21000));
  auto bad = [&](auto&& change) {
    UcxSendAttr b = a;
    change(b);
    return !b.layout_valid();
  };
  CHECK(bad([](UcxSendAttr& b) { b.span_bytes -= 4; }));          // the last element lies outside the span
  CHECK(bad([](UcxSendAttr& b) { b.stride[1] = 71; }));           // so does it here
  CHECK(bad([](UcxSendAttr& b) { b.stride[0] = -1; }));           // the address of the buffer would not be that of element 0
  CHECK(bad([](UcxSendAttr& b) { b.shape[0] = 0; }));
  CHECK(bad([](UcxSendAttr& b) { b.elem_size = 3; }));
  CHECK(bad([](UcxSendAttr& b) { b.ndim = 9; }));
  CHECK(bad([](UcxSendAttr& b) { b.dense_bytes += 4; }));         // the message would be longer than the elements
  CHECK(bad([](UcxSendAttr& b) { b.shape[1] = int64_t(1) << 50; b.stride[1] = 0; }));  // more elements than any message has
  // converted on the way: fp32 in memory, bf16 on the wire; the message is half the size of the elements
  UcxSendAttr c = a;
  c.src_dtype = 1;
  c.dst_dtype = 3;
  CHECK(!c.layout_valid());           // ... so the dense size of the fp32 elements is wrong for it
  c.dense_bytes = 300 * 70 * 2;
  CHECK(c.layout_valid() && c.casts());
  c.elem_size = 2;                    // the source's element size must be that of its type
  CHECK(!c.layout_valid());
  c.elem_size = 4;
  c.dst_dtype = 9;                    // a type the kernel does not know
  CHECK(!c.layout_valid());
  // a stride of zero (an expanded tensor) is fine: the span is smaller than the message
  UcxSendAttr e;
  e.ndim = 2;
  e.elem_size = 8;
  e.shape[0] = 50, e.shape[1] = 100;
  e.stride[0] = 0, e.stride[1] = 1;
  e.span_bytes = 800;
  e.dense_bytes = 50 * 100 * 8;
  CHECK(e.layout_valid());
}

EUX_TEST(rts_with_a_layout_from_a_peer_not_shown_to_be_local_is_staged) {
  // The frame is taken apart correctly (its length includes the layout), the region and the layout are
  // ignored because the peer never proved that it runs on this host, and the payload takes the host protocol.
  Harness h;
  RawPeer peer(h.w.address().port);
  peer.hello(uint32_t(getpid()), 0x1234567890abcdefull);
  CHECK(spin(h.w, [&] { return h.ep != nullptr; }));
  tr::FrameHeader fh;
  fh.type = tr::kAmRts;
  fh.flags = tr::kFlagDeviceRegions | tr::kFlagLayout;
  fh.header_len = 8;
  fh.seg_count = 1;
  fh.status = 1;
  fh.payload_len = 4096;
  fh.msg_id = 9;
  fh.mem_type = uint32_t(ucx_memory_type::CUDA);
  uint64_t hdr = 1, size = 4096;
  PeerRegionDesc d;
  d.length = 8192;
  tr::WireLayout l;
  l.ndim = 1;
  l.elem_size = 4;
  l.shape[0] = 1024;
  l.stride[0] = 2;
  l.span_bytes = 8192;
  peer.send_all(&fh, sizeof(fh));
  peer.send_all(&hdr, 8);
  peer.send_all(&size, 8);
  peer.send_all(&d, sizeof(d));
  peer.send_all(&l, sizeof(l));
  // a second, ordinary frame right behind it shows that the first one's length was counted right
  tr::FrameHeader eager;
  eager.type = tr::kAmEager;
  eager.header_len = 8;
  eager.payload_len = 0;
  eager.msg_id = 10;
  peer.send_all(&eager, sizeof(eager));
  peer.send_all(&hdr, 8);
  CHECK(spin(h.w, [&] { return h.arrivals.size() == 2; }));
  CHECK(h.arrivals[0].rndv && !h.arrivals[1].rndv);
  CHECK_EQ(h.w.stats().regions_ignored, uint64_t(1));
  CHECK_EQ(h.w.stats().frames_refused, uint64_t(0));
  h.free_arrivals();
}

EUX_TEST(rts_that_claims_too_many_regions_is_refused) {
  Harness h;
  RawPeer peer(h.w.address().port);
  peer.hello(uint32_t(getpid()), 0x1234567890abcdefull);
  CHECK(spin(h.w, [&] { return h.ep != nullptr; }));
  tr::FrameHeader fh;
  fh.type = tr::kAmRts;
  fh.flags = tr::kFlagDeviceRegions;
  fh.header_len = 8;
  fh.seg_count = 1;
  fh.status = 1 << 20;   // a million descriptors: 100 MB that this worker would have to buffer
  fh.payload_len = 4096;
  fh.msg_id = 1;
  peer.send_all(&fh, sizeof(fh));
  CHECK(spin(h.w, [&] { return h.w.stats().frames_refused == 1; }));
}

EUX_TEST(descriptor_channel_socket_is_private_and_ignores_strangers) {
  // A worker that manages device memory listens on a Unix socket over which file descriptors of device
  // allocations travel. The socket is this user's only; a connection that names no endpoint of the worker is
  // closed, and the worker goes on. (No GPU is needed: nothing is allocated.)
  ::setenv("EUX_SHM", "1", 1);  // the socket belongs to the shared-memory control plane; a run of the tests with it off gets it here
  UcxCudaMemoryResourceManager::Options mo;
  mo.device = 0;
  UcxCudaMemoryResourceManager mr(mo);
  tr::WorkerOptions o;
  o.name = "fd_owner";
  tr::Worker w(mr, o);
  char path[64];
  std::snprintf(path, sizeof(path), "/dev/shm/eux-fd-%016llx", static_cast<unsigned long long>(w.address().uid));
  struct stat st{};
  CHECK(::stat(path, &st) == 0);
  CHECK(S_ISSOCK(st.st_mode));
  CHECK_EQ(int(st.st_mode & 0777), 0600);
  int fd = ::socket(AF_UNIX, SOCK_SEQPACKET, 0);
  sockaddr_un un{};
  un.sun_family = AF_UNIX;
  std::strncpy(un.sun_path, path, sizeof(un.sun_path) - 1);
  CHECK(::connect(fd, reinterpret_cast<sockaddr*>(&un), sizeof(un)) == 0);
  struct {
    uint32_t magic = 0x44465845u, kind = 0;
    uint64_t a = 0x1122334455667788ull, b = 0;  // a worker id that this worker has no endpoint for
  } hello;
  CHECK(::send(fd, &hello, sizeof(hello), MSG_NOSIGNAL) == ssize_t(sizeof(hello)));
  char buf[8];
  ssize_t n = -1;
  for (int i = 0; i < 2000; ++i) {
    w.progress();
    n = ::recv(fd, buf, sizeof(buf), MSG_DONTWAIT);
    if (n == 0) break;  // closed by the worker
    std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
  CHECK_EQ(n, ssize_t(0));
  ::close(fd);
  CHECK_EQ(w.stats().vmm_fds_recv, uint64_t(0));
  {
    tr::Worker gone(mr, o);
    std::snprintf(path, sizeof(path), "/dev/shm/eux-fd-%016llx", static_cast<unsigned long long>(gone.address().uid));
    CHECK(::stat(path, &st) == 0);
  }
  CHECK(::stat(path, &st) != 0);  // the socket's name goes with its worker
}

EUX_TEST(short_data_frame_ends_the_receive_as_truncated) {
  Harness h;
  RawPeer peer(h.w.address().port);
  peer.hello(1, 1);
  CHECK(spin(h.w, [&] { return h.ep != nullptr; }));
  tr::FrameHeader fh;
  fh.type = tr::kAmRts;
  fh.header_len = 8;
  fh.seg_count = 1;
  fh.payload_len = 1024;
  fh.msg_id = 9;
  uint64_t hdr = 1, size = 1024;
  peer.send_all(&fh, sizeof(fh));
  peer.send_all(&hdr, 8);
  peer.send_all(&size, 8);
  CHECK(spin(h.w, [&] { return !h.arrivals.empty(); }));
  std::vector<char> dst(1024, 0);
  ucx_buffer_t seg{dst.data(), dst.size()};
  int result = 1;
  CHECK_EQ(h.w.rndv_recv(h.ep, 9, &seg, 1, ucx_memory_type::HOST, [&](int s) { result = s; }), int(UCS_INPROGRESS));
  tr::FrameHeader data;
  data.type = tr::kRndvData;
  data.msg_id = 9;
  data.payload_len = 100;  // 924 bytes short
  std::vector<char> some(100, 'x');
  peer.send_all(&data, sizeof(data));
  peer.send_all(some.data(), some.size());
  CHECK(spin(h.w, [&] { return result != 1; }));
  CHECK_EQ(result, int(UCS_ERR_MESSAGE_TRUNCATED));
  CHECK_EQ(h.w.stats().truncated, uint64_t(1));
  h.free_arrivals();
}

EUX_TEST(import_region_never_trusts_an_address_from_the_wire) {
  UcxCudaMemoryResourceManager::Options o;
  o.device = 0;
  UcxCudaMemoryResourceManager mr(o);
  PeerRegionDesc d;
  d.pid = uint32_t(getpid());
  d.device = 0;
  d.base = 0x7f00dead0000ull;
  d.offset = 0;
  d.length = 4096;
  d.exportable = 0;
  CHECK(mr.import_region(d, false) == nullptr);  // same pid, but nobody vouches for it, and no handle to open
  d.exportable = 1;
  std::memset(d.handle, 0x5a, sizeof(d.handle));
  CHECK(mr.import_region(d, false) == nullptr);  // a made-up handle does not open
  CHECK(mr.import_region(d, true) == nullptr);   // vouched for, but the driver knows no allocation there
  d.offset = ~uint64_t(0) - 10;
  CHECK(mr.import_region(d, true) == nullptr);   // offset + length wraps
}

EUX_TEST_MAIN()
