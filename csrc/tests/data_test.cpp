#include <fcntl.h>
#include <sys/stat.h>
#include <sys/mman.h>
// RAII buffers, memory resource, lock-free queue, connection manager (CPU only).
#include <cstring>
#include <thread>

#include "check.hpp"
#include "eux/ucxx/lock_free_queue.hpp"
#include "eux/ucxx/shm_channel.hpp"
#include "eux/ucxx/ucx_context_data.hpp"
#include "eux/ucxx/ucx_status.hpp"

using namespace eux::ucxx;

// counts what is outstanding so leaks and double frees show up
struct TrackingMr : DefaultUcxMemoryResourceManager {
  long live = 0;
  void* allocate(ucx_memory_type_t t, size_t n, size_t a = 8) override {
    ++live;
    return DefaultUcxMemoryResourceManager::allocate(t, n, a);
  }
  void deallocate(ucx_memory_type_t t, void* p, size_t n, size_t a = 8) override {
    if (p) --live;
    DefaultUcxMemoryResourceManager::deallocate(t, p, n, a);
  }
};

EUX_TEST(buffer_ownership_and_moves) {
  TrackingMr mr;
  {
    UcxBuffer a(mr, ucx_memory_type::HOST, 128);
    CHECK(a.data() != nullptr && a.size() == 128 && a.own_buffer());
    UcxBuffer b(std::move(a));
    CHECK(a.data() == nullptr && !a.own_buffer());
    CHECK(b.size() == 128);
    UcxBuffer c(mr, ucx_memory_type::HOST, 16);
    c = std::move(b);
    CHECK_EQ(mr.live, 1);
  }
  CHECK_EQ(mr.live, 0);
  int released = 0;
  char local[8];
  {
    UcxBuffer v(mr, ucx_memory_type::HOST, local, 8, nullptr, true, [&](void* p) { released += (p == local); });
    UcxBuffer w(std::move(v));
  }
  CHECK_EQ(released, 1);  // exactly once, by the last owner
  {
    UcxBuffer view(mr, ucx_memory_type::HOST, local, 8, nullptr, false);
  }
  CHECK_EQ(mr.live, 0);
}

EUX_TEST(to_buffer_vec_is_zero_copy_and_checked) {
  TrackingMr mr;
  {
    UcxBuffer big(mr, ucx_memory_type::HOST, 100);
    char* base = static_cast<char*>(big.data());
    for (int i = 0; i < 100; ++i) base[i] = char(i);
    UcxBufferVec v = std::move(big).to_buffer_vec({10, 20, 70});
    CHECK(v.has_backing_buffer() && v.size() == 3);
    CHECK(v[0].data == base && v[1].data == base + 10 && v[2].data == base + 30);
    CHECK_EQ(v.total_size(), 100u);
    CHECK_THROWS(std::move(v).ExtractBuffers());
    UcxBufferVec moved(std::move(v));
    CHECK_EQ(static_cast<char*>(moved[2].data)[0], char(30));
  }
  CHECK_EQ(mr.live, 0);
  UcxBuffer small(mr, ucx_memory_type::HOST, 10);
  CHECK_THROWS(std::move(small).to_buffer_vec({8, 8}));
}

EUX_TEST(buffer_vec_extract_and_am_types) {
  TrackingMr mr;
  {
    UcxBufferVec v(mr, ucx_memory_type::HOST, std::vector<size_t>{4, 8, 16});
    CHECK_EQ(mr.live, 3);
    auto bufs = std::move(v).ExtractBuffers();
    CHECK_EQ(bufs.size(), 3u);
    CHECK(bufs[2].size() == 16 && bufs[2].own_buffer());
    UcxBufferVec again(std::move(bufs));
    CHECK_EQ(again.size(), 3u);
  }
  CHECK_EQ(mr.live, 0);
  {
    UcxAmData d(mr, 16, 64, ucx_memory_type::HOST);
    CHECK(d.get()->header.size == 16 && d.get()->buffer.size == 64);
    UcxHeader h = d.move_header();
    UcxBuffer b = d.move_buffer();
    CHECK(h.size() == 16 && b.size() == 64 && !d.own_buffer() && !d.owns_header());
    UcxAmData re(mr, std::move(h), std::move(b));
    CHECK(re.get()->buffer.size == 64);
    UcxAmIovec io(mr, 8, {32, 32}, ucx_memory_type::HOST);
    CHECK_EQ(io.get()->buffer_count, 2u);
    UcxAmIovec io2(std::move(io));
    auto vec = io2.move_buffers();
    CHECK_EQ(vec.size(), 2u);
  }
  CHECK_EQ(mr.live, 0);
}

EUX_TEST(memory_resource_tables) {
  DefaultUcxMemoryResourceManager mr;
  CHECK(mr.get_memory_resource(ucx_memory_type::HOST) != nullptr);
  CHECK(mr.get_memory_resource(ucx_memory_type::CUDA) == nullptr);
  CHECK_THROWS(mr.allocate(ucx_memory_type::CUDA, 16));
  char a[4] = {1, 2, 3, 4}, b[4] = {};
  mr.memcpy(ucx_memory_type::HOST, b, ucx_memory_type::HOST, a, 4);
  CHECK_EQ(b[3], 4);
  CHECK_THROWS(mr.memcpy(ucx_memory_type::CUDA, b, ucx_memory_type::HOST, a, 4));
  int calls = 0;
  mr.register_memcpy_fn(ucx_memory_type::CUDA, ucx_memory_type::HOST, [&](void* d, const void* s, size_t n) { ++calls; return std::memcpy(d, s, n); });
  mr.memcpy(ucx_memory_type::CUDA, b, ucx_memory_type::HOST, a, 4);
  CHECK_EQ(calls, 1);
}

EUX_TEST(status_category) {
  std::error_code ok = make_error_code(UCS_OK), prog = make_error_code(UCS_INPROGRESS), to = make_error_code(UCS_ERR_TIMED_OUT);
  CHECK(std::string(ok.category().name()) == "UCX");
  CHECK(ok == std::error_condition(0, std::generic_category()));
  CHECK(prog == std::error_condition(0, std::generic_category()));
  CHECK(to == std::errc::timed_out);
  CHECK(to.message() == "Operation timed out");
}

EUX_TEST(lock_free_queue_mpmc) {
  LockFreeQueue<int> q;
  CHECK(!q.pop().has_value());
  const int P = 4, N = 20000;
  std::atomic<long> sum{0};
  std::atomic<int> popped{0};
  std::vector<std::thread> th;
  for (int p = 0; p < P; ++p) th.emplace_back([&, p] { for (int i = 0; i < N; ++i) q.push(p * N + i); });
  for (int c = 0; c < P; ++c)
    th.emplace_back([&] {
      while (popped.load() < P * N) {
        if (auto v = q.pop()) {
          sum += *v;
          popped.fetch_add(1);
        }
      }
    });
  for (auto& t : th) t.join();
  long want = 0;
  for (long i = 0; i < long(P) * N; ++i) want += i;
  CHECK_EQ(sum.load(), want);
  CHECK(q.empty());
}

// The shared-memory byte rings: a producer thread streams 16 MiB of a known sequence through a 2 MiB
// ring in odd-sized pieces while the consumer reads odd-sized pieces; every byte arrives in order,
// in both directions, and a full ring reports EAGAIN instead of overwriting.
// Ring indices that no honest peer produces (more bytes in flight than the ring holds, a head ahead of its tail)
// end as an error of the channel; nothing is copied through them.
EUX_TEST(shm_channel_refuses_impossible_indices) {
  using eux::ucxx::transport::ShmChannel;
  using eux::ucxx::transport::ShmRing;
  const std::string name = "/eux-test-idx-" + std::to_string(getpid());
  auto a = ShmChannel::create(name);
  CHECK(a != nullptr);
  int fd = ::shm_open(name.c_str(), O_RDWR, 0600);  // a second mapping of the same segment, to play the hostile peer with
  CHECK(fd >= 0);
  struct stat st{};
  CHECK(::fstat(fd, &st) == 0);
  char* raw = static_cast<char*>(::mmap(nullptr, size_t(st.st_size), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0));
  ::close(fd);
  CHECK(raw != MAP_FAILED);
  auto b = ShmChannel::open(name);
  CHECK(b != nullptr);
  auto* ring0 = reinterpret_cast<ShmRing*>(raw + 64);  // creator -> opener, right behind the 64-byte header
  char buf[16] = {0};
  CHECK_EQ(a->write("abc", 3), ssize_t(3));
  CHECK_EQ(b->read(buf, sizeof(buf)), ssize_t(3));
  const uint64_t at = ring0->tail.load();
  ring0->tail.store(at + ShmChannel::kRingBytes + 1);
  errno = 0;
  CHECK(b->read(buf, sizeof(buf)) == -1 && errno == EIO);
  errno = 0;
  CHECK(a->write(buf, sizeof(buf)) == -1 && errno == EIO);
  ring0->tail.store(at);
  ring0->head.store(at + 5);
  errno = 0;
  CHECK(b->read(buf, sizeof(buf)) == -1 && errno == EIO);
  errno = 0;
  CHECK(a->write(buf, sizeof(buf)) == -1 && errno == EIO);
  ring0->head.store(at);
  CHECK_EQ(a->write("z", 1), ssize_t(1));
  CHECK(b->read(buf, sizeof(buf)) == 1 && buf[0] == 'z');
  ::munmap(raw, size_t(st.st_size));
}

EUX_TEST(shm_channel_streams_bytes_both_ways) {
  using eux::ucxx::transport::ShmChannel;
  const std::string name = "/eux-test-" + std::to_string(getpid());
  auto a = ShmChannel::create(name);
  CHECK(a != nullptr);
  auto b = ShmChannel::open(name);
  CHECK(b != nullptr);
  CHECK(ShmChannel::open(name) == nullptr);  // the name is gone once the peer has mapped it
  // full ring
  std::vector<char> big(ShmChannel::kRingBytes + 100, 'x');
  CHECK_EQ(a->write(big.data(), big.size()), ssize_t(ShmChannel::kRingBytes));
  errno = 0;
  CHECK(a->write(big.data(), 1) == -1 && errno == EAGAIN);
  std::vector<char> sink(ShmChannel::kRingBytes);
  CHECK_EQ(b->read(sink.data(), sink.size()), ssize_t(ShmChannel::kRingBytes));
  CHECK(!b->readable());
  auto stream = [](ShmChannel* tx, ShmChannel* rx) {
    const size_t total = size_t(16) << 20;
    std::thread producer([&] {
      size_t sent = 0, piece = 1;
      std::vector<unsigned char> buf(70001);
      while (sent < total) {
        size_t n = std::min(total - sent, piece % buf.size() + 1);
        for (size_t i = 0; i < n; ++i) buf[i] = static_cast<unsigned char>((sent + i) * 2654435761u >> 24);
        size_t off = 0;
        while (off < n) {
          ssize_t w = tx->write(buf.data() + off, n - off);
          if (w > 0) off += size_t(w);
          else std::this_thread::yield();
        }
        sent += n;
        piece = piece * 7 + 13;
      }
    });
    size_t got = 0, piece = 3;
    bool ok = true;
    std::vector<unsigned char> buf(90001);
    while (got < total) {
      ssize_t r = rx->read(buf.data(), piece % buf.size() + 1);
      if (r <= 0) {
        std::this_thread::yield();
        continue;
      }
      for (ssize_t i = 0; i < r; ++i) ok = ok && buf[i] == static_cast<unsigned char>((got + i) * 2654435761u >> 24);
      got += size_t(r);
      piece = piece * 5 + 11;
    }
    producer.join();
    return ok;
  };
  CHECK(stream(a.get(), b.get()));
  CHECK(stream(b.get(), a.get()));
}

EUX_TEST_MAIN()
