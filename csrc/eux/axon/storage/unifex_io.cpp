#include "eux/axon/storage/unifex_io.hpp"

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <system_error>

namespace eux::axon::storage {

FileIoContext& FileIoContext::Default() {
  static FileIoContext ctx;
  return ctx;
}

AsyncFile::AsyncFile(const std::string& path, Mode mode) {
  fd_ = ::open(path.c_str(), mode == Mode::kRead ? (O_RDONLY | O_CLOEXEC) : (O_WRONLY | O_CREAT | O_TRUNC | O_CLOEXEC), 0644);
  if (fd_ < 0) throw std::system_error(errno, std::generic_category(), "open " + path);
}
AsyncFile::~AsyncFile() {
  if (fd_ >= 0) ::close(fd_);
}
uint64_t AsyncFile::size() const {
  struct stat st{};
  return ::fstat(fd_, &st) == 0 ? static_cast<uint64_t>(st.st_size) : 0;
}

exec::any_sender_of<size_t> AsyncFile::async_write_some_at(uint64_t offset, const void* data, size_t n) {
  int fd = fd_;
  return exec::on(FileIoContext::Default().get_scheduler(), exec::just_from([fd, offset, data, n]() -> size_t {
                    size_t done = 0;
                    while (done < n) {
                      ssize_t w = ::pwrite(fd, static_cast<const char*>(data) + done, n - done, static_cast<off_t>(offset + done));
                      if (w < 0) {
                        if (errno == EINTR) continue;
                        throw std::system_error(errno, std::generic_category(), "pwrite");
                      }
                      done += static_cast<size_t>(w);
                    }
                    return done;
                  }));
}
exec::any_sender_of<size_t> AsyncFile::async_read_some_at(uint64_t offset, void* data, size_t n) {
  int fd = fd_;
  return exec::on(FileIoContext::Default().get_scheduler(), exec::just_from([fd, offset, data, n]() -> size_t {
                    size_t done = 0;
                    while (done < n) {
                      ssize_t r = ::pread(fd, static_cast<char*>(data) + done, n - done, static_cast<off_t>(offset + done));
                      if (r < 0) {
                        if (errno == EINTR) continue;
                        throw std::system_error(errno, std::generic_category(), "pread");
                      }
                      if (r == 0) break;
                      done += static_cast<size_t>(r);
                    }
                    return done;
                  }));
}

// ---- output ----
UnifexOutputStream::UnifexOutputStream(const std::string& path) : file_(path, AsyncFile::Mode::kWriteTruncate) {
  buf_[0].reserve(kBufferSize);
  buf_[1].reserve(kBufferSize);
}
UnifexOutputStream::~UnifexOutputStream() {
  try {
    flush();
  } catch (...) {
  }
  exec::sync_wait(scope_.join());
}
void UnifexOutputStream::wait_inflight() {
  if (!inflight_) return;
  auto s = std::move(*inflight_);
  inflight_.reset();
  auto n = exec::sync_wait(std::move(s));
  if (!n || *n != inflight_len_) throw std::runtime_error("short write to the checkpoint file");
}
void UnifexOutputStream::submit_current() {
  if (buf_[cur_].empty()) return;
  wait_inflight();  // at most one write in flight; the other buffer is free again after this
  inflight_len_ = buf_[cur_].size();
  inflight_.emplace(scope_.spawn_future(file_.async_write_some_at(file_off_, buf_[cur_].data(), inflight_len_)));
  file_off_ += inflight_len_;
  cur_ ^= 1;
  buf_[cur_].clear();
}
void UnifexOutputStream::write(const void* data, size_t n) {
  const uint8_t* p = static_cast<const uint8_t*>(data);
  total_ += n;
  while (n) {
    size_t room = kBufferSize - buf_[cur_].size();
    size_t take = n < room ? n : room;
    buf_[cur_].insert(buf_[cur_].end(), p, p + take);
    p += take;
    n -= take;
    if (buf_[cur_].size() == kBufferSize) submit_current();
  }
}
void UnifexOutputStream::flush() {
  submit_current();
  wait_inflight();
}

// ---- input ----
UnifexInputStream::UnifexInputStream(const std::string& path) : file_(path, AsyncFile::Mode::kRead) {
  buf_[0].resize(kBufferSize);
  buf_[1].resize(kBufferSize);
  start_prefetch();  // fills buf_[cur_ ^ 1]
}
UnifexInputStream::~UnifexInputStream() {
  if (inflight_) {
    try {
      exec::sync_wait(std::move(*inflight_));
    } catch (...) {
    }
  }
  exec::sync_wait(scope_.join());
}
void UnifexInputStream::start_prefetch() {
  if (eof_) return;
  inflight_.emplace(scope_.spawn_future(file_.async_read_some_at(file_off_, buf_[cur_ ^ 1].data(), kBufferSize)));
}
bool UnifexInputStream::advance() {
  if (!inflight_) return false;
  auto s = std::move(*inflight_);
  inflight_.reset();
  auto n = exec::sync_wait(std::move(s));
  size_t got = n ? *n : 0;
  cur_ ^= 1;
  len_[cur_] = got;
  pos_ = 0;
  file_off_ += got;
  if (got < kBufferSize) eof_ = true;
  start_prefetch();  // read ahead while the caller consumes this buffer
  return got > 0;
}
size_t UnifexInputStream::read(void* data, size_t n) {
  uint8_t* out = static_cast<uint8_t*>(data);
  size_t done = 0;
  while (done < n) {
    if (pos_ == len_[cur_] && !advance()) break;
    size_t take = std::min(n - done, len_[cur_] - pos_);
    std::memcpy(out + done, buf_[cur_].data() + pos_, take);
    pos_ += take;
    done += take;
  }
  return done;
}
std::vector<uint8_t> UnifexInputStream::read_all() {
  std::vector<uint8_t> out;
  uint8_t tmp[65536];
  while (size_t n = read(tmp, sizeof(tmp))) out.insert(out.end(), tmp, tmp + n);
  return out;
}

}  // namespace eux::axon::storage
