// Asynchronous file streams for the checkpoint files: positional reads/writes
// run as senders on an IO context, and the streams double-buffer on top of
// them (one buffer is filled / consumed while the other is in flight). The
// reference does the same with libunifex's io_uring context and two 8 KiB
// buffers (axon/src/storage/unifex_io.cpp:104-140, 208-250); here the IO context
// is a thread that issues pread/pwrite, and the buffers are 256 KiB.
#pragma once

#include <cstdint>
#include <memory>
#include <optional>
#include <string>
#include <vector>

#include "eux/exec/async_scope.hpp"
#include "eux/exec/contexts.hpp"

namespace eux::axon::storage {

// One thread that performs blocking file calls on behalf of senders.
class FileIoContext {
 public:
  static FileIoContext& Default();
  exec::static_thread_pool::scheduler get_scheduler() { return pool_.get_scheduler(); }

 private:
  FileIoContext() : pool_(1) {}
  exec::static_thread_pool pool_;
};

class AsyncFile {
 public:
  enum class Mode { kRead, kWriteTruncate };
  AsyncFile(const std::string& path, Mode mode);
  ~AsyncFile();
  AsyncFile(const AsyncFile&) = delete;
  int fd() const { return fd_; }
  uint64_t size() const;
  // senders of the number of bytes transferred; errors are std::system_error
  exec::any_sender_of<size_t> async_write_some_at(uint64_t offset, const void* data, size_t n);
  exec::any_sender_of<size_t> async_read_some_at(uint64_t offset, void* data, size_t n);

 private:
  int fd_ = -1;
};

class UnifexOutputStream {
 public:
  static constexpr size_t kBufferSize = 256 * 1024;
  explicit UnifexOutputStream(const std::string& path);
  ~UnifexOutputStream();
  void write(const void* data, size_t n);
  void flush();  // waits until everything written so far is on its way to the file and done
  uint64_t byte_count() const { return total_; }

 private:
  void submit_current();
  void wait_inflight();
  AsyncFile file_;
  std::vector<uint8_t> buf_[2];
  int cur_ = 0;
  uint64_t file_off_ = 0, total_ = 0;
  exec::async_scope scope_;
  std::optional<exec::any_sender_of<size_t>> inflight_;
  size_t inflight_len_ = 0;
};

class UnifexInputStream {
 public:
  static constexpr size_t kBufferSize = 256 * 1024;
  explicit UnifexInputStream(const std::string& path);
  ~UnifexInputStream();
  // Reads up to n bytes; returns 0 at end of file.
  size_t read(void* data, size_t n);
  std::vector<uint8_t> read_all();

 private:
  void start_prefetch();
  bool advance();  // make the prefetched buffer current; false at EOF
  AsyncFile file_;
  std::vector<uint8_t> buf_[2];
  size_t len_[2] = {0, 0};
  int cur_ = 0;
  size_t pos_ = 0;
  uint64_t file_off_ = 0;
  bool eof_ = false;
  exec::async_scope scope_;
  std::optional<exec::any_sender_of<size_t>> inflight_;
};

}  // namespace eux::axon::storage
