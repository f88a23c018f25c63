// Minimal Avro: binary encoding of the primitive types (zig-zag varints, bytes,
// strings, arrays as counted blocks, union branch indices) and the object
// container file format (magic "Obj\1", metadata map with the schema, 16-byte
// sync marker, blocks of {count, byte size, records, sync}), codec "null".
// It stands in for avro-cpp, which the reference links
// (axon/src/storage/avro_serialization.cpp, async_io.hpp:205-255).
#pragma once

#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <string_view>
#include <vector>

namespace eux::axon::storage::avro {

class Encoder {
 public:
  explicit Encoder(std::vector<uint8_t>& out) : out_(out) {}
  void put_long(int64_t v) {
    uint64_t z = (static_cast<uint64_t>(v) << 1) ^ static_cast<uint64_t>(v >> 63);
    while (z >= 0x80) {
      out_.push_back(static_cast<uint8_t>(z) | 0x80);
      z >>= 7;
    }
    out_.push_back(static_cast<uint8_t>(z));
  }
  void put_int(int32_t v) { put_long(v); }
  void put_bool(bool b) { out_.push_back(b ? 1 : 0); }
  void put_float(float f) { raw(&f, 4); }
  void put_double(double d) { raw(&d, 8); }
  void put_bytes(const void* p, size_t n) {
    put_long(static_cast<int64_t>(n));
    raw(p, n);
  }
  void put_string(std::string_view s) { put_bytes(s.data(), s.size()); }
  void put_union(int branch) { put_long(branch); }
  // arrays: one block with all items, then the terminating empty block
  void array_start(size_t n) {
    if (n) put_long(static_cast<int64_t>(n));
  }
  void array_end() { put_long(0); }
  void raw(const void* p, size_t n) {
    const uint8_t* b = static_cast<const uint8_t*>(p);
    out_.insert(out_.end(), b, b + n);
  }

 private:
  std::vector<uint8_t>& out_;
};

class Decoder {
 public:
  Decoder(const uint8_t* p, size_t n) : p_(p), end_(p + n) {}
  int64_t get_long() {
    uint64_t z = 0;
    int shift = 0;
    for (;;) {
      need(1);
      uint8_t b = *p_++;
      z |= static_cast<uint64_t>(b & 0x7f) << shift;
      if (!(b & 0x80)) break;
      shift += 7;
      if (shift > 63) throw std::runtime_error("avro: varint too long");
    }
    return static_cast<int64_t>(z >> 1) ^ -static_cast<int64_t>(z & 1);
  }
  int32_t get_int() { return static_cast<int32_t>(get_long()); }
  bool get_bool() {
    need(1);
    return *p_++ != 0;
  }
  float get_float() {
    float f;
    raw(&f, 4);
    return f;
  }
  double get_double() {
    double d;
    raw(&d, 8);
    return d;
  }
  std::string get_string() {
    int64_t n = get_long();
    if (n < 0) throw std::runtime_error("avro: negative length");
    need(static_cast<size_t>(n));
    std::string s(reinterpret_cast<const char*>(p_), static_cast<size_t>(n));
    p_ += n;
    return s;
  }
  // returns a view into the input
  std::pair<const uint8_t*, size_t> get_bytes() {
    int64_t n = get_long();
    if (n < 0) throw std::runtime_error("avro: negative length");
    need(static_cast<size_t>(n));
    auto r = std::make_pair(p_, static_cast<size_t>(n));
    p_ += n;
    return r;
  }
  int get_union() { return static_cast<int>(get_long()); }
  // Iterate an array: call next_block() until it returns 0; each call gives the item count of a block.
  size_t next_block() {
    int64_t n = get_long();
    if (n < 0) {  // negative count: a byte size follows
      n = -n;
      (void)get_long();
    }
    return static_cast<size_t>(n);
  }
  void raw(void* dst, size_t n) {
    need(n);
    std::memcpy(dst, p_, n);
    p_ += n;
  }
  bool at_end() const { return p_ == end_; }
  const uint8_t* cursor() const { return p_; }
  void skip(size_t n) {
    need(n);
    p_ += n;
  }

 private:
  void need(size_t n) const {
    if (static_cast<size_t>(end_ - p_) < n) throw std::runtime_error("avro: truncated data");
  }
  const uint8_t* p_;
  const uint8_t* end_;
};

constexpr uint8_t kMagic[4] = {'O', 'b', 'j', 1};

// File header: magic, metadata map, sync marker.
inline void write_container_header(std::vector<uint8_t>& out, std::string_view schema_json, const uint8_t sync[16]) {
  Encoder e(out);
  e.raw(kMagic, 4);
  e.put_long(2);  // two metadata entries
  e.put_string("avro.schema");
  e.put_bytes(schema_json.data(), schema_json.size());
  e.put_string("avro.codec");
  e.put_bytes("null", 4);
  e.put_long(0);
  e.raw(sync, 16);
}
// One data block holding `count` already-encoded records.
inline void write_container_block(std::vector<uint8_t>& out, size_t count, const std::vector<uint8_t>& records, const uint8_t sync[16]) {
  Encoder e(out);
  e.put_long(static_cast<int64_t>(count));
  e.put_long(static_cast<int64_t>(records.size()));
  e.raw(records.data(), records.size());
  e.raw(sync, 16);
}

struct ContainerHeader {
  std::string schema;
  std::string codec;
  uint8_t sync[16];
};
inline ContainerHeader read_container_header(Decoder& d) {
  uint8_t magic[4];
  d.raw(magic, 4);
  if (std::memcmp(magic, kMagic, 4) != 0) throw std::runtime_error("avro: not an object container file");
  ContainerHeader h;
  while (size_t n = d.next_block()) {
    for (size_t i = 0; i < n; ++i) {
      std::string key = d.get_string();
      auto [p, len] = d.get_bytes();
      std::string val(reinterpret_cast<const char*>(p), len);
      if (key == "avro.schema") h.schema = std::move(val);
      else if (key == "avro.codec") h.codec = std::move(val);
    }
  }
  d.raw(h.sync, 16);
  if (!h.codec.empty() && h.codec != "null") throw std::runtime_error("avro: unsupported codec " + h.codec);
  return h;
}

}  // namespace eux::axon::storage::avro
