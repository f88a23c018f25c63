// 128-bit hashing used for function ids and worker keys. The arithmetic is a
// wire contract: a function addressed by name has id = low 32 bits of
// MHash(function_name, worker_name), so both ends must compute the same value
// (reference: axon/include/axon/utils/hash.hpp, axon/src/utils/hash.cpp:28-100,
// axon/python/src/bindings_runtime.cpp:80-86). Block hash: Murmur-style over
// 16-byte words with multiplier 0xc6a4a7935bd1e995 and shift 47; combination:
// a ^ (b * {101, 0x27d4eb2f165667c5} + 0x9e3779b97f4a7c15 + (a << 6) + (a >> 2)).
#pragma once

#include <cstdint>
#include <cstring>
#include <string>
#include <string_view>
#include <type_traits>
#include <vector>

namespace eux::axon::utils {

struct hash_t {
  unsigned __int128 value = 0;
  constexpr hash_t() = default;
  explicit constexpr hash_t(unsigned __int128 v) : value(v) {}
  explicit constexpr hash_t(uint64_t v) : value(v) {}
  constexpr hash_t(uint64_t high, uint64_t low) : value((static_cast<unsigned __int128>(high) << 64) | low) {}
  static constexpr hash_t from_u64(uint64_t v) { return hash_t(v); }
  constexpr uint64_t high() const { return static_cast<uint64_t>(value >> 64); }
  constexpr uint64_t low() const { return static_cast<uint64_t>(value); }
  constexpr uint32_t low32() const { return static_cast<uint32_t>(value); }
  friend constexpr bool operator==(hash_t a, hash_t b) { return a.value == b.value; }
  friend constexpr bool operator<(hash_t a, hash_t b) { return a.value < b.value; }
};

hash_t HashBlock(const void* data, size_t n, hash_t seed);
hash_t DataHash(const void* data, size_t size);

inline hash_t HashCombine(hash_t a, hash_t b) {
  constexpr hash_t mul(101, 0x27d4eb2f165667c5ull);
  unsigned __int128 seed = b.value * mul.value;
  seed += static_cast<unsigned __int128>(0x9e3779b97f4a7c15ull);
  seed += (a.value << 6) + (a.value >> 2);
  return hash_t(a.value ^ seed);
}
inline hash_t StringHash(std::string_view s) { return DataHash(s.data(), s.size()); }

template <class T>
  requires std::is_arithmetic_v<T>
hash_t Hash(const T& v) {
  return DataHash(&v, sizeof(v));
}
inline hash_t Hash(const std::string& s) { return DataHash(s.data(), s.size()); }
inline hash_t Hash(std::string_view s) { return DataHash(s.data(), s.size()); }
inline hash_t Hash(const char* s) { return DataHash(s, std::strlen(s)); }
inline hash_t Hash(hash_t h) { return h; }
template <class T>
hash_t Hash(const std::vector<T>& values) {
  hash_t h(static_cast<uint64_t>(0x85ebca77c2b2ae63ull));
  for (const auto& v : values) h = HashCombine(h, Hash(v));
  return h;
}

inline hash_t MHash() { return hash_t(static_cast<uint64_t>(0x165667b19e3779f9ull)); }
template <class T, class... Rest>
hash_t MHash(const T& value, const Rest&... rest) {
  return HashCombine(Hash(value), MHash(rest...));
}

// id of a function addressed by name on a given worker
inline uint32_t FunctionIdFromName(std::string_view function_name, std::string_view worker_name) {
  return MHash(function_name, worker_name).low32();
}
// key of a worker addressed by name
inline uint64_t WorkerKeyFromName(std::string_view worker_name) { return StringHash(worker_name).low(); }

}  // namespace eux::axon::utils
