#include "eux/axon/utils/hash.hpp"

namespace eux::axon::utils {

hash_t HashBlock(const void* data, size_t n, hash_t seed) {
  const unsigned __int128 m = 0xc6a4a7935bd1e995ull;
  const int r = 47;
  const uint8_t* p = static_cast<const uint8_t*>(data);
  const uint8_t* top = p + n;
  // the length term is reduced to 64 bits before it is mixed in
  unsigned __int128 h = seed.value ^ static_cast<uint64_t>(static_cast<unsigned __int128>(n) * m);
  while (p < top) {
    unsigned __int128 k = 0;
    const size_t take = static_cast<size_t>(top - p) >= sizeof(k) ? sizeof(k) : static_cast<size_t>(top - p);
    std::memcpy(&k, p, take);  // a short tail is zero-extended
    p += take;
    k *= m;
    k ^= k >> r;
    k *= m;
    h ^= k;
    h *= m;
  }
  h ^= h >> r;
  h *= m;
  h ^= h >> r;
  return hash_t(h);
}

hash_t DataHash(const void* data, size_t size) { return HashBlock(data, size, hash_t(static_cast<uint64_t>(0xc2b2ae3d27d4eb4full))); }

}  // namespace eux::axon::utils
