// Hybrid logical clock: 48 bits of physical milliseconds and a 16-bit logical
// counter in one uint64 (raw = physical_ms << 16 | logical), carried by every
// RPC header to order causally related messages (reference:
// rpc_core/utils/hybrid_logical_clock.hpp:42-190).
#pragma once

#include <chrono>
#include <string>
#include <cstdint>
#include <tuple>

#include "eux/rpc/data.hpp"

namespace eux::rpc::utils {

class HybridLogicalClock final {
 public:
  static constexpr uint64_t kLogicalBits = 16;
  static constexpr uint64_t kLogicalMask = (1ULL << kLogicalBits) - 1ULL;
  static constexpr uint64_t kPhysicalMask = ~kLogicalMask;

  constexpr HybridLogicalClock() noexcept = default;
  explicit constexpr HybridLogicalClock(uint64_t raw_timestamp) noexcept : raw_(raw_timestamp) {}
  constexpr HybridLogicalClock(uint64_t physical_time_ms, uint16_t logical_counter) noexcept
      : raw_(Pack(physical_time_ms, logical_counter)) {}

  static HybridLogicalClock Now() noexcept { return HybridLogicalClock{CurrentPhysicalTimeMs(), 0}; }

  [[nodiscard]] constexpr uint64_t Raw() const noexcept { return raw_; }
  [[nodiscard]] constexpr uint64_t PhysicalTimeMs() const noexcept { return raw_ >> kLogicalBits; }
  [[nodiscard]] constexpr uint16_t LogicalCounter() const noexcept { return static_cast<uint16_t>(raw_ & kLogicalMask); }

  // A local event (send, internal step): time moves forward, never backward.
  void TickLocal() noexcept { TickLocal(CurrentPhysicalTimeMs()); }
  void TickLocal(uint64_t observed_physical_ms) noexcept {
    const uint64_t phys = PhysicalTimeMs();
    if (observed_physical_ms > phys) {
      raw_ = Pack(observed_physical_ms, 0);
    } else {
      Bump(phys, LogicalCounter());
    }
  }
  // A message arrived carrying `remote`: the result is later than both clocks.
  void Merge(const HybridLogicalClock& remote) noexcept { Merge(remote, CurrentPhysicalTimeMs()); }
  void Merge(uint64_t remote_raw) noexcept { Merge(HybridLogicalClock{remote_raw}); }
  void Merge(const HybridLogicalClock& remote, uint64_t observed_physical_ms) noexcept {
    const uint64_t lp = PhysicalTimeMs(), rp = remote.PhysicalTimeMs();
    const uint64_t top = lp > rp ? lp : rp;
    if (observed_physical_ms > top) {
      raw_ = Pack(observed_physical_ms, 0);
      return;
    }
    uint64_t logical;
    if (lp == rp) logical = LogicalCounter() > remote.LogicalCounter() ? LogicalCounter() : remote.LogicalCounter();
    else logical = lp > rp ? LogicalCounter() : remote.LogicalCounter();
    Bump(top, static_cast<uint16_t>(logical));
  }
  // The remote clock as its raw 64-bit value, with the wall clock the caller observed
  // (reference: rpc_core/utils/hybrid_logical_clock.hpp:84-125).
  void Merge(uint64_t remote_raw, uint64_t observed_physical_ms) noexcept {
    Merge(HybridLogicalClock{remote_raw}, observed_physical_ms);
  }
  void Assign(uint64_t physical_ms, uint16_t logical) noexcept { raw_ = Pack(physical_ms, logical); }
  void AssignRaw(uint64_t raw) noexcept { raw_ = raw; }
  // Next logical value under the same physical time; the 16-bit counter wraps to 0 on its own
  // (no carry into the physical part: that is what the reference's BumpLogicalCounter does).
  void BumpLogicalCounter() noexcept {
    raw_ = (raw_ & ~kLogicalMask) | ((static_cast<uint64_t>(LogicalCounter()) + 1) & kLogicalMask);
  }
  // "<physical ms>.<logical>"
  [[nodiscard]] std::string ToString() const { return std::to_string(PhysicalTimeMs()) + "." + std::to_string(LogicalCounter()); }

  [[nodiscard]] constexpr bool operator==(const HybridLogicalClock& o) const noexcept { return raw_ == o.raw_; }
  [[nodiscard]] constexpr bool operator!=(const HybridLogicalClock& o) const noexcept { return raw_ != o.raw_; }
  [[nodiscard]] constexpr bool operator<(const HybridLogicalClock& o) const noexcept { return raw_ < o.raw_; }
  [[nodiscard]] constexpr bool operator<=(const HybridLogicalClock& o) const noexcept { return raw_ <= o.raw_; }
  [[nodiscard]] constexpr bool operator>(const HybridLogicalClock& o) const noexcept { return raw_ > o.raw_; }
  [[nodiscard]] constexpr bool operator>=(const HybridLogicalClock& o) const noexcept { return raw_ >= o.raw_; }

 private:
  static constexpr uint64_t Pack(uint64_t physical_ms, uint16_t logical) noexcept {
    return (physical_ms << kLogicalBits) | static_cast<uint64_t>(logical);
  }
  // next logical value; when the 16-bit counter is exhausted the physical part advances by 1 ms
  void Bump(uint64_t physical_ms, uint16_t logical) noexcept {
    if (logical == kLogicalMask) raw_ = Pack(physical_ms + 1, 0);
    else raw_ = Pack(physical_ms, static_cast<uint16_t>(logical + 1));
  }
  static uint64_t CurrentPhysicalTimeMs() noexcept {
    return static_cast<uint64_t>(
        std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::system_clock::now().time_since_epoch()).count());
  }
  uint64_t raw_{0};
};

using workflow_id_t = strong<uint32_t, struct workflow_id_tag>;

}  // namespace eux::rpc::utils
