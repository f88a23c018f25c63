// Generational slot map: insert returns a key {index, generation}; a key of an
// erased element never matches a later occupant of the same index. A wrapper
// with a shared_mutex serves the table of remote endpoints, read on every call
// (reference: axon/include/axon/utils/slot_map.hpp:36-330).
#pragma once

#include <cstdint>
#include <mutex>
#include <optional>
#include <shared_mutex>
#include <utility>
#include <vector>

namespace eux::axon::utils {

struct SlotKey {
  uint32_t index = 0;
  uint32_t generation = 0;
  friend bool operator==(SlotKey a, SlotKey b) { return a.index == b.index && a.generation == b.generation; }
  uint64_t packed() const { return (static_cast<uint64_t>(generation) << 32) | index; }
  static SlotKey unpack(uint64_t v) { return {static_cast<uint32_t>(v), static_cast<uint32_t>(v >> 32)}; }
};

template <class T>
class SlotMap {
 public:
  template <class... A>
  SlotKey emplace(A&&... a) {
    uint32_t idx;
    if (!free_.empty()) {
      idx = free_.back();
      free_.pop_back();
    } else {
      idx = static_cast<uint32_t>(slots_.size());
      slots_.emplace_back();
    }
    Slot& s = slots_[idx];
    s.value.emplace(std::forward<A>(a)...);
    ++size_;
    return {idx, s.generation};
  }
  SlotKey insert(T v) { return emplace(std::move(v)); }
  T* find(SlotKey k) {
    if (k.index >= slots_.size()) return nullptr;
    Slot& s = slots_[k.index];
    return (s.generation == k.generation && s.value) ? &*s.value : nullptr;
  }
  const T* find(SlotKey k) const { return const_cast<SlotMap*>(this)->find(k); }
  bool contains(SlotKey k) const { return find(k) != nullptr; }
  bool erase(SlotKey k) {
    if (!find(k)) return false;
    Slot& s = slots_[k.index];
    s.value.reset();
    ++s.generation;
    free_.push_back(k.index);
    --size_;
    return true;
  }
  size_t size() const { return size_; }
  bool empty() const { return size_ == 0; }
  void clear() {
    for (uint32_t i = 0; i < slots_.size(); ++i)
      if (slots_[i].value) erase({i, slots_[i].generation});
  }
  template <class F>
  void for_each(F&& f) {
    for (uint32_t i = 0; i < slots_.size(); ++i)
      if (slots_[i].value) f(SlotKey{i, slots_[i].generation}, *slots_[i].value);
  }

 private:
  struct Slot {
    uint32_t generation = 1;
    std::optional<T> value;
  };
  std::vector<Slot> slots_;
  std::vector<uint32_t> free_;
  size_t size_ = 0;
};

// Readers take a shared lock; `access_lockless` is for the owner thread when it
// knows no writer can run (e.g. during single-threaded start-up).
template <class T>
class SharedSlotMap {
 public:
  template <class... A>
  SlotKey emplace(A&&... a) {
    std::unique_lock lk(mu_);
    return map_.emplace(std::forward<A>(a)...);
  }
  bool erase(SlotKey k) {
    std::unique_lock lk(mu_);
    return map_.erase(k);
  }
  template <class F>
  auto access(SlotKey k, F&& f) const -> std::optional<std::invoke_result_t<F, const T&>> {
    std::shared_lock lk(mu_);
    const T* p = map_.find(k);
    if (!p) return std::nullopt;
    return f(*p);
  }
  template <class F>
  bool modify(SlotKey k, F&& f) {
    std::unique_lock lk(mu_);
    T* p = map_.find(k);
    if (!p) return false;
    f(*p);
    return true;
  }
  T* access_lockless(SlotKey k) { return map_.find(k); }
  template <class F>
  void for_each(F&& f) {
    std::shared_lock lk(mu_);
    map_.for_each(std::forward<F>(f));
  }
  size_t size() const {
    std::shared_lock lk(mu_);
    return map_.size();
  }
  void clear() {
    std::unique_lock lk(mu_);
    map_.clear();
  }

 private:
  mutable std::shared_mutex mu_;
  SlotMap<T> map_;
};

}  // namespace eux::axon::utils
