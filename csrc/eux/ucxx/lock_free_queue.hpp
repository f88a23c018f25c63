// Multi-producer multi-consumer FIFO (Michael & Scott, with a dummy head node).
// Used for the connection manager's free-slot list, like the reference's
// ucx_context/lock_free_queue.hpp:35-166. Nodes retired by pop() are kept on a
// lock-free free list and reused, so a node's memory is never returned to the
// allocator while another thread may still dereference it (that also removes
// the per-push allocation); counted pointers guard against ABA. A consumer reads
// the value before it tries to win the head, and a reused node may be refilled
// while a slow consumer still reads it (its compare-exchange then fails and the
// value is dropped), so values live in a relaxed atomic word: T must be
// trivially copyable and at most 8 bytes (indices, ids, pointers).
#pragma once

#include <atomic>
#include <cstdint>
#include <cstring>
#include <optional>
#include <type_traits>
#include <utility>

namespace eux::ucxx {

template <class T>
class LockFreeQueue {
  static_assert(std::is_trivially_copyable_v<T> && sizeof(T) <= 8, "LockFreeQueue holds small trivially copyable values");
  static std::uint64_t to_word(const T& v) {
    std::uint64_t w = 0;
    std::memcpy(&w, &v, sizeof(T));
    return w;
  }
  static T from_word(std::uint64_t w) {
    T v;
    std::memcpy(&v, &w, sizeof(T));
    return v;
  }
  struct Node;
  // Counted pointer packed into one 64-bit word (48-bit address, 16-bit tag) so
  // that every compare-exchange is a plain lock-free 8-byte operation.
  struct Ptr {
    Node* p;
    std::uintptr_t tag;
    Ptr() : p(nullptr), tag(0) {}
    Ptr(Node* p_, std::uintptr_t t) : p(p_), tag(t & 0xffffu) {}
    friend bool operator==(const Ptr& a, const Ptr& b) { return a.p == b.p && a.tag == b.tag; }
  };
  class AtomicPtr {
   public:
    AtomicPtr() : v_(0) {}
    explicit AtomicPtr(Ptr p) : v_(pack(p)) {}
    Ptr load(std::memory_order mo = std::memory_order_seq_cst) const { return unpack(v_.load(mo)); }
    void store(Ptr p, std::memory_order mo = std::memory_order_seq_cst) { v_.store(pack(p), mo); }
    bool compare_exchange_weak(Ptr& expected, Ptr desired, std::memory_order mo = std::memory_order_seq_cst) {
      std::uint64_t e = pack(expected);
      bool ok = v_.compare_exchange_weak(e, pack(desired), mo, std::memory_order_acquire);
      if (!ok) expected = unpack(e);
      return ok;
    }
    bool compare_exchange_strong(Ptr& expected, Ptr desired, std::memory_order mo = std::memory_order_seq_cst) {
      std::uint64_t e = pack(expected);
      bool ok = v_.compare_exchange_strong(e, pack(desired), mo, std::memory_order_acquire);
      if (!ok) expected = unpack(e);
      return ok;
    }

   private:
    static std::uint64_t pack(Ptr p) {
      return (reinterpret_cast<std::uint64_t>(p.p) & 0x0000ffffffffffffull) | (static_cast<std::uint64_t>(p.tag) << 48);
    }
    static Ptr unpack(std::uint64_t v) {
      return Ptr(reinterpret_cast<Node*>(v & 0x0000ffffffffffffull), static_cast<std::uintptr_t>(v >> 48));
    }
    std::atomic<std::uint64_t> v_;
  };
  struct Node {
    AtomicPtr next;
    std::atomic<std::uint64_t> value{0};
  };

 public:
  LockFreeQueue() {
    Node* dummy = new Node();
    head_.store(Ptr{dummy, 0});
    tail_.store(Ptr{dummy, 0});
  }
  ~LockFreeQueue() {
    while (pop()) {
    }
    delete head_.load().p;
    Node* f = free_.load().p;
    while (f) {
      Node* n = f->next.load().p;
      delete f;
      f = n;
    }
  }
  LockFreeQueue(const LockFreeQueue&) = delete;
  LockFreeQueue& operator=(const LockFreeQueue&) = delete;

  void push(T v) {
    Node* n = acquire();
    n->value.store(to_word(v), std::memory_order_relaxed);
    for (;;) {
      Ptr tail = tail_.load(std::memory_order_acquire);
      Ptr next = tail.p->next.load(std::memory_order_acquire);
      if (!(tail == tail_.load(std::memory_order_acquire))) continue;
      if (next.p == nullptr) {
        if (tail.p->next.compare_exchange_weak(next, Ptr{n, next.tag + 1}, std::memory_order_release)) {
          tail_.compare_exchange_strong(tail, Ptr{n, tail.tag + 1}, std::memory_order_release);
          size_.fetch_add(1, std::memory_order_relaxed);
          return;
        }
      } else {
        tail_.compare_exchange_strong(tail, Ptr{next.p, tail.tag + 1}, std::memory_order_release);
      }
    }
  }

  std::optional<T> pop() {
    for (;;) {
      Ptr head = head_.load(std::memory_order_acquire);
      Ptr tail = tail_.load(std::memory_order_acquire);
      Ptr next = head.p->next.load(std::memory_order_acquire);
      if (!(head == head_.load(std::memory_order_acquire))) continue;
      if (head.p == tail.p) {
        if (next.p == nullptr) return std::nullopt;
        tail_.compare_exchange_strong(tail, Ptr{next.p, tail.tag + 1}, std::memory_order_release);
        continue;
      }
      // read first: once the head moves past next.p another consumer may retire and refill it
      const std::uint64_t word = next.p->value.load(std::memory_order_relaxed);
      if (head_.compare_exchange_weak(head, Ptr{next.p, head.tag + 1}, std::memory_order_acq_rel)) {
        std::optional<T> out(from_word(word));
        release(head.p);
        size_.fetch_sub(1, std::memory_order_relaxed);
        return out;
      }
    }
  }

  bool empty() const { return size_.load(std::memory_order_relaxed) == 0; }
  std::size_t size() const { return size_.load(std::memory_order_relaxed); }

 private:
  Node* acquire() {
    for (;;) {
      Ptr f = free_.load(std::memory_order_acquire);
      if (!f.p) return new Node();
      Ptr next = f.p->next.load(std::memory_order_acquire);
      if (free_.compare_exchange_weak(f, Ptr{next.p, f.tag + 1}, std::memory_order_acq_rel)) {
        f.p->next.store(Ptr{nullptr, next.tag + 1}, std::memory_order_relaxed);
        return f.p;
      }
    }
  }
  void release(Node* n) {
    for (;;) {
      Ptr f = free_.load(std::memory_order_acquire);
      Ptr old = n->next.load(std::memory_order_relaxed);
      n->next.store(Ptr{f.p, old.tag + 1}, std::memory_order_relaxed);
      if (free_.compare_exchange_weak(f, Ptr{n, f.tag + 1}, std::memory_order_acq_rel)) return;
    }
  }
  alignas(64) AtomicPtr head_;
  alignas(64) AtomicPtr tail_;
  alignas(64) AtomicPtr free_;
  std::atomic<std::size_t> size_{0};
};

}  // namespace eux::ucxx
