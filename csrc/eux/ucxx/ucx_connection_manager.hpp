// ConnectionManager: owns every UcxConnection of a context and moves it through
// active -> inactive -> {failed queue | disconnecting list} -> recycled slot
// (reference: ucx_context/ucx_connection_manager.hpp:43-116). Slots are reused
// through a lock-free free list; all other methods run on the context's thread.
#pragma once

#include <deque>
#include <list>
#include <memory>
#include <optional>
#include <unordered_map>
#include <vector>

#include "eux/ucxx/lock_free_queue.hpp"
#include "eux/ucxx/ucx_connection.hpp"

namespace eux::ucxx {

class ConnectionManager {
 public:
  struct FailedConnection {
    conn_id_t id;
    int status;
    std::string peer_name;
    std::unique_ptr<UcxConnection> conn;
  };

  ConnectionManager() = default;
  ~ConnectionManager() = default;

  // Take ownership; the connection becomes active under its id.
  conn_id_t add_connection(std::unique_ptr<UcxConnection> conn);
  UcxConnection* get_connection(conn_id_t id) const;
  bool is_active(conn_id_t id) const { return active_map_.count(id) != 0; }
  size_t active_count() const { return active_map_.size(); }
  size_t failed_count() const { return failed_.size(); }
  size_t slot_count() const { return slots_.size(); }

  // active -> inactive (no new operations), keeps the object alive
  bool deactivate(conn_id_t id);
  // inactive/active -> failed queue (for handle_error_connection)
  bool mark_failed(conn_id_t id, int status);
  std::optional<FailedConnection> pop_failed();
  // inactive/active -> disconnecting list; closes the endpoint
  bool disconnect(conn_id_t id);
  // drop finished disconnects, returning their slots to the free list
  size_t reap_disconnected();
  void clear();
  template <class F>
  void for_each_active(F&& f) const {
    for (auto& [id, slot] : active_map_) f(id, *slots_[slot]);
  }

 private:
  size_t acquire_slot();
  void release_slot(size_t slot);
  std::vector<std::unique_ptr<UcxConnection>> slots_;
  std::unordered_map<conn_id_t, size_t> active_map_;
  std::unordered_map<conn_id_t, size_t> inactive_map_;
  std::deque<FailedConnection> failed_;
  std::list<std::unique_ptr<UcxConnection>> disconnecting_;
  LockFreeQueue<size_t> free_slots_;
};

}  // namespace eux::ucxx
