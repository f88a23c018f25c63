#include "eux/ucxx/ucx_connection_manager.hpp"

namespace eux::ucxx {

size_t ConnectionManager::acquire_slot() {
  if (auto s = free_slots_.pop()) return *s;
  slots_.emplace_back();
  return slots_.size() - 1;
}
void ConnectionManager::release_slot(size_t slot) {
  slots_[slot].reset();
  free_slots_.push(slot);
}

conn_id_t ConnectionManager::add_connection(std::unique_ptr<UcxConnection> conn) {
  const conn_id_t id = conn->id();
  const size_t slot = acquire_slot();
  slots_[slot] = std::move(conn);
  active_map_[id] = slot;
  return id;
}

UcxConnection* ConnectionManager::get_connection(conn_id_t id) const {
  auto it = active_map_.find(id);
  if (it != active_map_.end()) return slots_[it->second].get();
  auto jt = inactive_map_.find(id);
  return jt != inactive_map_.end() ? slots_[jt->second].get() : nullptr;
}

bool ConnectionManager::deactivate(conn_id_t id) {
  auto it = active_map_.find(id);
  if (it == active_map_.end()) return false;
  inactive_map_[id] = it->second;
  active_map_.erase(it);
  return true;
}

bool ConnectionManager::mark_failed(conn_id_t id, int status) {
  deactivate(id);
  auto it = inactive_map_.find(id);
  if (it == inactive_map_.end()) return false;
  const size_t slot = it->second;
  inactive_map_.erase(it);
  FailedConnection f{id, status, slots_[slot]->peer_name(), std::move(slots_[slot])};
  f.conn->mark_failed(status);
  failed_.push_back(std::move(f));
  release_slot(slot);
  return true;
}

std::optional<ConnectionManager::FailedConnection> ConnectionManager::pop_failed() {
  if (failed_.empty()) return std::nullopt;
  FailedConnection f = std::move(failed_.front());
  failed_.pop_front();
  return f;
}

bool ConnectionManager::disconnect(conn_id_t id) {
  deactivate(id);
  auto it = inactive_map_.find(id);
  if (it == inactive_map_.end()) return false;
  const size_t slot = it->second;
  inactive_map_.erase(it);
  slots_[slot]->disconnect();
  disconnecting_.push_back(std::move(slots_[slot]));
  release_slot(slot);
  return true;
}

size_t ConnectionManager::reap_disconnected() {
  size_t n = disconnecting_.size();
  disconnecting_.clear();
  return n;
}

void ConnectionManager::clear() {
  std::vector<conn_id_t> ids;
  for (auto& [id, s] : active_map_) ids.push_back(id);
  for (auto& [id, s] : inactive_map_) ids.push_back(id);
  for (auto id : ids) disconnect(id);
  reap_disconnected();
  failed_.clear();
}

}  // namespace eux::ucxx
