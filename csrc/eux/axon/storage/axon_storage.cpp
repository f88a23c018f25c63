#include "eux/axon/storage/axon_storage.hpp"

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <random>

#include "eux/axon/storage/avro_schema.hpp"
#include "eux/axon/storage/avro_serialization.hpp"
#include "eux/axon/storage/unifex_io.hpp"

namespace eux::axon::storage {

namespace {
// file work of whole checkpoints runs on its own thread so that it can wait for the stream's IO thread
exec::static_thread_pool::scheduler FileIoContextForSave() {
  static exec::static_thread_pool pool(1);
  return pool.get_scheduler();
}
}  // namespace

std::string AsyncUnifexAvroIO::MakeFileName(const std::string& dir, const std::string& prefix) {
  auto now = std::chrono::system_clock::now();
  auto secs = std::chrono::duration_cast<std::chrono::seconds>(now.time_since_epoch()).count();
  auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(now.time_since_epoch()).count() % 1000;
  char buf[64];
  std::snprintf(buf, sizeof(buf), "_%lld.%03d.avro", static_cast<long long>(secs), static_cast<int>(ms));
  return dir + (dir.empty() || dir.back() == '/' ? "" : "/") + prefix + buf;
}

std::string AsyncUnifexAvroIO::SaveSync(const std::vector<RequestPtr>& requests, ucxx::UcxMemoryResourceManager& mr,
                                        const std::string& dir, const std::string& prefix) {
  const std::string path = MakeFileName(dir, prefix);
  UnifexOutputStream out(path);
  uint8_t sync[16];
  std::random_device rd;
  for (auto& b : sync) b = static_cast<uint8_t>(rd());
  std::vector<uint8_t> chunk;
  avro::write_container_header(chunk, AvroSchema::GetArrivalRequestSchema(), sync);
  out.write(chunk.data(), chunk.size());
  // blocks of up to 64 records
  std::vector<uint8_t> records;
  size_t in_block = 0;
  auto flush_block = [&] {
    if (!in_block) return;
    chunk.clear();
    avro::write_container_block(chunk, in_block, records, sync);
    out.write(chunk.data(), chunk.size());
    records.clear();
    in_block = 0;
  };
  for (auto& r : requests) {
    if (!r) continue;
    AvroSerialization::Serialize(*r, mr, records);
    if (++in_block == 64 || records.size() > (8u << 20)) flush_block();
  }
  flush_block();
  out.flush();
  return path;
}

std::vector<RequestPtr> AsyncUnifexAvroIO::LoadSync(const std::string& path, ucxx::UcxMemoryResourceManager& mr) {
  UnifexInputStream in(path);
  std::vector<uint8_t> bytes = in.read_all();
  avro::Decoder d(bytes.data(), bytes.size());
  auto header = avro::read_container_header(d);
  std::vector<RequestPtr> out;
  while (!d.at_end()) {
    int64_t count = d.get_long();
    int64_t size = d.get_long();
    if (count < 0 || size < 0) throw std::runtime_error("avro: bad block header");
    const uint8_t* start = d.cursor();
    avro::Decoder block(start, static_cast<size_t>(size));
    d.skip(static_cast<size_t>(size));
    for (int64_t i = 0; i < count; ++i) out.push_back(AvroSerialization::Deserialize(block, mr));
    uint8_t sync[16];
    d.raw(sync, 16);
    if (std::memcmp(sync, header.sync, 16) != 0) throw std::runtime_error("avro: sync marker mismatch");
  }
  return out;
}

exec::any_sender_of<std::string> AsyncUnifexAvroIO::Save(std::vector<RequestPtr> requests, ucxx::UcxMemoryResourceManager& mr,
                                                         const std::string& dir, const std::string& prefix) {
  // serialisation runs on the IO context; the writes inside it overlap through the double-buffered stream
  return exec::on(FileIoContextForSave(), exec::just_from([requests = std::move(requests), &mr, dir, prefix] {
                    return SaveSync(requests, mr, dir, prefix);
                  }));
}
exec::any_sender_of<std::vector<RequestPtr>> AsyncUnifexAvroIO::Load(const std::string& path, ucxx::UcxMemoryResourceManager& mr) {
  return exec::on(FileIoContextForSave(), exec::just_from([path, &mr] { return LoadSync(path, mr); }));
}

utils::AxonMessageID AxonStorage::emplace(RequestPtr req) {
  const utils::AxonMessageID id = req->header.hlc.Raw();
  return emplace(std::move(req), id);
}
utils::AxonMessageID AxonStorage::emplace(RequestPtr req, utils::AxonMessageID id) {
  std::lock_guard lk(mu_);
  auto old = index_.find(id);
  if (old != index_.end()) {
    items_.erase(old->second);
    index_.erase(old);
  }
  items_.push_back(std::move(req));
  index_[id] = std::prev(items_.end());
  return id;
}
RequestPtr AxonStorage::find(utils::AxonMessageID id) const {
  std::lock_guard lk(mu_);
  auto it = index_.find(id);
  return it == index_.end() ? nullptr : *it->second;
}
bool AxonStorage::erase(utils::AxonMessageID id) {
  std::lock_guard lk(mu_);
  auto it = index_.find(id);
  if (it == index_.end()) return false;
  items_.erase(it->second);
  index_.erase(it);
  return true;
}
size_t AxonStorage::size() const {
  std::lock_guard lk(mu_);
  return items_.size();
}
void AxonStorage::clear() {
  std::lock_guard lk(mu_);
  items_.clear();
  index_.clear();
}
std::vector<std::pair<utils::AxonMessageID, RequestPtr>> AxonStorage::snapshot() const {
  std::lock_guard lk(mu_);
  std::vector<std::pair<utils::AxonMessageID, RequestPtr>> out;
  out.reserve(items_.size());
  for (auto& [id, it] : index_) out.emplace_back(id, *it);
  std::sort(out.begin(), out.end(), [](auto& a, auto& b) { return a.first < b.first; });
  return out;
}
std::string AxonStorage::save(ucxx::UcxMemoryResourceManager& mr, const std::string& dir, const std::string& prefix) const {
  std::vector<RequestPtr> reqs;
  for (auto& [id, r] : snapshot()) reqs.push_back(r);
  return AsyncUnifexAvroIO::SaveSync(reqs, mr, dir, prefix);
}
size_t AxonStorage::load(ucxx::UcxMemoryResourceManager& mr, const std::string& path) {
  auto reqs = AsyncUnifexAvroIO::LoadSync(path, mr);
  for (auto& r : reqs) emplace(r);
  return reqs.size();
}
std::string AxonStorage::save_request(ucxx::UcxMemoryResourceManager& mr, utils::AxonMessageID id, const std::string& dir) const {
  RequestPtr r = find(id);
  if (!r) throw std::out_of_range("no stored request with this id");
  return AsyncUnifexAvroIO::SaveSync({r}, mr, dir, std::to_string(r->header.session_id.v_));
}

}  // namespace eux::axon::storage
