// AxonStorage: the worker's collection of retained requests (insertion keeps
// references stable, erasure is O(1)), with save/load to Avro container files
// named "<prefix>_<epoch seconds>.<milliseconds>.avro"
// (reference: axon/include/axon/storage/axon_storage.hpp:63-194,
// storage/async_io.hpp:150-255).
#pragma once

#include <list>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "eux/axon/utils/axon_message.hpp"
#include "eux/exec/async_scope.hpp"

namespace eux::axon::storage {

using RequestPtr = std::shared_ptr<utils::AxonRequest>;

// File-level IO: a range of requests <-> one container file.
class AsyncUnifexAvroIO {
 public:
  // "<dir>/<prefix>_<time_t>.<ms>.avro"
  static std::string MakeFileName(const std::string& dir, const std::string& prefix);
  // senders; Save completes with the path written, Load with the requests read
  static exec::any_sender_of<std::string> Save(std::vector<RequestPtr> requests, ucxx::UcxMemoryResourceManager& mr,
                                               const std::string& dir, const std::string& prefix);
  static exec::any_sender_of<std::vector<RequestPtr>> Load(const std::string& path, ucxx::UcxMemoryResourceManager& mr);
  // blocking forms used by the senders
  static std::string SaveSync(const std::vector<RequestPtr>& requests, ucxx::UcxMemoryResourceManager& mr, const std::string& dir,
                              const std::string& prefix);
  static std::vector<RequestPtr> LoadSync(const std::string& path, ucxx::UcxMemoryResourceManager& mr);
};

class AxonStorage {
 public:
  using iterator = std::list<RequestPtr>::iterator;

  AxonStorage() = default;
  AxonStorage(const AxonStorage&) = delete;

  // keep a request; returns its id (the request's hybrid-logical-clock value unless one is given)
  utils::AxonMessageID emplace(RequestPtr req);
  utils::AxonMessageID emplace(RequestPtr req, utils::AxonMessageID id);
  RequestPtr find(utils::AxonMessageID id) const;
  bool erase(utils::AxonMessageID id);
  size_t size() const;
  bool empty() const { return size() == 0; }
  void clear();
  std::vector<std::pair<utils::AxonMessageID, RequestPtr>> snapshot() const;

  // checkpoint everything / restore (restored requests are appended); the path of the file is returned
  std::string save(ucxx::UcxMemoryResourceManager& mr, const std::string& dir, const std::string& prefix = "axon") const;
  size_t load(ucxx::UcxMemoryResourceManager& mr, const std::string& path);
  // one request to its own file
  std::string save_request(ucxx::UcxMemoryResourceManager& mr, utils::AxonMessageID id, const std::string& dir) const;

 private:
  mutable std::mutex mu_;
  std::list<RequestPtr> items_;
  std::unordered_map<utils::AxonMessageID, iterator> index_;
};

}  // namespace eux::axon::storage
