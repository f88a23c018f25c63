#include "eux/axon/services/peer_memory_service.hpp"

#include <cuda_runtime_api.h>
#include <unistd.h>

#include <cstring>
#include <stdexcept>

#include "eux/axon/utils/hash.hpp"
#include "eux/ucxx/transport.hpp"

namespace eux::axon::services {

namespace ex = eux::exec;
using rpc::data::vector;
using ucxx::PeerRegionDesc;

PeerMemoryService::PeerMemoryService(AxonWorker& worker, std::shared_ptr<ucxx::UcxCudaMemoryResourceManager> mr, int rank, int world)
    : worker_(worker), mr_(std::move(mr)), rank_(rank), world_(world) {
  if (!mr_) throw std::invalid_argument("PeerMemoryService needs the CUDA memory resource manager of its worker");
  if (rank < 0 || world <= 0 || rank >= world) throw std::invalid_argument("PeerMemoryService: rank outside of the world");
}

PeerMemoryService::~PeerMemoryService() {
  if (registered_) worker_.UnregisterFunction(rpc::function_id_t{utils::FunctionIdFromName(kFunctionName, worker_.name())});
  for (auto& [tag, l] : local_) {
    try {
      if (l.base) mr_->deallocate(ucx_memory_type::CUDA, l.base, l.bytes);
    } catch (...) {
    }
  }
}

bool PeerMemoryService::Register() {
  if (registered_) return true;
  auto* self = this;
  auto handler = [self](uint32_t tag, int32_t from_rank, uint64_t uid, const vector<uint8_t>& desc) -> int32_t {
    if (desc.size() != sizeof(PeerRegionDesc) || from_rank < 0 || from_rank >= self->world_)
      throw std::invalid_argument("peer memory: malformed announcement");
    Remote r;
    std::memcpy(&r.desc, desc.data(), sizeof(PeerRegionDesc));
    r.uid = uid;
    std::lock_guard lk(self->mu_);
    self->remote_[tag][from_rank] = r;
    return 0;
  };
  ServerMemoryPolicy mp;
  mp.handler_inline = true;  // a map insertion
  registered_ = worker_.RegisterFunction(rpc::function_id_t{utils::FunctionIdFromName(kFunctionName, worker_.name())}, handler, kFunctionName,
                                         std::move(mp), MessageLifecyclePolicy{});
  return registered_;
}

void* PeerMemoryService::Allocate(uint32_t tag, size_t nbytes) {
  std::lock_guard lk(mu_);
  if (local_.count(tag)) throw std::invalid_argument("peer memory: the tag is in use");
  Local l;
  l.bytes = nbytes ? nbytes : 256;
  l.base = mr_->allocate(ucx_memory_type::CUDA, l.bytes);
  cudaSetDevice(mr_->device());
  if (cudaMemset(l.base, 0, l.bytes) != cudaSuccess) {
    cudaGetLastError();
    mr_->deallocate(ucx_memory_type::CUDA, l.base, l.bytes);
    throw std::runtime_error("peer memory: could not clear the region");
  }
  local_[tag] = l;
  return l.base;
}

exec::any_sender_of<int32_t> PeerMemoryService::Publish(std::string_view worker_name, uint32_t tag) {
  PeerRegionDesc d;
  {
    std::lock_guard lk(mu_);
    auto it = local_.find(tag);
    if (it == local_.end()) throw std::invalid_argument("peer memory: nothing allocated under this tag");
    if (!mr_->export_region(it->second.base, it->second.bytes, &d) || !d.exportable)
      throw std::runtime_error("peer memory: the region cannot be exported");
  }
  vector<uint8_t> bytes(sizeof(d));
  std::memcpy(bytes.data(), &d, sizeof(d));
  auto* ctx = worker_.client_context();
  const uint64_t uid = ctx ? ctx->worker().address().uid : 0;
  const rpc::function_id_t fid{utils::FunctionIdFromName(kFunctionName, std::string(worker_name))};
  auto call = worker_.InvokeRpc(worker_name, rpc::session_id_t{0}, fid, rpc::utils::workflow_id_t{0}, ClientMemoryPolicy{}, tag,
                                static_cast<int32_t>(rank_), uid, std::move(bytes));
  return exec::any_sender_of<int32_t>(ex::then(std::move(call), [](InvokeResult r) -> int32_t {
    if (!r.header.status.ok()) throw std::runtime_error("peer memory: the announcement was refused");
    return 0;
  }));
}

int PeerMemoryService::Arrived(uint32_t tag) const {
  std::lock_guard lk(mu_);
  auto it = remote_.find(tag);
  return it == remote_.end() ? 0 : static_cast<int>(it->second.size());
}

std::vector<uintptr_t> PeerMemoryService::Resolve(uint32_t tag) {
  std::lock_guard lk(mu_);
  auto mine = local_.find(tag);
  if (mine == local_.end()) throw std::invalid_argument("peer memory: nothing allocated under this tag");
  std::vector<uintptr_t> out(static_cast<size_t>(world_), 0);
  out[static_cast<size_t>(rank_)] = reinterpret_cast<uintptr_t>(mine->second.base);
  auto& peers = remote_[tag];
  for (int r = 0; r < world_; ++r) {
    if (r == rank_) continue;
    auto it = peers.find(r);
    if (it == peers.end()) throw std::runtime_error("peer memory: rank " + std::to_string(r) + " has not announced tag " + std::to_string(tag));
    const bool same = ucxx::transport::is_live_local_uid(it->second.uid) && it->second.desc.pid == static_cast<uint32_t>(getpid());
    void* p = mr_->import_region(it->second.desc, same);
    if (!p) throw std::runtime_error("peer memory: the region of rank " + std::to_string(r) + " cannot be mapped on this GPU");
    out[static_cast<size_t>(r)] = reinterpret_cast<uintptr_t>(p);
  }
  return out;
}

void PeerMemoryService::Free(uint32_t tag) {
  std::lock_guard lk(mu_);
  auto it = local_.find(tag);
  if (it != local_.end()) {
    mr_->deallocate(ucx_memory_type::CUDA, it->second.base, it->second.bytes);
    local_.erase(it);
  }
  remote_.erase(tag);
}

}  // namespace eux::axon::services
