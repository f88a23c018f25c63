// Symmetric device buffers over the runtime: every rank allocates a region from its CUDA memory
// resource, exports it (UcxCudaMemoryResourceManager::export_region) and tells its peers about it with an
// Axon call that travels as an active message over ucx_am_context; the peers map it
// (import_region) and get a pointer they can hand to kernels. This is how the all-to-all workloads
// (MoE dispatch / combine, all-peers GEMM) obtain each other's arenas, flag blocks and row headers:
// the handle exchange is the runtime's own control plane, not an out-of-band channel.
//
// The reference registers memory with ucp_mem_map and leaves every exchange of rkeys to the
// application (ucx_context/ucx_am_context/ucx_am_context.cpp:1128-1147); here the exchange is a service.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "eux/axon/axon_worker.hpp"
#include "eux/ucxx/cuda/ucx_cuda_memory_manager.hpp"

namespace eux::axon::services {

class PeerMemoryService {
 public:
  static constexpr const char* kFunctionName = "eux.peer_memory.publish";

  PeerMemoryService(AxonWorker& worker, std::shared_ptr<ucxx::UcxCudaMemoryResourceManager> mr, int rank, int world);
  ~PeerMemoryService();
  PeerMemoryService(const PeerMemoryService&) = delete;

  bool Register();  // the Axon function through which peers announce their regions
  int rank() const { return rank_; }
  int world() const { return world_; }

  // A zeroed region of `nbytes` of this rank's device memory under `tag` (tags are chosen by the
  // application, the same on every rank for the same buffer). Returns its address.
  void* Allocate(uint32_t tag, size_t nbytes);
  // Tell the worker `worker_name` where this rank's region `tag` is. Value: 0.
  exec::any_sender_of<int32_t> Publish(std::string_view worker_name, uint32_t tag);
  // How many peers have announced their region `tag` so far.
  int Arrived(uint32_t tag) const;
  // Map every announced region `tag`: `world` addresses usable on this GPU (this rank's own at `rank`).
  // Throws when a peer is missing or its memory cannot be mapped here.
  std::vector<uintptr_t> Resolve(uint32_t tag);
  // Give this rank's region back (the peers must have stopped using it).
  void Free(uint32_t tag);

 private:
  struct Local {
    void* base = nullptr;
    size_t bytes = 0;
  };
  struct Remote {
    ucxx::PeerRegionDesc desc;
    uint64_t uid = 0;
  };
  AxonWorker& worker_;
  std::shared_ptr<ucxx::UcxCudaMemoryResourceManager> mr_;
  const int rank_, world_;
  mutable std::mutex mu_;
  std::map<uint32_t, Local> local_;
  std::map<uint32_t, std::map<int, Remote>> remote_;  // tag -> rank -> announced region
  bool registered_ = false;
};

}  // namespace eux::axon::services
