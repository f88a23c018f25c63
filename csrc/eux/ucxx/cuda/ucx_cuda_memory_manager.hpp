// CUDA memory resource manager with pooled, registered and peer-exportable
// device memory.
//
// The reference ships a test-grade manager (cudaMalloc per allocation, blocking
// cudaMemcpy; ucx_context/cuda/ucx_cuda_memory_manager.hpp:43-154) and registers
// user memory with ucp_mem_map (ucx_am_context.cpp:1128-1147). Here:
//   * CUDA allocations are carved out of large cudaMalloc arenas (first fit,
//     256-byte granules, coalescing free list), so a receive never pays for
//     cudaMalloc and every pooled byte is already registered;
//   * register_memory() records an allocation (found from any interior pointer)
//     and export_region() produces a PeerRegionDesc carrying its CUDA IPC
//     handle, which a peer process opens once with import_region() and caches;
//   * memory that somebody else made with cuMemCreate and mapped into a reserved address range (a tensor
//     library's "expandable segments") has no CUDA IPC handle; each physical allocation under it is
//     exported as a POSIX file descriptor instead (export_vmm_fd), which the transport passes to the peer
//     over a Unix socket, and the peer maps it into a range of its own (import_vmm);
//   * the same descriptor works inside one process (the address is used as is).
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "eux/ucxx/ucx_memory_resource.hpp"

namespace eux::ucxx {

// Wire-format description of a byte range in some process's device memory.
struct PeerRegionDesc {
  uint32_t pid = 0;
  int32_t device = -1;
  uint64_t base = 0;    // base address of the allocation in the owner's address space
  uint64_t offset = 0;  // start of the range inside the allocation
  uint64_t length = 0;
  uint8_t exportable = 0;
  uint8_t kind = 0;  // kRegionIpc: `handle` is a cudaIpcMemHandle_t; kRegionVmm: it starts with a PeerVmmRef
  uint8_t reserved[6] = {0};
  unsigned char handle[64] = {0};
};
constexpr uint8_t kRegionIpc = 0, kRegionVmm = 1;
// What stands for the handle of a cuMemCreate allocation: the owner's number for it (never reused within
// the owner's process) and its size. The file descriptor itself cannot travel in a message; the owner
// passes it once per peer over a Unix socket, labelled with the same number.
struct PeerVmmRef {
  uint64_t id = 0;
  uint64_t size = 0;
};
static_assert(sizeof(PeerRegionDesc) == 104, "PeerRegionDesc travels on the wire");

class UcxCudaMemoryResourceManager : public UcxMemoryResourceManager {
 public:
  struct Options {
    int device = 0;
    size_t arena_bytes = size_t(64) << 20;
    bool pinned_host = false;  // HOST allocations from cudaHostAlloc (staging buffers)
    // Blocks too large for an arena are kept after they are freed and handed out again for a
    // request of a similar size (cudaMalloc/cudaFree synchronise the device, and a reused block
    // keeps its export handle, so the peers' mappings stay valid). Up to this many idle bytes.
    size_t large_cache_bytes = size_t(32) << 30;
  };
  struct Registration {
    void* base = nullptr;
    size_t size = 0;
    int device = -1;
    bool exportable = false;
    unsigned char handle[64] = {0};
    uint64_t buffer_id = 0;  // the driver's id of the allocation (0: unknown), to recognise it again cheaply
    uint8_t kind = kRegionIpc;
    uint64_t vmm_id = 0;     // kRegionVmm: this process's number for the physical allocation
  };

  UcxCudaMemoryResourceManager();
  explicit UcxCudaMemoryResourceManager(const Options& opt);
  ~UcxCudaMemoryResourceManager() override;

  void* allocate(ucx_memory_type_t type, size_t bytes, size_t alignment = 8) override;
  void deallocate(ucx_memory_type_t type, void* p, size_t bytes, size_t alignment = 8) override;
  void* memcpy(ucx_memory_type_t dest_type, void* dest, ucx_memory_type_t src_type, const void* src,
               size_t count) override;

  // Record the allocation that contains ptr (its extent is asked from the driver).
  const Registration* register_memory(const void* ptr, size_t size);
  bool unregister_memory(const void* ptr);
  const Registration* find_registration(const void* ptr) const;
  // Describe [ptr, ptr+len) for a peer; registers the allocation on first use.
  bool export_region(const void* ptr, size_t len, PeerRegionDesc* out);
  // The same for a range that may run across several allocations that lie back to back in the address
  // space (a large tensor in expandable segments is backed by one cuMemCreate allocation per 20 MiB):
  // one descriptor per allocation touched, appended to `out`. False (and `out` as it was) when any part
  // of the range is unknown to the driver.
  bool export_regions(const void* ptr, size_t len, std::vector<PeerRegionDesc>* out);
  // A new file descriptor for the cuMemCreate allocation described by a kRegionVmm descriptor of this
  // process (the caller passes it on and closes it), or -1.
  int export_vmm_fd(const PeerRegionDesc& d);
  // Map a peer's cuMemCreate allocation, received as a file descriptor (not closed here), and remember it
  // under (owner, id). `owner` is the caller's name for the peer (the transport uses the peer worker's
  // random id). True when it is mapped (now or before).
  bool import_vmm(uint64_t owner, const PeerVmmRef& ref, int fd);
  // Forget one mapping of that owner (it said that the allocation is gone), or all of them.
  void release_vmm(uint64_t owner, uint64_t id);
  void release_vmm_of(uint64_t owner);
  // Map a peer's region into this process (cached per owner pid + allocation); nullptr on failure.
  // `same_process` is the caller's own knowledge that the region's owner lives in this process (the
  // transport derives it from its registry of live workers, never from the descriptor): only then
  // is the descriptor's address used as it is, and only after the driver confirmed that the whole
  // range lies inside one allocation of this process. A mapped region is checked the same way.
  // kRegionVmm descriptors of another process are looked up among the mappings made by import_vmm under `owner`.
  void* import_region(const PeerRegionDesc& d, bool same_process = false, uint64_t owner = 0);
  void release_imports();

  int device() const { return opt_.device; }
  size_t pooled_bytes() const;
  size_t pooled_bytes_in_use() const;

 private:
  struct Arena {
    char* base = nullptr;
    size_t size = 0;
    std::map<size_t, size_t> free_by_off;  // offset -> length
    size_t in_use = 0;
  };
  void* pool_alloc(size_t bytes);
  bool pool_free(void* p, size_t bytes);
  Options opt_;
  mutable std::mutex mu_;
  std::vector<Arena> arenas_;
  std::unordered_map<void*, size_t> dedicated_;  // oversize allocations in use (rounded size)
  std::multimap<size_t, void*> large_idle_;      // oversize allocations waiting for reuse
  size_t large_idle_bytes_ = 0;
  std::map<uintptr_t, Registration> regs_;       // by base address
  struct ImportKey {
    uint32_t pid;
    uint64_t base;
    bool operator<(const ImportKey& o) const { return pid != o.pid ? pid < o.pid : base < o.base; }
  };
  struct Imported {
    void* mapped = nullptr;
    unsigned char handle[64] = {0};  // the handle this mapping was opened with
  };
  std::map<ImportKey, Imported> imports_;
  struct VmmImported {
    uint64_t va = 0;
    uint64_t size = 0;
    uint64_t handle = 0;  // CUmemGenericAllocationHandle
  };
  std::map<std::pair<uint64_t, uint64_t>, VmmImported> vmm_imports_;  // by (owner, id)
  void unmap_vmm(VmmImported& m);                                       // mu_ held
  bool is_pool_base(const void* base) const;  // mu_ held
};

}  // namespace eux::ucxx
