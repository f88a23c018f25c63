#include "eux/ucxx/cuda/ucx_cuda_memory_manager.hpp"

#include <cuda.h>  // types of the virtual memory management calls; the functions come through the runtime's entry-point lookup
#include <cuda_runtime_api.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>

#include <cstring>
#include <new>
#include <stdexcept>

#include "eux/ucxx/cuda/ucx_cuda_macro.h"

namespace eux::ucxx {

namespace {
constexpr size_t kGranule = 256;
size_t round_up(size_t n, size_t a) { return (n + a - 1) / a * a; }

// cuMemGetAddressRange through the runtime's driver entry point (no link-time libcuda dependency)
bool address_range(const void* ptr, void** base, size_t* size) {
  using Fn = int (*)(unsigned long long*, size_t*, unsigned long long);
  static Fn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<Fn>(p);
  }();
  if (!fn) return false;
  unsigned long long b = 0;
  size_t s = 0;
  if (fn(&b, &s, reinterpret_cast<unsigned long long>(ptr)) != 0) return false;
  *base = reinterpret_cast<void*>(b);
  *size = s;
  return true;
}

// CU_POINTER_ATTRIBUTE_BUFFER_ID: a number the driver gives every allocation and never reuses, so a
// remembered allocation can be told from a new one at the same address in about a microsecond
// (asking for the IPC handle again, the other way to tell, costs tens of microseconds per message).
bool buffer_id_of(const void* ptr, uint64_t* id) {
  using Fn = int (*)(void*, int, unsigned long long);
  static Fn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuPointerGetAttribute", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<Fn>(p);
  }();
  if (!fn) return false;
  unsigned long long v = 0;
  constexpr int kBufferId = 9;  // CU_POINTER_ATTRIBUTE_BUFFER_ID
  if (fn(&v, kBufferId, reinterpret_cast<unsigned long long>(ptr)) != 0) return false;
  *id = v;
  return true;
}

// A driver function by name, through the runtime (no link-time libcuda dependency); null where there is no driver.
template <class Fn>
Fn driver_fn(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
    cudaGetLastError();
    p = nullptr;
  }
  return reinterpret_cast<Fn>(p);
}
// The virtual memory management calls used to pass cuMemCreate allocations between processes.
struct VmmApi {
  CUresult (*retain)(CUmemGenericAllocationHandle*, void*) = nullptr;
  CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*export_handle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*import_handle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*address_free)(CUdeviceptr, size_t) = nullptr;
  CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*set_access)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  bool ok = false;
};
const VmmApi& vmm_api() {
  static const VmmApi api = [] {
    VmmApi a;
    a.retain = driver_fn<decltype(a.retain)>("cuMemRetainAllocationHandle");
    a.release = driver_fn<decltype(a.release)>("cuMemRelease");
    a.export_handle = driver_fn<decltype(a.export_handle)>("cuMemExportToShareableHandle");
    a.import_handle = driver_fn<decltype(a.import_handle)>("cuMemImportFromShareableHandle");
    a.reserve = driver_fn<decltype(a.reserve)>("cuMemAddressReserve");
    a.address_free = driver_fn<decltype(a.address_free)>("cuMemAddressFree");
    a.map = driver_fn<decltype(a.map)>("cuMemMap");
    a.unmap = driver_fn<decltype(a.unmap)>("cuMemUnmap");
    a.set_access = driver_fn<decltype(a.set_access)>("cuMemSetAccess");
    a.ok = a.retain && a.release && a.export_handle && a.import_handle && a.reserve && a.address_free && a.map && a.unmap && a.set_access;
    return a;
  }();
  return api;
}
std::atomic<uint64_t> g_next_vmm_id{1};

// Allocation and release run on whatever thread asks (a pool thread, the caller's thread): the
// manager's device becomes current for the duration, whatever that thread had before.
struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  explicit DeviceGuard(int want) {
    if (want < 0) return;
    if (cudaGetDevice(&prev) == cudaSuccess && prev != want) switched = cudaSetDevice(want) == cudaSuccess;
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
};

class PinnedHostResource final : public std::pmr::memory_resource {
  void* do_allocate(size_t bytes, size_t) override {
    void* p = nullptr;
    if (cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocPortable) != cudaSuccess) throw std::bad_alloc();
    return p;
  }
  void do_deallocate(void* p, size_t, size_t) override { cudaFreeHost(p); }
  bool do_is_equal(const std::pmr::memory_resource& o) const noexcept override { return this == &o; }
};
PinnedHostResource& pinned_resource() {
  static PinnedHostResource r;
  return r;
}
}  // namespace

UcxCudaMemoryResourceManager::UcxCudaMemoryResourceManager() : UcxCudaMemoryResourceManager(Options{}) {}

UcxCudaMemoryResourceManager::UcxCudaMemoryResourceManager(const Options& opt) : opt_(opt) {
  if (opt_.pinned_host) register_memory_resource(ucx_memory_type::HOST, pinned_resource());
  else register_memory_resource(ucx_memory_type::HOST, *std::pmr::new_delete_resource());
  auto copy = [](cudaMemcpyKind kind) {
    return [kind](void* d, const void* s, size_t n) -> void* {
      if (n) EUX_CUDA_CHECK(cudaMemcpy(d, s, n, kind));
      return d;
    };
  };
  const ucx_memory_type_t dev_kinds[] = {ucx_memory_type::CUDA, ucx_memory_type::CUDA_MANAGED};
  register_memcpy_fn(ucx_memory_type::HOST, ucx_memory_type::HOST,
                     [](void* d, const void* s, size_t n) { return std::memcpy(d, s, n); });
  for (auto k : dev_kinds) {
    register_memcpy_fn(k, ucx_memory_type::HOST, copy(cudaMemcpyHostToDevice));
    register_memcpy_fn(ucx_memory_type::HOST, k, copy(cudaMemcpyDeviceToHost));
    for (auto k2 : dev_kinds) register_memcpy_fn(k, k2, copy(cudaMemcpyDeviceToDevice));
  }
}

UcxCudaMemoryResourceManager::~UcxCudaMemoryResourceManager() {
  release_imports();
  std::lock_guard lk(mu_);
  DeviceGuard on_device(opt_.device);
  for (auto& a : arenas_) cudaFree(a.base);
  for (auto& [p, n] : dedicated_) cudaFree(p);
  for (auto& [n, p] : large_idle_) cudaFree(p);
}

void* UcxCudaMemoryResourceManager::pool_alloc(size_t bytes) {
  bytes = round_up(bytes ? bytes : 1, kGranule);
  std::lock_guard lk(mu_);
  DeviceGuard on_device(opt_.device);
  if (bytes > opt_.arena_bytes / 2) {
    bytes = round_up(bytes, size_t(2) << 20);
    // an idle block of at most twice the size serves the request
    if (auto it = large_idle_.lower_bound(bytes); it != large_idle_.end() && it->first <= 2 * bytes) {
      void* p = it->second;
      dedicated_[p] = it->first;
      large_idle_bytes_ -= it->first;
      large_idle_.erase(it);
      return p;
    }
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
      cudaGetLastError();
      // give the idle blocks back and try once more
      for (auto& [n, q] : large_idle_) {
        regs_.erase(reinterpret_cast<uintptr_t>(q));
        cudaFree(q);
      }
      large_idle_.clear();
      large_idle_bytes_ = 0;
      if (cudaMalloc(&p, bytes) != cudaSuccess) throw std::bad_alloc();
    }
    dedicated_[p] = bytes;
    return p;
  }
  for (int pass = 0; pass < 2; ++pass) {
    for (auto& a : arenas_) {
      for (auto it = a.free_by_off.begin(); it != a.free_by_off.end(); ++it) {
        if (it->second < bytes) continue;
        size_t off = it->first, len = it->second;
        a.free_by_off.erase(it);
        if (len > bytes) a.free_by_off[off + bytes] = len - bytes;
        a.in_use += bytes;
        return a.base + off;
      }
    }
    Arena a;
    void* p = nullptr;
    if (cudaMalloc(&p, opt_.arena_bytes) != cudaSuccess) throw std::bad_alloc();
    a.base = static_cast<char*>(p);
    a.size = opt_.arena_bytes;
    a.free_by_off[0] = a.size;
    arenas_.push_back(std::move(a));
  }
  throw std::bad_alloc();
}

bool UcxCudaMemoryResourceManager::pool_free(void* p, size_t bytes) {
  std::lock_guard lk(mu_);
  DeviceGuard on_device(opt_.device);
  if (auto it = dedicated_.find(p); it != dedicated_.end()) {
    const size_t n = it->second;
    dedicated_.erase(it);
    if (large_idle_bytes_ + n <= opt_.large_cache_bytes) {
      large_idle_.emplace(n, p);  // the registration (and its export handle) stays
      large_idle_bytes_ += n;
    } else {
      regs_.erase(reinterpret_cast<uintptr_t>(p));
      cudaFree(p);
    }
    return true;
  }
  bytes = round_up(bytes ? bytes : 1, kGranule);
  for (auto& a : arenas_) {
    char* c = static_cast<char*>(p);
    if (c < a.base || c >= a.base + a.size) continue;
    size_t off = static_cast<size_t>(c - a.base);
    auto [it, ok] = a.free_by_off.emplace(off, bytes);
    if (!ok) return false;  // double free
    a.in_use -= bytes;
    auto next = std::next(it);
    if (next != a.free_by_off.end() && it->first + it->second == next->first) {
      it->second += next->second;
      a.free_by_off.erase(next);
    }
    if (it != a.free_by_off.begin()) {
      auto prev = std::prev(it);
      if (prev->first + prev->second == it->first) {
        prev->second += it->second;
        a.free_by_off.erase(it);
      }
    }
    return true;
  }
  return false;
}

void* UcxCudaMemoryResourceManager::allocate(ucx_memory_type_t type, size_t bytes, size_t alignment) {
  switch (type) {
    case ucx_memory_type::CUDA: return pool_alloc(bytes);
    case ucx_memory_type::CUDA_MANAGED: {
      DeviceGuard on_device(opt_.device);
      void* p = nullptr;
      if (cudaMallocManaged(&p, bytes ? bytes : 1) != cudaSuccess) throw std::bad_alloc();
      return p;
    }
    default: {
      auto* r = get_memory_resource(type);
      if (!r) throw std::bad_alloc();
      return r->allocate(bytes, alignment);
    }
  }
}

void UcxCudaMemoryResourceManager::deallocate(ucx_memory_type_t type, void* p, size_t bytes, size_t alignment) {
  if (!p) return;
  switch (type) {
    case ucx_memory_type::CUDA:
      if (!pool_free(p, bytes)) throw std::invalid_argument("pointer does not belong to the CUDA pool");
      return;
    case ucx_memory_type::CUDA_MANAGED: cudaFree(p); return;
    default: {
      auto* r = get_memory_resource(type);
      if (!r) throw std::invalid_argument("no memory resource registered for this memory type");
      r->deallocate(p, bytes, alignment);
    }
  }
}

void* UcxCudaMemoryResourceManager::memcpy(ucx_memory_type_t dest_type, void* dest, ucx_memory_type_t src_type,
                                           const void* src, size_t count) {
  auto fn = get_memcpy_fn(dest_type, src_type);
  if (!fn) throw std::invalid_argument("no memcpy function registered for this pair of memory types");
  return fn(dest, src, count);
}

const UcxCudaMemoryResourceManager::Registration* UcxCudaMemoryResourceManager::find_registration(const void* ptr) const {
  std::lock_guard lk(mu_);
  auto key = reinterpret_cast<uintptr_t>(ptr);
  auto it = regs_.upper_bound(key);
  if (it == regs_.begin()) return nullptr;
  --it;
  if (key >= it->first && key < it->first + it->second.size) return &it->second;
  return nullptr;
}

bool UcxCudaMemoryResourceManager::is_pool_base(const void* base) const {
  for (auto& a : arenas_)
    if (a.base == base) return true;
  if (dedicated_.count(const_cast<void*>(base))) return true;
  for (auto& [n, p] : large_idle_)
    if (p == base) return true;
  return false;
}

const UcxCudaMemoryResourceManager::Registration* UcxCudaMemoryResourceManager::register_memory(const void* ptr, size_t) {
  if (auto* r = find_registration(ptr)) {
    bool ours;
    {
      std::lock_guard lk(mu_);
      ours = is_pool_base(r->base);
    }
    if (ours) return r;
    // Memory of somebody else's allocator (a tensor library's cache, say) can be freed and handed
    // out again at the same address: the remembered range and handle are checked against the
    // allocation that is there now.
    uint64_t id = 0;
    if (r->buffer_id && buffer_id_of(ptr, &id) && id == r->buffer_id) return r;  // the very allocation that was registered
    void* base = nullptr;
    size_t size = 0;
    if (r->kind == kRegionVmm) {
      // no handle to compare: without the driver's id to go by, register it again under a new number
    } else if (address_range(ptr, &base, &size) && base == r->base && size == r->size) {
      cudaIpcMemHandle_t h;
      if (cudaIpcGetMemHandle(&h, base) == cudaSuccess) {
        if (std::memcmp(&h, r->handle, 64) == 0 && r->exportable) return r;
      } else {
        cudaGetLastError();
        if (!r->exportable) return r;
      }
    }
    unregister_memory(r->base);
  }
  void* base = nullptr;
  size_t size = 0;
  if (!address_range(ptr, &base, &size)) return nullptr;
  Registration reg;
  reg.base = base;
  reg.size = size;
  cudaPointerAttributes attr{};
  reg.device = cudaPointerGetAttributes(&attr, ptr) == cudaSuccess ? attr.device : opt_.device;
  if (!buffer_id_of(base, &reg.buffer_id)) reg.buffer_id = 0;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, base) == cudaSuccess) {
    static_assert(sizeof(h) == 64);
    std::memcpy(reg.handle, &h, 64);
    reg.exportable = true;
  } else {
    cudaGetLastError();  // clear; the region can still be used inside this process
    // Not a cudaMalloc allocation. If it is a cuMemCreate allocation that was made shareable as a file
    // descriptor, that is how it travels (a trial export tells; the descriptor itself is made per peer).
    const VmmApi& api = vmm_api();
    CUmemGenericAllocationHandle h = 0;
    if (api.ok && api.retain(&h, base) == CUDA_SUCCESS) {
      int fd = -1;
      if (api.export_handle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) == CUDA_SUCCESS && fd >= 0) {
        ::close(fd);
        reg.kind = kRegionVmm;
        reg.vmm_id = g_next_vmm_id.fetch_add(1);
        reg.exportable = true;
      }
      api.release(h);
    }
  }
  std::lock_guard lk(mu_);
  auto [it, ok] = regs_.emplace(reinterpret_cast<uintptr_t>(base), reg);
  return &it->second;
}

bool UcxCudaMemoryResourceManager::unregister_memory(const void* ptr) {
  std::lock_guard lk(mu_);
  auto key = reinterpret_cast<uintptr_t>(ptr);
  auto it = regs_.upper_bound(key);
  if (it == regs_.begin()) return false;
  --it;
  if (key < it->first || key >= it->first + it->second.size) return false;
  regs_.erase(it);
  return true;
}

bool UcxCudaMemoryResourceManager::export_region(const void* ptr, size_t len, PeerRegionDesc* out) {
  const Registration* r = register_memory(ptr, len);
  if (!r) return false;
  auto p = reinterpret_cast<uintptr_t>(ptr), b = reinterpret_cast<uintptr_t>(r->base);
  if (p + len > b + r->size) return false;
  out->pid = static_cast<uint32_t>(getpid());
  out->device = r->device;
  out->base = b;
  out->offset = p - b;
  out->length = len;
  out->exportable = r->exportable;
  out->kind = r->kind;
  if (r->kind == kRegionVmm) {
    PeerVmmRef ref{r->vmm_id, r->size};
    std::memset(out->handle, 0, 64);
    std::memcpy(out->handle, &ref, sizeof(ref));
  } else {
    std::memcpy(out->handle, r->handle, 64);
  }
  return true;
}

bool UcxCudaMemoryResourceManager::export_regions(const void* ptr, size_t len, std::vector<PeerRegionDesc>* out) {
  const size_t before = out->size();
  const char* p = static_cast<const char*>(ptr);
  size_t left = len;
  do {
    const Registration* r = register_memory(p, left);
    if (!r) {
      out->resize(before);
      return false;
    }
    const auto a = reinterpret_cast<uintptr_t>(p), b = reinterpret_cast<uintptr_t>(r->base);
    const size_t here = std::min<size_t>(left, b + r->size - a);
    PeerRegionDesc d;
    if (!export_region(p, here, &d)) {
      out->resize(before);
      return false;
    }
    out->push_back(d);
    p += here;
    left -= here;
  } while (left > 0);
  return true;
}

int UcxCudaMemoryResourceManager::export_vmm_fd(const PeerRegionDesc& d) {
  const VmmApi& api = vmm_api();
  if (!api.ok || d.kind != kRegionVmm || d.pid != static_cast<uint32_t>(getpid())) return -1;
  PeerVmmRef ref;
  std::memcpy(&ref, d.handle, sizeof(ref));
  const Registration* r = find_registration(reinterpret_cast<const void*>(d.base));
  if (!r || r->kind != kRegionVmm || r->vmm_id != ref.id) return -1;
  CUmemGenericAllocationHandle h = 0;
  if (api.retain(&h, r->base) != CUDA_SUCCESS) return -1;
  int fd = -1;
  if (api.export_handle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS) fd = -1;
  api.release(h);
  return fd;
}

bool UcxCudaMemoryResourceManager::import_vmm(uint64_t owner, const PeerVmmRef& ref, int fd) {
  const VmmApi& api = vmm_api();
  if (!api.ok || fd < 0 || ref.size == 0 || ref.size > (uint64_t(1) << 40)) return false;
  std::lock_guard lk(mu_);
  auto key = std::make_pair(owner, ref.id);
  if (vmm_imports_.count(key)) return true;
  DeviceGuard on_device(opt_.device);
  cudaFree(nullptr);  // the calls below want a current context on this thread
  VmmImported m;
  m.size = ref.size;
  CUmemGenericAllocationHandle h = 0;
  if (api.import_handle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS) return false;
  m.handle = h;
  CUdeviceptr va = 0;
  if (api.reserve(&va, ref.size, 0, 0, 0) != CUDA_SUCCESS) {
    api.release(h);
    return false;
  }
  // a size that is not the allocation's own (a peer that lies about it) fails here, not in a kernel
  if (api.map(va, ref.size, 0, h, 0) != CUDA_SUCCESS) {
    api.address_free(va, ref.size);
    api.release(h);
    return false;
  }
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = opt_.device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (api.set_access(va, ref.size, &acc, 1) != CUDA_SUCCESS) {
    api.unmap(va, ref.size);
    api.address_free(va, ref.size);
    api.release(h);
    return false;
  }
  m.va = va;
  vmm_imports_.emplace(key, m);
  return true;
}

void UcxCudaMemoryResourceManager::unmap_vmm(VmmImported& m) {
  const VmmApi& api = vmm_api();
  if (!api.ok || !m.va) return;
  api.unmap(m.va, m.size);
  api.address_free(m.va, m.size);
  api.release(m.handle);
  m.va = 0;
}

void UcxCudaMemoryResourceManager::release_vmm(uint64_t owner, uint64_t id) {
  std::lock_guard lk(mu_);
  auto it = vmm_imports_.find({owner, id});
  if (it == vmm_imports_.end()) return;
  DeviceGuard on_device(opt_.device);
  unmap_vmm(it->second);
  vmm_imports_.erase(it);
}

void UcxCudaMemoryResourceManager::release_vmm_of(uint64_t owner) {
  std::lock_guard lk(mu_);
  DeviceGuard on_device(opt_.device);
  for (auto it = vmm_imports_.lower_bound({owner, 0}); it != vmm_imports_.end() && it->first.first == owner;) {
    unmap_vmm(it->second);
    it = vmm_imports_.erase(it);
  }
}

namespace {
// [p, p+len) lies inside one allocation known to the driver in this process
bool range_is_mapped(const void* p, uint64_t len) {
  void* base = nullptr;
  size_t size = 0;
  if (!p || !address_range(p, &base, &size)) return false;
  const auto a = reinterpret_cast<uintptr_t>(p), b = reinterpret_cast<uintptr_t>(base);
  return a >= b && len <= size && a - b <= size - len;
}
}  // namespace

void* UcxCudaMemoryResourceManager::import_region(const PeerRegionDesc& d, bool same_process, uint64_t owner) {
  if (d.offset + d.length < d.offset) return nullptr;  // wraps
  if (same_process) {
    if (d.device != opt_.device) {
      int can = 0;
      if (cudaDeviceCanAccessPeer(&can, opt_.device, d.device) != cudaSuccess || !can) return nullptr;
      DeviceGuard on_device(opt_.device);
      cudaError_t e = cudaDeviceEnablePeerAccess(d.device, 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return nullptr;
      cudaGetLastError();
    }
    void* p = reinterpret_cast<void*>(d.base + d.offset);
    if (!range_is_mapped(p, d.length)) {
      cudaGetLastError();
      return nullptr;  // not (or no longer) an allocation of this process: the caller stages through the host
    }
    return p;
  }
  // A descriptor that names this process's pid without the caller vouching for it comes from another
  // pid namespace or host (or is forged): its addresses mean nothing here. The IPC handle decides.
  if (!d.exportable) return nullptr;
  if (d.kind == kRegionVmm) {
    PeerVmmRef ref;
    std::memcpy(&ref, d.handle, sizeof(ref));
    std::lock_guard lk(mu_);
    auto it = vmm_imports_.find({owner, ref.id});
    if (it == vmm_imports_.end()) return nullptr;  // its file descriptor never arrived
    if (d.length > it->second.size || d.offset > it->second.size - d.length) return nullptr;
    return reinterpret_cast<void*>(it->second.va + d.offset);
  }
  if (d.kind != kRegionIpc) return nullptr;
  std::lock_guard lk(mu_);
  DeviceGuard on_device(opt_.device);
  ImportKey key{d.pid, d.base};
  auto it = imports_.find(key);
  if (it != imports_.end() && std::memcmp(it->second.handle, d.handle, 64) != 0) {
    // the peer's allocation at this address is no longer the one that was mapped
    cudaIpcCloseMemHandle(it->second.mapped);
    imports_.erase(it);
    it = imports_.end();
  }
  if (it == imports_.end()) {
    cudaIpcMemHandle_t h;
    std::memcpy(&h, d.handle, 64);
    Imported imp;
    if (cudaIpcOpenMemHandle(&imp.mapped, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    std::memcpy(imp.handle, d.handle, 64);
    it = imports_.emplace(key, imp).first;
  }
  char* p = static_cast<char*>(it->second.mapped) + d.offset;
  if (!range_is_mapped(p, d.length)) {
    cudaGetLastError();
    return nullptr;  // offset + length reach past the mapped allocation
  }
  return p;
}

void UcxCudaMemoryResourceManager::release_imports() {
  std::lock_guard lk(mu_);
  DeviceGuard on_device(opt_.device);
  for (auto& [k, p] : imports_) cudaIpcCloseMemHandle(p.mapped);
  imports_.clear();
  for (auto& [k, m] : vmm_imports_) unmap_vmm(m);
  vmm_imports_.clear();
}

size_t UcxCudaMemoryResourceManager::pooled_bytes() const {
  std::lock_guard lk(mu_);
  size_t n = 0;
  for (auto& a : arenas_) n += a.size;
  return n;
}
size_t UcxCudaMemoryResourceManager::pooled_bytes_in_use() const {
  std::lock_guard lk(mu_);
  size_t n = 0;
  for (auto& a : arenas_) n += a.in_use;
  return n;
}

}  // namespace eux::ucxx
