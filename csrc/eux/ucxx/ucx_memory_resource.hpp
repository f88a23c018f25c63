// PMR-style memory resource manager: one std::pmr::memory_resource per memory
// kind plus a [dst][src] table of copy functions. Same surface as the
// reference's ucx_context/ucx_memory_resource.hpp:40-188.
#pragma once

#include <array>
#include <cstddef>
#include <functional>
#include <memory_resource>
#include <optional>
#include <type_traits>

#include "eux/ucxx/ucx_context_def.h"

namespace eux::ucxx {

class UcxMemoryResourceManager {
 public:
  using memcpy_fn_t = std::function<void*(void*, const void*, size_t)>;
  static constexpr size_t UCX_MEMORY_TYPE_COUNT = static_cast<size_t>(ucx_memory_type::LAST) + 1;

  UcxMemoryResourceManager() = default;
  virtual ~UcxMemoryResourceManager() = default;

  void register_memory_resource(ucx_memory_type_t type, std::reference_wrapper<std::pmr::memory_resource> resource);
  void register_memcpy_fn(ucx_memory_type_t dest_type, ucx_memory_type_t src_type, memcpy_fn_t memcpy_fn);
  std::pmr::memory_resource* get_memory_resource(ucx_memory_type_t type) const;
  memcpy_fn_t get_memcpy_fn(ucx_memory_type_t dest_type, ucx_memory_type_t src_type) const;

  virtual void* allocate(ucx_memory_type_t type, size_t bytes, size_t alignment = 8) = 0;
  virtual void deallocate(ucx_memory_type_t type, void* p, size_t bytes, size_t alignment = 8) = 0;
  virtual void* memcpy(ucx_memory_type_t dest_type, void* dest, ucx_memory_type_t src_type, const void* src,
                       size_t count) = 0;

 protected:
  static size_t index_of(ucx_memory_type_t t);
  std::array<std::optional<std::reference_wrapper<std::pmr::memory_resource>>, UCX_MEMORY_TYPE_COUNT> memory_resources_;
  std::array<std::array<memcpy_fn_t, UCX_MEMORY_TYPE_COUNT>, UCX_MEMORY_TYPE_COUNT> memcpy_fns_;  // [src][dest]
};

// Host memory through std::pmr::new_delete_resource; any other kind must be
// registered by the user, otherwise allocate() throws std::bad_alloc.
class DefaultUcxMemoryResourceManager : public UcxMemoryResourceManager {
 public:
  DefaultUcxMemoryResourceManager();
  ~DefaultUcxMemoryResourceManager() override = default;
  void* allocate(ucx_memory_type_t type, size_t bytes, size_t alignment = 8) override;
  void deallocate(ucx_memory_type_t type, void* p, size_t bytes, size_t alignment = 8) override;
  void* memcpy(ucx_memory_type_t dest_type, void* dest, ucx_memory_type_t src_type, const void* src,
               size_t count) override;
};

}  // namespace eux::ucxx
