#include "eux/ucxx/ucx_memory_resource.hpp"

#include <cstring>
#include <new>
#include <stdexcept>

namespace eux::ucxx {

size_t UcxMemoryResourceManager::index_of(ucx_memory_type_t t) {
  auto i = static_cast<size_t>(t);
  if (i >= UCX_MEMORY_TYPE_COUNT) throw std::out_of_range("unknown ucx_memory_type");
  return i;
}

void UcxMemoryResourceManager::register_memory_resource(ucx_memory_type_t type,
                                                        std::reference_wrapper<std::pmr::memory_resource> resource) {
  memory_resources_[index_of(type)] = resource;
}

void UcxMemoryResourceManager::register_memcpy_fn(ucx_memory_type_t dest_type, ucx_memory_type_t src_type,
                                                  memcpy_fn_t memcpy_fn) {
  memcpy_fns_[index_of(src_type)][index_of(dest_type)] = std::move(memcpy_fn);
}

std::pmr::memory_resource* UcxMemoryResourceManager::get_memory_resource(ucx_memory_type_t type) const {
  const auto& r = memory_resources_[index_of(type)];
  return r ? &r->get() : nullptr;
}

UcxMemoryResourceManager::memcpy_fn_t UcxMemoryResourceManager::get_memcpy_fn(ucx_memory_type_t dest_type,
                                                                              ucx_memory_type_t src_type) const {
  return memcpy_fns_[index_of(src_type)][index_of(dest_type)];
}

DefaultUcxMemoryResourceManager::DefaultUcxMemoryResourceManager() {
  register_memory_resource(ucx_memory_type::HOST, *std::pmr::new_delete_resource());
  register_memcpy_fn(ucx_memory_type::HOST, ucx_memory_type::HOST,
                     [](void* d, const void* s, size_t n) { return std::memcpy(d, s, n); });
}

void* DefaultUcxMemoryResourceManager::allocate(ucx_memory_type_t type, size_t bytes, size_t alignment) {
  auto* r = get_memory_resource(type);
  if (!r) throw std::bad_alloc();
  return r->allocate(bytes, alignment);
}

void DefaultUcxMemoryResourceManager::deallocate(ucx_memory_type_t type, void* p, size_t bytes, size_t alignment) {
  if (!p) return;
  auto* r = get_memory_resource(type);
  if (!r) throw std::invalid_argument("no memory resource registered for this memory type");
  r->deallocate(p, bytes, alignment);
}

void* DefaultUcxMemoryResourceManager::memcpy(ucx_memory_type_t dest_type, void* dest, ucx_memory_type_t src_type,
                                              const void* src, size_t count) {
  auto fn = get_memcpy_fn(dest_type, src_type);
  if (!fn) throw std::invalid_argument("no memcpy function registered for this pair of memory types");
  return fn(dest, src, count);
}

}  // namespace eux::ucxx
