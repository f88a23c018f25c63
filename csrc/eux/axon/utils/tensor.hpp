// TensorBase: a DLTensor that owns its shape/strides arrays, built from wire
// metadata plus a data pointer; Tensor<T> adds an element-type tag
// (reference: axon/include/axon/utils/tensor.hpp:42-225).
#pragma once

#include <cstdint>
#include <stdexcept>
#include <vector>

#include "eux/dlpack.h"
#include "eux/rpc/utils/tensor_meta.hpp"

namespace eux::axon::utils {

class TensorBase : public DLTensor {
 public:
  TensorBase() : DLTensor{} {}
  TensorBase(void* data_ptr, const rpc::utils::TensorMeta& meta) : DLTensor{} { assign(data_ptr, meta); }
  explicit TensorBase(const DLTensor& t) : DLTensor(t) {
    if (t.ndim > 0) {
      shape_.assign(t.shape, t.shape + t.ndim);
      if (t.strides) strides_.assign(t.strides, t.strides + t.ndim);
    }
    rebind();
  }
  TensorBase(const TensorBase& o) : DLTensor(o), shape_(o.shape_), strides_(o.strides_) { rebind(); }
  TensorBase(TensorBase&& o) noexcept : DLTensor(o), shape_(std::move(o.shape_)), strides_(std::move(o.strides_)) {
    rebind();
    o.data = nullptr;
    o.shape = o.strides = nullptr;
    o.ndim = 0;
  }
  TensorBase& operator=(TensorBase o) noexcept {
    static_cast<DLTensor&>(*this) = o;
    shape_ = std::move(o.shape_);
    strides_ = std::move(o.strides_);
    rebind();
    return *this;
  }
  void assign(void* data_ptr, const rpc::utils::TensorMeta& meta) {
    data = data_ptr;
    device = meta.device;
    ndim = meta.ndim;
    dtype = meta.dtype;
    byte_offset = meta.byte_offset;
    shape_.assign(meta.shape.begin(), meta.shape.end());
    strides_.assign(meta.strides.begin(), meta.strides.end());
    rebind();
  }
  rpc::utils::TensorMeta meta() const { return rpc::utils::TensorMeta(static_cast<const DLTensor&>(*this)); }
  size_t nbytes() const { return rpc::utils::CalculateTensorSize(meta()); }
  int64_t numel() const {
    int64_t n = 1;
    for (auto s : shape_) n *= s;
    return ndim == 0 ? 0 : n;
  }

 private:
  void rebind() {
    shape = shape_.empty() ? nullptr : shape_.data();
    strides = strides_.empty() ? nullptr : strides_.data();
  }
  std::vector<int64_t> shape_;
  std::vector<int64_t> strides_;
};

// T = void: untyped. Otherwise construction checks that the dtype holds T-sized elements.
template <class T = void>
class Tensor : public TensorBase {
 public:
  using TensorBase::TensorBase;
  Tensor(void* data_ptr, const rpc::utils::TensorMeta& meta) : TensorBase(data_ptr, meta) {
    if constexpr (!std::is_void_v<T>) {
      if (meta.dtype.bits * (meta.dtype.lanes ? meta.dtype.lanes : 1) != sizeof(T) * 8)
        throw std::invalid_argument("Tensor<T>: element size differs from the metadata's dtype");
    }
  }
  auto* typed_data() const {
    using E = std::conditional_t<std::is_void_v<T>, unsigned char, T>;
    return reinterpret_cast<E*>(static_cast<char*>(data) + byte_offset);
  }
};

}  // namespace eux::axon::utils
