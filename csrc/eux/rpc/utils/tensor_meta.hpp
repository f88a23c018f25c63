// TensorMeta: the part of a DLPack tensor that travels in an RPC header
// (device, rank, dtype, byte offset, shape, strides); the bytes travel as the
// message payload (reference: rpc_core/utils/tensor_meta.hpp:32-104).
#pragma once

#include <cstdint>
#include <functional>
#include <span>
#include <stdexcept>
#include <vector>

#include "eux/dlpack.h"
#include "eux/rpc/data.hpp"

namespace eux::rpc::utils {

struct TensorMeta {
  TensorMeta() = default;
  explicit TensorMeta(const DLTensor& source)
      : device(source.device), ndim(source.ndim), dtype(source.dtype), byte_offset(source.byte_offset) {
    if (source.ndim > 0) {
      if (!source.shape) throw std::runtime_error("TensorMeta: the DLTensor has dimensions but no shape");
      shape.assign(source.shape, source.shape + source.ndim);
      if (source.strides) {
        strides.assign(source.strides, source.strides + source.ndim);
      } else {  // DLPack: null strides mean a compact row-major tensor
        strides.resize(source.ndim);
        int64_t s = 1;
        for (int i = source.ndim - 1; i >= 0; --i) {
          strides[i] = s;
          s *= source.shape[i];
        }
      }
    }
  }
  bool is_compact() const {
    if (ndim < 0 || size_t(ndim) > shape.size() || size_t(ndim) > strides.size()) return false;
    for (int i = 0; i < ndim; ++i)
      if (shape[i] == 0) return true;  // no elements: any strides describe the same (empty) bytes
    int64_t s = 1;
    for (int i = ndim - 1; i >= 0; --i) {
      if (shape[i] != 1 && strides[i] != s) return false;
      s *= shape[i];
    }
    return true;
  }
  friend bool operator==(const TensorMeta& a, const TensorMeta& b) {
    return a.device.device_type == b.device.device_type && a.device.device_id == b.device.device_id && a.ndim == b.ndim &&
           a.dtype.code == b.dtype.code && a.dtype.bits == b.dtype.bits && a.dtype.lanes == b.dtype.lanes &&
           a.byte_offset == b.byte_offset && a.shape == b.shape && a.strides == b.strides;
  }

  DLDevice device{kDLCPU, 0};
  int32_t ndim = 0;
  DLDataType dtype{kDLUInt, 8, 1};
  uint64_t byte_offset = 0;
  data::vector<int64_t> shape;
  data::vector<int64_t> strides;
};

using TensorMetaRef = std::reference_wrapper<const TensorMeta>;
using TensorMetaRefVec = std::vector<TensorMetaRef>;
using TensorMetaSpan = std::span<const TensorMeta>;

// Bytes of the dense tensor the metadata describes: prod(shape) * ceil(bits/8).
// Rank-0 metadata counts as empty, like the reference (tensor_meta.hpp:91-104).
// A description that is no tensor (rank and shape disagree, a negative extent, a byte count beyond size_t)
// counts as the largest size there is, so that every "does it fit" check of a caller fails for it.
inline size_t CalculateTensorSize(const TensorMeta& meta) {
  if (meta.ndim == 0) return 0;
  constexpr size_t kInvalid = static_cast<size_t>(-1);
  if (meta.ndim < 0 || static_cast<size_t>(meta.ndim) > meta.shape.size()) return kInvalid;
  size_t n = 1;
  for (int32_t i = 0; i < meta.ndim; ++i) {
    if (meta.shape[i] < 0 || __builtin_mul_overflow(n, static_cast<size_t>(meta.shape[i]), &n)) return kInvalid;
  }
  const size_t elem = (size_t(meta.dtype.bits) * (meta.dtype.lanes ? meta.dtype.lanes : 1) + 7) / 8;
  size_t bytes = 0;
  if (__builtin_mul_overflow(n, elem, &bytes)) return kInvalid;
  return bytes;
}

// Bytes a tensor of this description takes in a payload. The same as CalculateTensorSize, except that a
// rank-0 tensor is one element there (the senders put the element on the wire, so the receivers must make
// room for it).
inline size_t TensorPayloadBytes(const TensorMeta& meta) {
  if (meta.ndim == 0) return (size_t(meta.dtype.bits) * (meta.dtype.lanes ? meta.dtype.lanes : 1) + 7) / 8;
  return CalculateTensorSize(meta);
}

}  // namespace eux::rpc::utils
