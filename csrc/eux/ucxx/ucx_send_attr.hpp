// What the sender of a device payload may say about it beyond "these bytes":
//   * a layout: the payload is a strided view (a transposed or sliced tensor); the bytes that travel are its
//     elements in row-major order, gathered by the transfer kernel on the way (into the peer's receive ring
//     for a small message, by the receiver's pull for a large one), so the sender makes no dense copy first;
//   * a cast: the elements travel in another floating-point type than they have in memory (fp32 activations
//     as bf16, say), converted by the same kernel on the way; the message's size is that of the converted elements;
//   * an event: the payload is complete once this CUDA event has completed (the producer's kernels may still
//     be running when the send is issued). The transport orders its own kernels after the event on the
//     device and holds back the announcement of a payload that a peer will read until the event is done;
//     the sending thread never waits.
// The reference has neither: its senders hand dense, finished buffers to ucp_am_send_nbx
// (ucx_context/ucx_am_context/ucx_am_context.cpp:915-937) and its Python layer asks for contiguous tensors.
#pragma once

#include <cstdint>
#include <memory>

namespace eux::ucxx {

constexpr int kSendAttrMaxDims = 8;

struct UcxSendAttr {
  // ---- layout (ndim == 0: the payload is dense) ----
  int32_t ndim = 0;
  uint32_t elem_size = 0;                 // 1, 2, 4, 8 or 16 bytes
  int64_t shape[kSendAttrMaxDims] = {0};
  int64_t stride[kSendAttrMaxDims] = {0};  // in elements, none negative: the buffer's address is that of element 0
  uint64_t span_bytes = 0;                // from element 0 to one past the last element touched
  uint64_t dense_bytes = 0;               // the size of the buffer as a message: number of elements * element size on the wire
  // ---- cast (both 0: the elements travel as they are) ----
  uint8_t src_dtype = 0, dst_dtype = 0;   // kernel element types (eux_dtype: 1 fp32, 2 fp16, 3 bf16); elem_size is the source's
  // ---- readiness ----
  void* ready_event = nullptr;            // cudaEvent_t, or null: the payload is complete now
  int device = -1;                        // the device of the event
  std::shared_ptr<void> keep;             // owns the event (and whatever else must live as long as the send)

  uint64_t elements() const {
    uint64_t n = 1;
    for (int i = 0; i < ndim; ++i) n *= static_cast<uint64_t>(shape[i]);
    return n;
  }
  // A layout that a kernel can be handed: sane sizes, no element outside the span.
  bool layout_valid() const {
    if (ndim == 0) return true;
    if (ndim < 0 || ndim > kSendAttrMaxDims) return false;
    if (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8 && elem_size != 16) return false;
    unsigned __int128 last = 0, n = 1;
    for (int i = 0; i < ndim; ++i) {
      if (shape[i] <= 0 || stride[i] < 0) return false;
      last += static_cast<unsigned __int128>(shape[i] - 1) * static_cast<unsigned __int128>(stride[i]);
      n *= static_cast<unsigned __int128>(shape[i]);
      if (n > (static_cast<unsigned __int128>(1) << 48) || last > (static_cast<unsigned __int128>(1) << 48)) return false;
    }
    unsigned wire_size = elem_size;
    if (src_dtype || dst_dtype) {
      auto size_of = [](uint8_t dt) -> unsigned { return dt == 1 ? 4u : (dt == 2 || dt == 3 ? 2u : 0u); };
      if (size_of(src_dtype) != elem_size || size_of(dst_dtype) == 0) return false;
      wire_size = size_of(dst_dtype);
    }
    return (last + 1) * elem_size <= span_bytes && n * wire_size == dense_bytes;
  }
  bool casts() const { return src_dtype != dst_dtype; }
};

}  // namespace eux::ucxx
