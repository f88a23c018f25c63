// Where the payload of a rendezvous message is received: always into host
// memory, or into buffers chosen by a user callable that sees the tensor
// metadata first (e.g. device tensors allocated by the application). Consulted
// only on the rendezvous path; small eager payloads arrive in host memory
// (reference: axon/include/axon/memory_policy.hpp:56-93).
#pragma once

#include <functional>
#include <variant>

#include "eux/rpc/rpc_payload_types.hpp"
#include "eux/rpc/utils/tensor_meta.hpp"

namespace eux::axon {

struct AlwaysOnHostPolicy {};

// ReceivedBufferT(TensorMetaSpan): returns the buffer(s) to receive into.
template <class ReceivedBufferT>
using BufferProvider = std::function<ReceivedBufferT(rpc::utils::TensorMetaSpan)>;
template <class ReceivedBufferT>
using CustomMemoryPolicy = BufferProvider<ReceivedBufferT>;
template <class ReceivedBufferT>
using ReceiverMemoryPolicy = std::variant<AlwaysOnHostPolicy, CustomMemoryPolicy<ReceivedBufferT>>;

template <class T, class ReceivedBufferT>
inline constexpr bool is_receiver_memory_policy_v =
    std::is_same_v<std::decay_t<ReceivedBufferT>, std::monostate> || std::is_same_v<std::decay_t<T>, AlwaysOnHostPolicy> ||
    std::is_same_v<std::decay_t<T>, CustomMemoryPolicy<ReceivedBufferT>> ||
    std::is_same_v<std::decay_t<T>, ReceiverMemoryPolicy<ReceivedBufferT>>;

}  // namespace eux::axon
