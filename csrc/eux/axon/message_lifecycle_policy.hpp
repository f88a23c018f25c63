// What happens to a request after its handler ran: dropped (transient) or shown
// to a user callable that decides to keep it in the worker's storage for later
// re-processing or checkpointing
// (reference: axon/include/axon/message_lifecycle_policy.hpp:32-110).
#pragma once

#include <cstdint>
#include <functional>
#include <memory>
#include <variant>

#include "eux/axon/utils/axon_message.hpp"

namespace eux::axon {

enum class LifecycleStatus : uint8_t { Discard = 0, Preserve, Error };

// LifecycleStatus(request, id): the id is the request's hybrid-logical-clock value.
using LifecycleStatusHandler = std::function<LifecycleStatus(std::shared_ptr<utils::AxonRequest>, utils::AxonMessageID)>;
struct TransientPolicy {};
using RetentionPolicy = LifecycleStatusHandler;
using MessageLifecyclePolicy = std::variant<TransientPolicy, RetentionPolicy>;

template <class T>
inline constexpr bool is_message_lifecycle_policy_v = std::is_same_v<std::decay_t<T>, MessageLifecyclePolicy> ||
                                                      std::is_same_v<std::decay_t<T>, TransientPolicy> ||
                                                      std::is_same_v<std::decay_t<T>, RetentionPolicy>;

}  // namespace eux::axon
