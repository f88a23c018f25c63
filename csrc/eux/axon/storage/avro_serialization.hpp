// AxonRequest <-> Avro record (schema in avro_schema.hpp). Device payloads are
// copied to host through the memory resource manager when saving; loading
// always produces host buffers
// (reference: axon/src/storage/avro_serialization.cpp:230-254, 478-523, 762-807).
#pragma once

#include <memory>
#include <vector>

#include "eux/axon/storage/avro_codec.hpp"
#include "eux/axon/utils/axon_message.hpp"

namespace eux::axon::storage {

struct AvroSerialization {
  static void Serialize(const utils::AxonRequest& req, ucxx::UcxMemoryResourceManager& mr, std::vector<uint8_t>& out);
  static std::shared_ptr<utils::AxonRequest> Deserialize(avro::Decoder& d, ucxx::UcxMemoryResourceManager& mr);
};

}  // namespace eux::axon::storage
