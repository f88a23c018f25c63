// Avro schema of a stored request: {header: RpcRequestHeader, payload: null |
// UcxBuffer{bytes data, long size} | array<UcxBuffer>}. Field names, order and
// the union branches of a parameter value are the file-format contract
// (reference: axon/src/storage/avro_schema.cpp:24-176).
#pragma once

#include <string_view>

namespace eux::axon::storage {

struct AvroSchema {
  static std::string_view GetArrivalRequestSchema();
  // branch numbers of the ParamMeta.value union
  enum ValueBranch : int {
    kNull = 0, kBoolean, kInt, kLong, kFloat, kDouble, kString,
    kBooleanArray, kIntArray, kLongArray, kFloatArray, kDoubleArray, kTensorMeta, kTensorMetaVec,
  };
  enum PayloadBranch : int { kNoPayload = 0, kBuffer = 1, kBufferArray = 2 };
};

}  // namespace eux::axon::storage
