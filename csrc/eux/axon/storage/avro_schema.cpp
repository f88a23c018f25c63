#include "eux/axon/storage/avro_schema.hpp"

namespace eux::axon::storage {

namespace {
// helpers spell repeated shapes once: a record wrapping one array field named "items"
#define EUX_ARR(name, item) "{\"name\":\"" name "\",\"type\":\"record\",\"fields\":[{\"name\":\"items\",\"type\":{\"type\":\"array\",\"items\":" item "}}]}"
constexpr const char kSchema[] =
    "{\"type\":\"record\",\"name\":\"AxonRequest\",\"namespace\":\"eux.axon\",\"fields\":["
    "{\"name\":\"header\",\"type\":{\"type\":\"record\",\"name\":\"RpcRequestHeader\",\"fields\":["
    "{\"name\":\"function_id\",\"type\":\"int\"},{\"name\":\"session_id\",\"type\":\"int\"},{\"name\":\"request_id\",\"type\":\"int\"},"
    "{\"name\":\"params\",\"type\":{\"type\":\"array\",\"items\":{\"type\":\"record\",\"name\":\"ParamMeta\",\"fields\":["
    "{\"name\":\"type\",\"type\":\"int\"},"
    "{\"name\":\"value\",\"type\":[\"null\",\"boolean\",\"int\",\"long\",\"float\",\"double\",\"string\","
    EUX_ARR("BooleanArray", "\"boolean\"") "," EUX_ARR("IntArray", "\"int\"") "," EUX_ARR("LongArray", "\"long\"") ","
    EUX_ARR("FloatArray", "\"float\"") "," EUX_ARR("DoubleArray", "\"double\"") ","
    "{\"name\":\"TensorMeta\",\"type\":\"record\",\"fields\":["
    "{\"name\":\"device\",\"type\":{\"name\":\"DLDevice\",\"type\":\"record\",\"fields\":[{\"name\":\"device_type\",\"type\":\"int\"},{\"name\":\"device_id\",\"type\":\"int\"}]}},"
    "{\"name\":\"ndim\",\"type\":\"int\"},"
    "{\"name\":\"dtype\",\"type\":{\"name\":\"DLDataType\",\"type\":\"record\",\"fields\":[{\"name\":\"code\",\"type\":\"int\"},{\"name\":\"bits\",\"type\":\"int\"},{\"name\":\"lanes\",\"type\":\"int\"}]}},"
    "{\"name\":\"byte_offset\",\"type\":\"long\"},"
    "{\"name\":\"shape\",\"type\":{\"type\":\"array\",\"items\":\"long\"}},{\"name\":\"strides\",\"type\":{\"type\":\"array\",\"items\":\"long\"}}]},"
    EUX_ARR("TensorMetaVec", "\"TensorMeta\"")
    "]},{\"name\":\"name\",\"type\":\"string\"}]}}},"
    "{\"name\":\"hlc\",\"type\":{\"name\":\"HybridLogicalClock\",\"type\":\"record\",\"fields\":[{\"name\":\"raw\",\"type\":\"long\"}]}},"
    "{\"name\":\"workflow_id\",\"type\":\"int\"}]}},"
    "{\"name\":\"payload\",\"type\":[\"null\",{\"type\":\"record\",\"name\":\"UcxBuffer\",\"fields\":[{\"name\":\"data\",\"type\":\"bytes\"},{\"name\":\"size\",\"type\":\"long\"}]},"
    "{\"type\":\"array\",\"items\":\"UcxBuffer\"}]}]}";
#undef EUX_ARR
}  // namespace

std::string_view AvroSchema::GetArrivalRequestSchema() { return kSchema; }

}  // namespace eux::axon::storage
