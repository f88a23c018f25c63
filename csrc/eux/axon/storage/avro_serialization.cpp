#include "eux/axon/storage/avro_serialization.hpp"

#include "eux/axon/storage/avro_schema.hpp"

namespace eux::axon::storage {

using rpc::ParamMeta;
using rpc::ParamType;
using rpc::TensorMeta;

namespace {

void put_tensor_meta(avro::Encoder& e, const TensorMeta& m) {
  e.put_int(static_cast<int32_t>(m.device.device_type));
  e.put_int(m.device.device_id);
  e.put_int(m.ndim);
  e.put_int(m.dtype.code);
  e.put_int(m.dtype.bits);
  e.put_int(m.dtype.lanes);
  e.put_long(static_cast<int64_t>(m.byte_offset));
  e.array_start(m.shape.size());
  for (auto v : m.shape) e.put_long(v);
  e.array_end();
  e.array_start(m.strides.size());
  for (auto v : m.strides) e.put_long(v);
  e.array_end();
}
void get_tensor_meta(avro::Decoder& d, TensorMeta& m) {
  m.device.device_type = static_cast<DLDeviceType>(d.get_int());
  m.device.device_id = d.get_int();
  m.ndim = d.get_int();
  m.dtype.code = static_cast<uint8_t>(d.get_int());
  m.dtype.bits = static_cast<uint8_t>(d.get_int());
  m.dtype.lanes = static_cast<uint16_t>(d.get_int());
  m.byte_offset = static_cast<uint64_t>(d.get_long());
  m.shape.clear();
  while (size_t n = d.next_block())
    for (size_t i = 0; i < n; ++i) m.shape.push_back(d.get_long());
  m.strides.clear();
  while (size_t n = d.next_block())
    for (size_t i = 0; i < n; ++i) m.strides.push_back(d.get_long());
}

void put_param(avro::Encoder& e, const ParamMeta& p) {
  e.put_int(static_cast<int32_t>(p.type));
  std::visit(
      [&](const auto& alt) {
        using A = std::decay_t<decltype(alt)>;
        if constexpr (std::is_same_v<A, rpc::PrimitiveValue>) {
          std::visit(
              [&](auto x) {
                using X = decltype(x);
                if constexpr (std::is_same_v<X, bool>) {
                  e.put_union(AvroSchema::kBoolean);
                  e.put_bool(x);
                } else if constexpr (std::is_same_v<X, float>) {
                  e.put_union(AvroSchema::kFloat);
                  e.put_float(x);
                } else if constexpr (std::is_same_v<X, double>) {
                  e.put_union(AvroSchema::kDouble);
                  e.put_double(x);
                } else if constexpr (sizeof(X) == 8) {
                  e.put_union(AvroSchema::kLong);
                  e.put_long(static_cast<int64_t>(x));
                } else if constexpr (std::is_same_v<X, uint32_t>) {  // does not fit Avro's int
                  e.put_union(AvroSchema::kLong);
                  e.put_long(static_cast<int64_t>(x));
                } else {
                  e.put_union(AvroSchema::kInt);
                  e.put_int(static_cast<int32_t>(x));
                }
              },
              alt);
        } else if constexpr (std::is_same_v<A, rpc::VectorValue>) {
          std::visit(
              [&](const auto& vec) {
                using E = typename std::decay_t<decltype(vec)>::value_type;
                if constexpr (std::is_same_v<E, rpc::data::bool_t>) {
                  e.put_union(AvroSchema::kBooleanArray);
                  e.array_start(vec.size());
                  for (auto x : vec) e.put_bool(x);
                } else if constexpr (std::is_same_v<E, float>) {
                  e.put_union(AvroSchema::kFloatArray);
                  e.array_start(vec.size());
                  for (auto x : vec) e.put_float(x);
                } else if constexpr (std::is_same_v<E, double>) {
                  e.put_union(AvroSchema::kDoubleArray);
                  e.array_start(vec.size());
                  for (auto x : vec) e.put_double(x);
                } else if constexpr (sizeof(E) == 8 || std::is_same_v<E, uint32_t>) {
                  e.put_union(AvroSchema::kLongArray);
                  e.array_start(vec.size());
                  for (auto x : vec) e.put_long(static_cast<int64_t>(x));
                } else {
                  e.put_union(AvroSchema::kIntArray);
                  e.array_start(vec.size());
                  for (auto x : vec) e.put_int(static_cast<int32_t>(x));
                }
                e.array_end();
              },
              alt);
        } else if constexpr (std::is_same_v<A, rpc::data::string>) {
          e.put_union(AvroSchema::kString);
          e.put_string(alt.view());
        } else if constexpr (std::is_same_v<A, std::nullptr_t>) {
          e.put_union(AvroSchema::kNull);
        } else if constexpr (std::is_same_v<A, TensorMeta>) {
          e.put_union(AvroSchema::kTensorMeta);
          put_tensor_meta(e, alt);
        } else {
          e.put_union(AvroSchema::kTensorMetaVec);
          e.array_start(alt.size());
          for (auto& m : alt) put_tensor_meta(e, m);
          e.array_end();
        }
      },
      p.value);
  e.put_string(p.name.view());
}

template <class T, class Get>
rpc::data::vector<T> get_array(avro::Decoder& d, Get get) {
  rpc::data::vector<T> out;
  while (size_t n = d.next_block())
    for (size_t i = 0; i < n; ++i) out.push_back(static_cast<std::conditional_t<std::is_same_v<T, bool>, rpc::data::bool_t, T>>(get()));
  return out;
}

// the stored ParamType says which C++ type the Avro branch value had
template <class T>
rpc::ParamValue prim(T v) {
  return rpc::ParamValue(std::in_place_type<rpc::PrimitiveValue>, rpc::PrimitiveValue(std::in_place_type<T>, v));
}
template <class T>
rpc::ParamValue vecval(rpc::data::vector<T>&& v) {
  return rpc::ParamValue(std::in_place_type<rpc::VectorValue>, rpc::VectorValue(std::in_place_type<rpc::data::vector<T>>, std::move(v)));
}

void get_param(avro::Decoder& d, ParamMeta& p) {
  p.type = static_cast<ParamType>(d.get_int());
  const int branch = d.get_union();
  switch (branch) {
    case AvroSchema::kNull: p.value = rpc::ParamValue(nullptr); break;
    case AvroSchema::kBoolean: p.value = prim<bool>(d.get_bool()); break;
    case AvroSchema::kInt: {
      int32_t v = d.get_int();
      switch (p.type) {
        case ParamType::PRIMITIVE_INT8: p.value = prim<int8_t>(static_cast<int8_t>(v)); break;
        case ParamType::PRIMITIVE_INT16: p.value = prim<int16_t>(static_cast<int16_t>(v)); break;
        case ParamType::PRIMITIVE_UINT8: p.value = prim<uint8_t>(static_cast<uint8_t>(v)); break;
        case ParamType::PRIMITIVE_UINT16: p.value = prim<uint16_t>(static_cast<uint16_t>(v)); break;
        default: p.value = prim<int32_t>(v); break;
      }
      break;
    }
    case AvroSchema::kLong: {
      int64_t v = d.get_long();
      if (p.type == ParamType::PRIMITIVE_UINT64) p.value = prim<uint64_t>(static_cast<uint64_t>(v));
      else if (p.type == ParamType::PRIMITIVE_UINT32) p.value = prim<uint32_t>(static_cast<uint32_t>(v));
      else p.value = prim<int64_t>(v);
      break;
    }
    case AvroSchema::kFloat: p.value = prim<float>(d.get_float()); break;
    case AvroSchema::kDouble: p.value = prim<double>(d.get_double()); break;
    case AvroSchema::kString: p.value = rpc::ParamValue(std::in_place_type<rpc::data::string>, d.get_string()); break;
    case AvroSchema::kBooleanArray: p.value = vecval<bool>(get_array<bool>(d, [&] { return d.get_bool(); })); break;
    case AvroSchema::kIntArray:
      switch (p.type) {
        case ParamType::VECTOR_INT8: p.value = vecval<int8_t>(get_array<int8_t>(d, [&] { return d.get_int(); })); break;
        case ParamType::VECTOR_INT16: p.value = vecval<int16_t>(get_array<int16_t>(d, [&] { return d.get_int(); })); break;
        case ParamType::VECTOR_UINT8: p.value = vecval<uint8_t>(get_array<uint8_t>(d, [&] { return d.get_int(); })); break;
        case ParamType::VECTOR_UINT16: p.value = vecval<uint16_t>(get_array<uint16_t>(d, [&] { return d.get_int(); })); break;
        default: p.value = vecval<int32_t>(get_array<int32_t>(d, [&] { return d.get_int(); })); break;
      }
      break;
    case AvroSchema::kLongArray:
      if (p.type == ParamType::VECTOR_UINT64) p.value = vecval<uint64_t>(get_array<uint64_t>(d, [&] { return d.get_long(); }));
      else if (p.type == ParamType::VECTOR_UINT32) p.value = vecval<uint32_t>(get_array<uint32_t>(d, [&] { return d.get_long(); }));
      else p.value = vecval<int64_t>(get_array<int64_t>(d, [&] { return d.get_long(); }));
      break;
    case AvroSchema::kFloatArray: p.value = vecval<float>(get_array<float>(d, [&] { return d.get_float(); })); break;
    case AvroSchema::kDoubleArray: p.value = vecval<double>(get_array<double>(d, [&] { return d.get_double(); })); break;
    case AvroSchema::kTensorMeta: {
      TensorMeta m;
      get_tensor_meta(d, m);
      p.value = rpc::ParamValue(std::in_place_type<TensorMeta>, std::move(m));
      break;
    }
    case AvroSchema::kTensorMetaVec: {
      rpc::TensorMetaVec v;
      while (size_t n = d.next_block())
        for (size_t i = 0; i < n; ++i) get_tensor_meta(d, v.emplace_back());
      p.value = rpc::ParamValue(std::in_place_type<rpc::TensorMetaVec>, std::move(v));
      break;
    }
    default: throw std::runtime_error("avro: unknown parameter value branch");
  }
  p.name = rpc::data::string(d.get_string());
}

// payload bytes, staged to host when they live on a device
void put_buffer(avro::Encoder& e, ucxx::UcxMemoryResourceManager& mr, ucx_memory_type_t type, const void* data, size_t size) {
  if (type == ucx_memory_type::HOST || size == 0) {
    e.put_bytes(data, size);
  } else {
    std::vector<uint8_t> host(size);
    mr.memcpy(ucx_memory_type::HOST, host.data(), type, data, size);
    e.put_bytes(host.data(), size);
  }
  e.put_long(static_cast<int64_t>(size));
}

}  // namespace

void AvroSerialization::Serialize(const utils::AxonRequest& req, ucxx::UcxMemoryResourceManager& mr, std::vector<uint8_t>& out) {
  avro::Encoder e(out);
  const auto& h = req.header;
  e.put_int(static_cast<int32_t>(h.function_id.v_));
  e.put_int(static_cast<int32_t>(h.session_id.v_));
  e.put_int(static_cast<int32_t>(h.request_id.v_));
  e.array_start(h.params.size());
  for (auto& p : h.params) put_param(e, p);
  e.array_end();
  e.put_long(static_cast<int64_t>(h.hlc.Raw()));
  e.put_int(static_cast<int32_t>(h.workflow_id.v_));
  if (auto* b = std::get_if<ucxx::UcxBuffer>(&req.payload)) {
    e.put_union(AvroSchema::kBuffer);
    put_buffer(e, mr, b->type(), b->data(), b->size());
  } else if (auto* v = std::get_if<ucxx::UcxBufferVec>(&req.payload)) {
    e.put_union(AvroSchema::kBufferArray);
    e.array_start(v->size());
    for (auto& s : *v) put_buffer(e, mr, v->type(), s.data, s.size);
    e.array_end();
  } else {
    e.put_union(AvroSchema::kNoPayload);
  }
}

std::shared_ptr<utils::AxonRequest> AvroSerialization::Deserialize(avro::Decoder& d, ucxx::UcxMemoryResourceManager& mr) {
  rpc::RpcRequestHeader h;
  h.function_id.v_ = static_cast<uint32_t>(d.get_int());
  h.session_id.v_ = static_cast<uint32_t>(d.get_int());
  h.request_id.v_ = static_cast<uint32_t>(d.get_int());
  while (size_t n = d.next_block())
    for (size_t i = 0; i < n; ++i) get_param(d, h.params.emplace_back());
  h.hlc = rpc::HybridLogicalClock(static_cast<uint64_t>(d.get_long()));
  h.workflow_id.v_ = static_cast<uint32_t>(d.get_int());
  rpc::PayloadVariant payload;
  auto read_buffer = [&](ucxx::UcxBuffer& dst) {
    auto [p, n] = d.get_bytes();
    (void)d.get_long();
    dst = ucxx::UcxBuffer(mr, ucx_memory_type::HOST, n);
    if (n) std::memcpy(dst.data(), p, n);
  };
  switch (d.get_union()) {
    case AvroSchema::kNoPayload: break;
    case AvroSchema::kBuffer: {
      ucxx::UcxBuffer b(mr, ucx_memory_type::HOST, size_t(0));
      read_buffer(b);
      payload = std::move(b);
      break;
    }
    case AvroSchema::kBufferArray: {
      std::vector<ucxx::UcxBuffer> bufs;
      while (size_t n = d.next_block())
        for (size_t i = 0; i < n; ++i) {
          bufs.emplace_back(mr, ucx_memory_type::HOST, size_t(0));
          read_buffer(bufs.back());
        }
      if (bufs.empty()) payload = ucxx::UcxBufferVec(mr, ucx_memory_type::HOST, std::vector<size_t>{});
      else payload = ucxx::UcxBufferVec(std::move(bufs));
      break;
    }
    default: throw std::runtime_error("avro: unknown payload branch");
  }
  return std::make_shared<utils::AxonRequest>(std::move(h), std::move(payload));
}

}  // namespace eux::axon::storage
