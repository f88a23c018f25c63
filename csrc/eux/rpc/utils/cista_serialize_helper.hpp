// Wire serialisation of the RPC types.
//
// The byte image is the one cista produces in "offset" mode with mode::NONE for
// the reference's types (rpc_core/utils/cista_serialize_helper.hpp:32-135): the
// root struct is copied first, then every vector's elements and every long
// string's characters are appended depth-first in member order, and each
// pointer field holds the distance from its own position to its target:
//
//   offset_ptr      int64, target - address_of_field; INT64_MIN = null
//   vector<T>       {offset_ptr el; u32 used; u32 allocated; u8 self_allocated; pad[7]}   24 bytes
//   string          16 bytes: short form {u8 is_short = 1; char s[15]} (NUL padded), or
//                   long form {u8 is_short = 0; u8 self_allocated; u16 fill; u32 size; offset_ptr ptr}
//   variant<T...>   {u8 index (255 = empty); storage at the alternatives' alignment}
//   strong<T>       T
//
// In memory the types are standard containers; this file is the only place that
// knows the image layout, so it can be swapped for cista itself where available.
#pragma once

#include <cstdint>
#include <cstring>
#include <limits>
#include <stdexcept>
#include <string_view>

#include "eux/rpc/rpc_types.hpp"

namespace eux::rpc {

namespace wire {

constexpr int64_t kNullOffset = std::numeric_limits<int64_t>::min();

// image sizes / alignments of the wire types
constexpr size_t kVectorSize = 24, kStringSize = 16;
constexpr size_t kPrimitiveValueSize = 16, kVectorValueSize = 32, kTensorMetaSize = 72;
constexpr size_t kParamValueSize = 80, kParamMetaSize = 104;
constexpr size_t kRequestHeaderSize = 56, kResponseHeaderSize = 72, kStatusSize = 24, kSignatureSize = 96;

// ---- sinks: count bytes, write into a fixed buffer, or grow a byte_buf -------
// All three take absolute positions; `reserve_at_end` appends aligned zeroed space.
class SizeCounter {
 public:
  size_t reserve_at_end(size_t n, size_t align) {
    size_ = (size_ + align - 1) / align * align;
    size_t pos = size_;
    size_ += n;
    return pos;
  }
  void put(size_t, const void*, size_t) {}
  size_t size() const { return size_; }

 private:
  size_t size_ = 0;
};

// the name the reference uses for the counting sink (rpc_core/utils/cista_serialize_helper.hpp:43-78)
using CistaSizeCalculator = SizeCounter;

class FixedBufferWriter {
 public:
  FixedBufferWriter(void* buf, size_t capacity) : buf_(static_cast<uint8_t*>(buf)), cap_(capacity) {}
  size_t reserve_at_end(size_t n, size_t align) {
    size_t start = (size_ + align - 1) / align * align;
    if (start + n > cap_) throw std::length_error("FixedBufferWriter: the buffer is too small for the serialised message");
    std::memset(buf_ + size_, 0, start + n - size_);
    size_ = start + n;
    return start;
  }
  void put(size_t pos, const void* p, size_t n) { std::memcpy(buf_ + pos, p, n); }
  size_t size() const { return size_; }

 private:
  uint8_t* buf_;
  size_t cap_;
  size_t size_ = 0;
};

class BufWriter {
 public:
  explicit BufWriter(byte_buf& b) : buf_(b) { buf_.clear(); }
  size_t reserve_at_end(size_t n, size_t align) {
    size_t start = (buf_.size() + align - 1) / align * align;
    buf_.resize(start + n, 0);
    return start;
  }
  void put(size_t pos, const void* p, size_t n) { std::memcpy(buf_.data() + pos, p, n); }
  size_t size() const { return buf_.size(); }

 private:
  byte_buf& buf_;
};

template <class W, class T>
void put_scalar(W& w, size_t pos, T v) {
  w.put(pos, &v, sizeof(T));
}

// ---- encoders: each writes the fixed part at `pos` (already reserved) and appends children ----
template <class W>
void enc_string(W& w, size_t pos, std::string_view s) {
  // The short form has no length field: a reader takes the bytes up to the first NUL. A short string that
  // holds a NUL (a binary blob carried as a string parameter) is therefore written in the long form, which
  // every reader accepts at any length.
  if (s.size() <= 15 && std::memchr(s.data(), 0, s.size()) == nullptr) {
    uint8_t img[16] = {0};
    img[0] = 1;
    std::memcpy(img + 1, s.data(), s.size());
    w.put(pos, img, 16);
    return;
  }
  size_t start = w.reserve_at_end(s.size(), 1);
  w.put(start, s.data(), s.size());
  put_scalar<W, uint8_t>(w, pos, 0);
  put_scalar<W, uint8_t>(w, pos + 1, 0);
  put_scalar<W, uint16_t>(w, pos + 2, 0);
  put_scalar<W, uint32_t>(w, pos + 4, static_cast<uint32_t>(s.size()));
  put_scalar<W, int64_t>(w, pos + 8, static_cast<int64_t>(start) - static_cast<int64_t>(pos + 8));
}

// vector of trivially copyable elements (scalars, enums, bool_t)
template <class W, class E>
void enc_scalar_vector(W& w, size_t pos, const std::vector<E>& v) {
  int64_t off = kNullOffset;
  if (!v.empty()) {
    size_t start = w.reserve_at_end(sizeof(E) * v.size(), alignof(E));
    w.put(start, v.data(), sizeof(E) * v.size());
    off = static_cast<int64_t>(start) - static_cast<int64_t>(pos);
  }
  put_scalar<W, int64_t>(w, pos, off);
  put_scalar<W, uint32_t>(w, pos + 8, static_cast<uint32_t>(v.size()));
  put_scalar<W, uint32_t>(w, pos + 12, static_cast<uint32_t>(v.size()));
  put_scalar<W, uint8_t>(w, pos + 16, 0);
}

// vector of structured elements: the element array first, then each element's children
template <class W, class E, class Enc>
void enc_struct_vector(W& w, size_t pos, const std::vector<E>& v, size_t elem_size, Enc&& enc_elem) {
  int64_t off = kNullOffset;
  size_t start = 0;
  if (!v.empty()) {
    start = w.reserve_at_end(elem_size * v.size(), 8);
    off = static_cast<int64_t>(start) - static_cast<int64_t>(pos);
  }
  put_scalar<W, int64_t>(w, pos, off);
  put_scalar<W, uint32_t>(w, pos + 8, static_cast<uint32_t>(v.size()));
  put_scalar<W, uint32_t>(w, pos + 12, static_cast<uint32_t>(v.size()));
  put_scalar<W, uint8_t>(w, pos + 16, 0);
  for (size_t i = 0; i < v.size(); ++i) enc_elem(w, start + i * elem_size, v[i]);
}

template <class W>
void enc_tensor_meta(W& w, size_t pos, const TensorMeta& m) {
  put_scalar<W, int32_t>(w, pos, static_cast<int32_t>(m.device.device_type));
  put_scalar<W, int32_t>(w, pos + 4, m.device.device_id);
  put_scalar<W, int32_t>(w, pos + 8, m.ndim);
  put_scalar<W, uint8_t>(w, pos + 12, m.dtype.code);
  put_scalar<W, uint8_t>(w, pos + 13, m.dtype.bits);
  put_scalar<W, uint16_t>(w, pos + 14, m.dtype.lanes);
  put_scalar<W, uint64_t>(w, pos + 16, m.byte_offset);
  enc_scalar_vector(w, pos + 24, m.shape);
  enc_scalar_vector(w, pos + 48, m.strides);
}

template <class W>
void enc_param_value(W& w, size_t pos, const ParamValue& v) {
  put_scalar<W, uint8_t>(w, pos, static_cast<uint8_t>(v.index()));
  const size_t s = pos + 8;  // storage
  switch (v.index()) {
    case 0: {
      const auto& p = std::get<0>(v);
      put_scalar<W, uint8_t>(w, s, static_cast<uint8_t>(p.index()));
      std::visit([&](auto x) { put_scalar(w, s + 8, x); }, p);
      break;
    }
    case 1: {
      const auto& vv = std::get<1>(v);
      put_scalar<W, uint8_t>(w, s, static_cast<uint8_t>(vv.index()));
      std::visit([&](const auto& vec) { enc_scalar_vector(w, s + 8, vec); }, vv);
      break;
    }
    case 2: enc_string(w, s, std::get<2>(v).view()); break;
    case 3: break;  // null: nothing in the storage
    case 4: enc_tensor_meta(w, s, std::get<4>(v)); break;
    case 5: enc_struct_vector(w, s, std::get<5>(v), kTensorMetaSize, [](W& ww, size_t p, const TensorMeta& m) { enc_tensor_meta(ww, p, m); }); break;
  }
}

template <class W>
void enc_param_meta(W& w, size_t pos, const ParamMeta& m) {
  put_scalar<W, uint8_t>(w, pos, static_cast<uint8_t>(m.type));
  enc_param_value(w, pos + 8, m.value);
  enc_string(w, pos + 88, m.name.view());
}

template <class W>
void enc_param_vector(W& w, size_t pos, const data::vector<ParamMeta>& v) {
  enc_struct_vector(w, pos, v, kParamMetaSize, [](W& ww, size_t p, const ParamMeta& m) { enc_param_meta(ww, p, m); });
}

template <class W>
void encode(W& w, const RpcRequestHeader& h) {
  size_t pos = w.reserve_at_end(kRequestHeaderSize, 8);
  put_scalar<W, uint32_t>(w, pos, h.session_id.v_);
  put_scalar<W, uint32_t>(w, pos + 4, h.request_id.v_);
  put_scalar<W, uint32_t>(w, pos + 8, h.function_id.v_);
  put_scalar<W, uint64_t>(w, pos + 16, h.hlc.Raw());
  put_scalar<W, uint32_t>(w, pos + 24, h.workflow_id.v_);
  enc_param_vector(w, pos + 32, h.params);
}

template <class W>
void encode(W& w, const RpcResponseHeader& h) {
  size_t pos = w.reserve_at_end(kResponseHeaderSize, 8);
  put_scalar<W, uint32_t>(w, pos, h.session_id.v_);
  put_scalar<W, uint32_t>(w, pos + 4, h.request_id.v_);
  put_scalar<W, uint64_t>(w, pos + 8, h.hlc.Raw());
  put_scalar<W, uint32_t>(w, pos + 16, h.workflow_id.v_);
  put_scalar<W, int32_t>(w, pos + 24, h.status.value);
  enc_string(w, pos + 32, h.status.category_name.view());
  enc_param_vector(w, pos + 48, h.results);
}

template <class W>
void enc_signature(W& w, size_t pos, const RpcFunctionSignature& s) {
  enc_string(w, pos, s.instance_name.view());
  put_scalar<W, uint32_t>(w, pos + 16, s.id.v_);
  enc_string(w, pos + 24, s.function_name.view());
  enc_scalar_vector(w, pos + 40, s.param_types);
  enc_scalar_vector(w, pos + 64, s.return_types);
  put_scalar<W, uint8_t>(w, pos + 88, static_cast<uint8_t>(s.input_payload_type));
  put_scalar<W, uint8_t>(w, pos + 89, static_cast<uint8_t>(s.return_payload_type));
}

template <class W>
void encode(W& w, const data::vector<RpcFunctionSignature>& sigs) {
  size_t pos = w.reserve_at_end(kVectorSize, 8);
  enc_struct_vector(w, pos, sigs, kSignatureSize, [](W& ww, size_t p, const RpcFunctionSignature& s) { enc_signature(ww, p, s); });
}

// ---- decoder (bounds-checked) -------------------------------------------------
class Reader {
 public:
  Reader(const void* p, size_t n) : p_(static_cast<const uint8_t*>(p)), n_(n) {}
  template <class T>
  T get(size_t pos) const {
    check(pos, sizeof(T));
    if constexpr (std::is_same_v<T, bool>) {
      return p_[pos] != 0;  // any byte may stand there; only 0 and 1 are values of a bool
    } else {
      T v;
      std::memcpy(&v, p_ + pos, sizeof(T));
      return v;
    }
  }
  const uint8_t* at(size_t pos, size_t len) const {
    check(pos, len);
    return p_ + pos;
  }
  // resolves an offset_ptr stored at `pos`; returns false for null
  bool target(size_t pos, size_t* out) const {
    int64_t off = get<int64_t>(pos);
    if (off == kNullOffset) return false;
    int64_t t = static_cast<int64_t>(pos) + off;
    if (t < 0 || static_cast<size_t>(t) > n_) throw std::runtime_error("deserialize: pointer outside the message");
    *out = static_cast<size_t>(t);
    return true;
  }

 private:
  void check(size_t pos, size_t len) const {
    if (pos > n_ || len > n_ - pos) throw std::runtime_error("deserialize: truncated message");
  }
  const uint8_t* p_;
  size_t n_;
};

inline data::string dec_string(const Reader& r, size_t pos) {
  if (r.get<uint8_t>(pos) != 0) {
    const char* s = reinterpret_cast<const char*>(r.at(pos + 1, 15));
    return data::string(std::string_view(s, strnlen(s, 15)));
  }
  uint32_t size = r.get<uint32_t>(pos + 4);
  size_t t;
  if (!r.target(pos + 8, &t) || size == 0) return {};
  return data::string(std::string_view(reinterpret_cast<const char*>(r.at(t, size)), size));
}

template <class E>
void dec_scalar_vector(const Reader& r, size_t pos, std::vector<E>& out) {
  uint32_t n = r.get<uint32_t>(pos + 8);
  size_t t;
  out.clear();
  if (n == 0 || !r.target(pos, &t)) return;
  // the count comes from the wire: the elements must be inside the message before room is made for them
  const uint8_t* src = r.at(t, sizeof(E) * size_t(n));
  out.resize(n);
  std::memcpy(static_cast<void*>(out.data()), src, sizeof(E) * size_t(n));
}

inline void dec_tensor_meta(const Reader& r, size_t pos, TensorMeta& m) {
  m.device.device_type = static_cast<DLDeviceType>(r.get<int32_t>(pos));
  m.device.device_id = r.get<int32_t>(pos + 4);
  m.ndim = r.get<int32_t>(pos + 8);
  m.dtype.code = r.get<uint8_t>(pos + 12);
  m.dtype.bits = r.get<uint8_t>(pos + 13);
  m.dtype.lanes = r.get<uint16_t>(pos + 14);
  m.byte_offset = r.get<uint64_t>(pos + 16);
  dec_scalar_vector(r, pos + 24, m.shape);
  dec_scalar_vector(r, pos + 48, m.strides);
  // rank, shape and strides travel as three separate fields; the code that reads a description indexes the two
  // vectors by the rank, so a description in which they disagree (or with a negative extent) is refused here
  bool ok = m.ndim >= 0 && m.ndim <= 64 && m.shape.size() == size_t(m.ndim) && (m.strides.empty() || m.strides.size() == size_t(m.ndim));
  for (size_t i = 0; ok && i < m.shape.size(); ++i) ok = m.shape[i] >= 0;
  if (!ok) throw std::runtime_error("deserialize: tensor metadata whose rank, shape and strides disagree");
  if (m.strides.empty() && m.ndim > 0) {  // a sender that left the strides out meant the dense ones
    m.strides.resize(m.ndim);
    int64_t st = 1;
    for (int i = m.ndim - 1; i >= 0; --i) {
      m.strides[i] = st;
      if (m.shape[i] > 0 && __builtin_mul_overflow(st, m.shape[i], &st)) throw std::runtime_error("deserialize: tensor metadata too large");
    }
  }
}

template <size_t I = 0>
void dec_primitive(const Reader& r, size_t pos, uint8_t idx, PrimitiveValue& out) {
  if constexpr (I < std::variant_size_v<PrimitiveValue>) {
    if (idx == I) out.emplace<I>(r.get<std::variant_alternative_t<I, PrimitiveValue>>(pos));
    else dec_primitive<I + 1>(r, pos, idx, out);
  } else {
    throw std::runtime_error("deserialize: bad primitive index");
  }
}
template <size_t I = 0>
void dec_vector_value(const Reader& r, size_t pos, uint8_t idx, VectorValue& out) {
  if constexpr (I < std::variant_size_v<VectorValue>) {
    if (idx == I) dec_scalar_vector(r, pos, out.emplace<I>());
    else dec_vector_value<I + 1>(r, pos, idx, out);
  } else {
    throw std::runtime_error("deserialize: bad vector index");
  }
}

inline void dec_param_value(const Reader& r, size_t pos, ParamValue& v) {
  const uint8_t idx = r.get<uint8_t>(pos);
  const size_t s = pos + 8;
  switch (idx) {
    case 0: dec_primitive(r, s + 8, r.get<uint8_t>(s), v.emplace<0>()); break;
    case 1: dec_vector_value(r, s + 8, r.get<uint8_t>(s), v.emplace<1>()); break;
    case 2: v.emplace<2>(dec_string(r, s)); break;
    case 3: v.emplace<3>(nullptr); break;
    case 4: dec_tensor_meta(r, s, v.emplace<4>()); break;
    case 5: {
      auto& vec = v.emplace<5>();
      uint32_t n = r.get<uint32_t>(s + 8);
      size_t t;
      if (n && r.target(s, &t)) {
        (void)r.at(t, size_t(n) * kTensorMetaSize);  // all inside the message, or an exception before any allocation
        vec.resize(n);
        for (uint32_t i = 0; i < n; ++i) dec_tensor_meta(r, t + size_t(i) * kTensorMetaSize, vec[i]);
      }
      break;
    }
    default: v.emplace<3>(nullptr); break;  // empty variant
  }
}

// A parameter's declared type and the alternative its value holds come from two separate bytes of the message.
// Every typed accessor looks at the first and then takes the second for granted, so a message in which they
// disagree is refused here, once, instead of surfacing as a bad variant access wherever the value is read.
// UNKNOWN (and numbers no version of the enum has) promise nothing and are left alone.
inline bool type_matches_value(ParamType t, const ParamValue& v) {
  const unsigned k = static_cast<unsigned>(t);
  if (k <= static_cast<unsigned>(ParamType::PRIMITIVE_FLOAT64)) {
    auto* p = std::get_if<PrimitiveValue>(&v);
    return p && p->index() == k;
  }
  if (k <= static_cast<unsigned>(ParamType::VECTOR_FLOAT64)) {
    auto* p = std::get_if<VectorValue>(&v);
    return p && p->index() == k - static_cast<unsigned>(ParamType::VECTOR_BOOL);
  }
  switch (t) {
    case ParamType::STRING: return std::holds_alternative<data::string>(v);
    case ParamType::VOID: return std::holds_alternative<std::nullptr_t>(v);
    case ParamType::TENSOR_META: return std::holds_alternative<TensorMeta>(v);
    case ParamType::TENSOR_META_VEC: return std::holds_alternative<TensorMetaVec>(v);
    default: return true;
  }
}

inline void dec_param_vector(const Reader& r, size_t pos, data::vector<ParamMeta>& out) {
  out.clear();
  uint32_t n = r.get<uint32_t>(pos + 8);
  size_t t;
  if (n == 0 || !r.target(pos, &t)) return;
  (void)r.at(t, size_t(n) * kParamMetaSize);
  out.resize(n);
  for (uint32_t i = 0; i < n; ++i) {
    size_t p = t + size_t(i) * kParamMetaSize;
    out[i].type = static_cast<ParamType>(r.get<uint8_t>(p));
    dec_param_value(r, p + 8, out[i].value);
    if (!type_matches_value(out[i].type, out[i].value)) throw std::runtime_error("deserialize: a parameter's type does not match its value");
    out[i].name = dec_string(r, p + 88);
  }
}

inline void decode(const Reader& r, RpcRequestHeader& h) {
  h.session_id.v_ = r.get<uint32_t>(0);
  h.request_id.v_ = r.get<uint32_t>(4);
  h.function_id.v_ = r.get<uint32_t>(8);
  h.hlc = HybridLogicalClock(r.get<uint64_t>(16));
  h.workflow_id.v_ = r.get<uint32_t>(24);
  dec_param_vector(r, 32, h.params);
}
inline void decode(const Reader& r, RpcResponseHeader& h) {
  h.session_id.v_ = r.get<uint32_t>(0);
  h.request_id.v_ = r.get<uint32_t>(4);
  h.hlc = HybridLogicalClock(r.get<uint64_t>(8));
  h.workflow_id.v_ = r.get<uint32_t>(16);
  h.status.value = r.get<int32_t>(24);
  h.status.category_name = dec_string(r, 32);
  dec_param_vector(r, 48, h.results);
}
inline void decode(const Reader& r, data::vector<RpcFunctionSignature>& out) {
  out.clear();
  uint32_t n = r.get<uint32_t>(8);
  size_t t;
  if (n == 0 || !r.target(0, &t)) return;
  (void)r.at(t, size_t(n) * kSignatureSize);
  out.resize(n);
  for (uint32_t i = 0; i < n; ++i) {
    size_t p = t + size_t(i) * kSignatureSize;
    out[i].instance_name = dec_string(r, p);
    out[i].id.v_ = r.get<uint32_t>(p + 16);
    out[i].function_name = dec_string(r, p + 24);
    dec_scalar_vector(r, p + 40, out[i].param_types);
    dec_scalar_vector(r, p + 64, out[i].return_types);
    out[i].input_payload_type = static_cast<PayloadType>(r.get<uint8_t>(p + 88));
    out[i].return_payload_type = static_cast<PayloadType>(r.get<uint8_t>(p + 89));
  }
}

}  // namespace wire

using wire::FixedBufferWriter;

// Exact size of the serialised form.
template <class T>
size_t GetSerializedSize(const T& v) {
  wire::SizeCounter c;
  wire::encode(c, v);
  return c.size();
}
template <class T>
byte_buf Serialize(const T& v) {
  byte_buf out;
  wire::BufWriter w(out);
  wire::encode(w, v);
  return out;
}
// Serialise straight into caller-provided memory (e.g. an active-message header buffer).
template <class T>
size_t SerializeInto(FixedBufferWriter& w, const T& v) {
  wire::encode(w, v);
  return w.size();
}
template <class T>
T Deserialize(const void* p, size_t n) {
  T out;
  wire::decode(wire::Reader(p, n), out);
  return out;
}
template <class T>
T Deserialize(const byte_buf& b) {
  return Deserialize<T>(b.data(), b.size());
}

}  // namespace eux::rpc
