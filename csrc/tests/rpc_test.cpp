// rpc_core: wire image (hand-derived golden bytes), dispatcher, builders, async
// dispatcher, hybrid logical clock (CPU only).
#include <atomic>
#include <cstring>
#include <chrono>
#include <random>

#include "check.hpp"
#include "eux/exec/contexts.hpp"
#include "eux/rpc/async_rpc_dispatcher.hpp"
#include "eux/rpc/rpc_facade_helpers.hpp"

using namespace eux::rpc;
using eux::ucxx::DefaultUcxMemoryResourceManager;
using eux::ucxx::UcxBuffer;
using eux::ucxx::UcxBufferVec;
namespace ex = eux::exec;

static int64_t i64_at(const byte_buf& b, size_t pos) { int64_t v; std::memcpy(&v, b.data() + pos, 8); return v; }
static uint32_t u32_at(const byte_buf& b, size_t pos) { uint32_t v; std::memcpy(&v, b.data() + pos, 4); return v; }

// Layout derived by hand from the offset-mode rules: 56-byte root, params vector at 32,
// one 104-byte ParamMeta appended at 56 (8-aligned), long strings appended after it.
EUX_TEST(golden_request_image) {
  RpcRequestHeader h;
  h.session_id = session_id_t{0x11223344};
  h.request_id = request_id_t{7};
  h.function_id = function_id_t{0xabcd};
  h.hlc = HybridLogicalClock(0x0102030405060708ull);
  h.workflow_id = workflow_id_t{9};
  h.AddParam(int32_t(-5));
  byte_buf b = Serialize(h);
  CHECK_EQ(b.size(), 56u + 104u);
  CHECK_EQ(GetSerializedSize(h), b.size());
  CHECK_EQ(u32_at(b, 0), 0x11223344u);
  CHECK_EQ(u32_at(b, 4), 7u);
  CHECK_EQ(u32_at(b, 8), 0xabcdu);
  CHECK_EQ(u32_at(b, 12), 0u);  // padding before the 8-aligned clock
  CHECK_EQ((uint64_t)i64_at(b, 16), 0x0102030405060708ull);
  CHECK_EQ(u32_at(b, 24), 9u);
  CHECK_EQ(i64_at(b, 32), 56 - 32);  // vector.el_: distance from the field to the element array
  CHECK_EQ(u32_at(b, 40), 1u);       // used
  CHECK_EQ(u32_at(b, 44), 1u);       // allocated
  CHECK_EQ(b[48], 0);                // self_allocated
  // ParamMeta at 56: type u8, value variant at +8 {index 0 -> PrimitiveValue {index 3 (int32), storage +8}}, name at +88
  CHECK_EQ(b[56], (uint8_t)ParamType::PRIMITIVE_INT32);
  CHECK_EQ(b[64], 0);
  CHECK_EQ(b[72], 3);
  int32_t v;
  std::memcpy(&v, b.data() + 80, 4);
  CHECK_EQ(v, -5);
  CHECK_EQ(b[56 + 88], 1);  // empty name = short string
  CHECK_EQ(b[56 + 89], 0);
}

EUX_TEST(golden_strings_and_empty_vector) {
  RpcResponseHeader r;
  r.session_id = session_id_t{1};
  r.request_id = request_id_t{2};
  r.status = RpcStatus(make_error_code(RpcErrc::NOT_FOUND));  // category "RPC": short string
  byte_buf b = Serialize(r);
  CHECK_EQ(b.size(), 72u);
  int32_t sv;
  std::memcpy(&sv, b.data() + 24, 4);
  CHECK_EQ(sv, 5);
  CHECK_EQ(b[32], 1);
  CHECK(std::memcmp(b.data() + 33, "RPC\0", 4) == 0);
  CHECK_EQ(i64_at(b, 48), std::numeric_limits<int64_t>::min());  // empty vector: null pointer
  CHECK_EQ(u32_at(b, 56), 0u);
  // a string longer than 15 characters goes to the heap form
  r.AddResult(data::string("a string that is definitely longer than fifteen"));
  b = Serialize(r);
  const size_t pm = 72, str = pm + 8 + 8;  // ParamMeta at 72; value storage at +16
  CHECK_EQ(b[pm], (uint8_t)ParamType::STRING);
  CHECK_EQ(b[pm + 8], 2);  // variant index of string
  CHECK_EQ(b[str], 0);     // long form
  CHECK_EQ(u32_at(b, str + 4), 47u);
  size_t target = size_t(int64_t(str + 8) + i64_at(b, str + 8));
  CHECK_EQ(target, 72u + 104u);
  CHECK(std::memcmp(b.data() + target, "a string that", 13) == 0);
  CHECK_EQ(b.size(), 72u + 104u + 47u);
  // a short string with a NUL inside (a binary blob carried as a string parameter) keeps every byte: it goes
  // to the long form, because the short form ends at the first NUL for its reader
  RpcResponseHeader blobs;
  const std::string blob("\x02\x00\x00\x00\x01\x00\x00\x00" "a", 9);
  blobs.AddResult(data::string(blob));
  blobs.AddResult(data::string(std::string("tail\0", 5)));
  blobs.AddResult(data::string("plain"));
  b = Serialize(blobs);
  CHECK_EQ(b[72 + 16], 0);              // long form
  CHECK_EQ(b[72 + 2 * 104 + 16], 1);    // "plain": short form, as before
  RpcResponseHeader back = Deserialize<RpcResponseHeader>(b.data(), b.size());
  CHECK_EQ(back.results.size(), 3u);
  CHECK(std::get<data::string>(back.results[0].value) == data::string(blob));
  CHECK_EQ(std::get<data::string>(back.results[1].value).size(), 5u);
  CHECK(std::get<data::string>(back.results[2].value) == data::string("plain"));
}

EUX_TEST(round_trip_all_kinds) {
  RpcRequestHeader h;
  h.session_id = session_id_t{3};
  h.AddParam(true);
  h.AddParam(int8_t(-1));
  h.AddParam(uint16_t(65000));
  h.AddParam(int64_t(-1234567890123));
  h.AddParam(3.5f);
  h.AddParam(2.25);
  h.AddParam(data::string("short"));
  h.AddParam(std::string(100, 'x'));
  h.AddParam(data::vector<int32_t>{1, 2, 3});
  h.AddParam(data::vector<double>{});
  h.AddParam(data::vector<bool>{true, false, true});
  h.AddParam(nullptr);
  TensorMeta tm;
  tm.device = {kDLCUDA, 3};
  tm.ndim = 2;
  tm.dtype = {kDLBfloat, 16, 1};
  tm.shape = {4, 8};
  tm.strides = {8, 1};
  h.AddParam(tm);
  TensorMetaVec tv{tm, tm};
  tv[1].shape = {2, 2};
  h.AddParam(tv);
  h.params.back().name = data::string("tensors");
  byte_buf b = Serialize(h);
  CHECK_EQ(GetSerializedSize(h), b.size());
  std::vector<uint8_t> fixed(b.size());
  FixedBufferWriter w(fixed.data(), fixed.size());
  CHECK_EQ(SerializeInto(w, h), b.size());
  CHECK(std::memcmp(fixed.data(), b.data(), b.size()) == 0);
  std::vector<uint8_t> small(b.size() - 1);
  FixedBufferWriter w2(small.data(), small.size());
  CHECK_THROWS(SerializeInto(w2, h));
  auto d = Deserialize<RpcRequestHeader>(b);
  CHECK_EQ(d.params.size(), h.params.size());
  CHECK_EQ(d.GetPrimitive<bool>(0), true);
  CHECK_EQ(d.GetPrimitive<int8_t>(1), -1);
  CHECK_EQ(d.GetPrimitive<uint16_t>(2), 65000);
  CHECK_EQ(d.GetPrimitive<int64_t>(3), -1234567890123);
  CHECK_EQ(d.GetPrimitive<float>(4), 3.5f);
  CHECK_EQ(d.GetPrimitive<double>(5), 2.25);
  CHECK(d.GetString(6) == "short");
  CHECK_EQ(d.GetString(7).size(), 100u);
  CHECK((d.GetVector<int32_t>(8) == data::vector<int32_t>{1, 2, 3}));
  CHECK(d.GetVector<double>(9).empty());
  CHECK_EQ(d.GetVector<bool>(10).size(), 3u);
  CHECK(d.GetVector<bool>(10)[2]);
  CHECK(d.params[11].type == ParamType::VOID);
  CHECK(d.GetTensor(12) == tm);
  CHECK(d.GetTensorVec(13)[1].shape == (data::vector<int64_t>{2, 2}));
  CHECK(d.params[13].name == "tensors");
  CHECK_THROWS(d.GetPrimitive<int32_t>(0));
  CHECK_THROWS(d.GetString(99));
  CHECK_THROWS(Deserialize<RpcRequestHeader>(b.data(), 20));
  // truncation anywhere must throw or parse, never read outside
  for (size_t n = 0; n < b.size(); n += 7) {
    try { (void)Deserialize<RpcRequestHeader>(b.data(), n); } catch (const std::exception&) {}
  }
}

// A count read from the wire is checked against the message before memory is reserved for it: an image that
// claims four billion elements is refused at once instead of after tens of gigabytes of allocation.
EUX_TEST(counts_from_the_wire_are_checked_before_memory_is_reserved) {
  RpcRequestHeader h;
  h.session_id = session_id_t{1};
  h.AddParam(data::vector<int64_t>{1, 2, 3});
  TensorMetaVec metas(2);
  h.params.push_back(ParamMeta(ParamType::TENSOR_META_VEC, ParamValue(std::in_place_type<TensorMetaVec>, metas)));
  const byte_buf good = Serialize(h);
  CHECK_EQ(Deserialize<RpcRequestHeader>(good.data(), good.size()).params.size(), 2u);
  const uint32_t huge = 0xffffffffu;
  auto refused_quickly = [&](size_t count_at) {
    byte_buf bad = good;
    std::memcpy(bad.data() + count_at, &huge, 4);
    auto t0 = std::chrono::steady_clock::now();
    bool threw = false;
    try {
      (void)Deserialize<RpcRequestHeader>(bad.data(), bad.size());
    } catch (const std::exception&) {
      threw = true;
    }
    return threw && std::chrono::steady_clock::now() - t0 < std::chrono::milliseconds(200);
  };
  const size_t params_at = 56;                      // the header's fixed part; the ParamMeta records follow
  CHECK(refused_quickly(32 + 8));                   // how many parameters
  CHECK(refused_quickly(params_at + 8 + 8 + 8 + 8));              // elements of the int64 vector: ParamMeta +8 value, +8 storage, +8 vector, +8 count
  CHECK(refused_quickly(params_at + 104 + 8 + 8 + 8));            // tensor descriptions in the second parameter
}

// The declared type of a parameter and the alternative its value holds are separate bytes of the image; so are a
// tensor description's rank and the lengths of its shape and strides. An image in which they disagree is refused
// when it is read, not wherever the value is used later.
EUX_TEST(images_that_contradict_themselves_are_refused) {
  RpcRequestHeader h;
  h.AddParam(int64_t{5});
  TensorMeta m;
  m.ndim = 2;
  m.dtype = {kDLFloat, 32, 1};
  m.shape = {3, 4};
  m.strides = {4, 1};
  h.params.push_back(ParamMeta(ParamType::TENSOR_META, ParamValue(std::in_place_type<TensorMeta>, m)));
  const byte_buf good = Serialize(h);
  RpcRequestHeader back = Deserialize<RpcRequestHeader>(good.data(), good.size());
  CHECK_EQ(back.GetPrimitive<int64_t>(0), int64_t{5});
  CHECK_EQ(utils::CalculateTensorSize(back.GetTensor(1)), size_t(48));
  const size_t p0 = 56, p1 = 56 + 104;  // the two ParamMeta records
  auto refused = [&](size_t at, auto value) {
    byte_buf bad = good;
    std::memcpy(bad.data() + at, &value, sizeof(value));
    try {
      (void)Deserialize<RpcRequestHeader>(bad.data(), bad.size());
    } catch (const std::exception&) {
      return true;
    }
    return false;
  };
  CHECK(refused(p0, uint8_t(ParamType::STRING)));              // says string, holds an int64
  CHECK(refused(p0, uint8_t(ParamType::PRIMITIVE_FLOAT64)));   // says double, holds an int64
  CHECK(refused(p0, uint8_t(ParamType::TENSOR_META)));         // says tensor, holds an int64
  CHECK(refused(p1, uint8_t(ParamType::VECTOR_INT64)));        // says vector, holds a tensor description
  CHECK(!refused(p0, uint8_t(ParamType::UNKNOWN)));            // promises nothing: nobody reads it by type
  const size_t meta_at = p1 + 8 + 8;                           // ParamMeta +8 value, +8 storage
  CHECK(refused(meta_at + 8, int32_t(3)));                     // rank 3, two extents
  CHECK(refused(meta_at + 8, int32_t(-1)));
  CHECK(refused(meta_at + 8, int32_t(1 << 20)));
  // descriptions that are no tensor count as larger than any buffer
  TensorMeta huge = m;
  huge.shape = {int64_t(1) << 62, 8};
  CHECK_EQ(utils::CalculateTensorSize(huge), static_cast<size_t>(-1));
  huge.shape = {-3, 4};
  CHECK_EQ(utils::CalculateTensorSize(huge), static_cast<size_t>(-1));
  huge.ndim = 5;
  CHECK_EQ(utils::CalculateTensorSize(huge), static_cast<size_t>(-1));
  CHECK(!huge.is_compact());
}

static int32_t add(int32_t a, int32_t b) { return a + b; }

EUX_TEST(thousand_add_calls) {
  RpcDispatcher disp("calc");
  CHECK(disp.RegisterFunction(function_id_t{1}, &add, data::string("add")));
  CHECK(!disp.RegisterFunction(function_id_t{1}, &add, data::string("add")));
  std::mt19937 rng(42);
  std::uniform_int_distribution<int32_t> dist(-(1 << 20), 1 << 20);
  RpcRequestBuilder rb;
  for (int i = 0; i < 1000; ++i) {
    int32_t a = dist(rng), b = dist(rng);
    auto req = rb.PrepareRequest({session_id_t{1}, request_id_t{uint32_t(i)}, function_id_t{1}}, a, b);
    auto res = disp.Dispatch<std::monostate>(Serialize(req));  // through the wire form
    CHECK(res.header.status.ok());
    CHECK_EQ(res.header.request_id.v_, uint32_t(i));
    CHECK_EQ(res.header.GetPrimitive<int32_t>(0), a + b);
  }
  auto sig = disp.GetSignature(function_id_t{1});
  CHECK(sig.has_value());
  CHECK((sig->param_types == data::vector<ParamType>{ParamType::PRIMITIVE_INT32, ParamType::PRIMITIVE_INT32}));
  CHECK((sig->return_types == data::vector<ParamType>{ParamType::PRIMITIVE_INT32}));
  auto blob = disp.GetAllSignatures();
  auto sigs = RpcDispatcher::DeserializeSignatures(blob.data(), blob.size());
  CHECK_EQ(sigs.size(), 1u);
  CHECK(sigs[0].function_name == "add" && sigs[0].instance_name == "calc");
  // signature-checked request building
  CHECK_THROWS(rb.PrepareRequest(*sig, {}, int32_t(1)));
  CHECK_THROWS(rb.PrepareRequest(*sig, {}, int32_t(1), 2.0));
  auto ok = rb.PrepareRequest(*sig, {}, int32_t(1), int32_t(2));
  CHECK_EQ(ok.function_id.v_, 1u);
}

// Forty thousand mutated copies of a valid request image go through the dispatcher, payload attached: each ends
// as a response with a status (or as an exception from the reader), none as a fault, and the handler only ever
// sees arguments that agree with the image it was given.
EUX_TEST(mutated_request_images_end_as_statuses) {
  DefaultUcxMemoryResourceManager mr;
  RpcDispatcher disp("svc");
  size_t handled = 0, beyond_the_payload = 0;
  disp.RegisterFunction(
      function_id_t{3},
      [&handled, &beyond_the_payload](const RpcRequestHeader& req, int32_t a, const data::string& s, const data::vector<int64_t>& v, const TensorMeta& m,
                                      UcxBuffer& buf, const RpcResponseBuilder& b) {
        ++handled;
        uint64_t sum = static_cast<uint64_t>(a);   // unsigned: the mutated values may be anything
        for (auto x : v) sum += static_cast<uint64_t>(x);
        // the dispatcher has checked the description against the payload: every element may be touched
        const size_t bytes = utils::CalculateTensorSize(m);
        if (bytes > buf.size()) {  // counted, not thrown: the dispatcher would turn an exception into a status
          ++beyond_the_payload;
          return b.PrepareResponse(req.session_id, req.request_id, data::string(), int64_t(0));
        }
        unsigned char acc = 0;
        for (size_t i = 0; i < bytes; ++i) acc ^= static_cast<unsigned char*>(buf.data())[i];
        return b.PrepareResponse(req.session_id, req.request_id, data::string(s.str() + "!"), static_cast<int64_t>(sum + acc));
      },
      data::string("mixed"));
  TensorMeta m;
  m.ndim = 2;
  m.dtype = {kDLFloat, 32, 1};
  m.shape = {4, 8};
  m.strides = {8, 1};
  UcxBuffer buf(mr, ucx_memory_type::HOST, 128);
  std::memset(buf.data(), 1, 128);
  auto [req, payload] = RpcRequestBuilder{}.PrepareRequest({session_id_t{8}, request_id_t{9}, function_id_t{3}}, int32_t(5),
                                                          data::string("a string of more than fifteen bytes"),
                                                          data::vector<int64_t>{1, 2, 3}, m, std::move(buf));
  const byte_buf good = Serialize(req);
  CHECK(disp.Dispatch(Deserialize<RpcRequestHeader>(good.data(), good.size()), payload).header.status.ok());
  std::mt19937 rng(7);
  size_t refused_by_reader = 0, statuses = 0, served = 0;
  for (int i = 0; i < 40000; ++i) {
    byte_buf bad = good;
    const int flips = 1 + int(rng() % 6);
    for (int k = 0; k < flips; ++k) {
      const size_t at = rng() % bad.size();
      if (rng() % 10 < 6) bad[at] = static_cast<unsigned char>(rng() & 0xff);
      else bad[at] ^= static_cast<unsigned char>(1u << (rng() % 8));
    }
    size_t len = bad.size();
    if (rng() % 4 == 0) len = rng() % (bad.size() + 1);
    try {
      RpcRequestHeader h = Deserialize<RpcRequestHeader>(bad.data(), len);
      auto res = disp.Dispatch(h, payload);
      res.header.status.ok() ? ++served : ++statuses;
    } catch (const std::exception&) {
      ++refused_by_reader;
    }
  }
  CHECK_EQ(refused_by_reader + statuses + served, size_t(40000));
  CHECK(served > 0 && statuses > 0 && refused_by_reader > 0);
  CHECK(handled >= served);
  CHECK_EQ(beyond_the_payload, size_t(0));
}

EUX_TEST(dispatch_errors_and_argument_kinds) {
  DefaultUcxMemoryResourceManager mr;
  RpcDispatcher disp("svc");
  auto missing = disp.Dispatch(RpcRequestBuilder{}.PrepareRequest({session_id_t{5}, request_id_t{6}, function_id_t{99}}));
  CHECK_EQ(missing.header.status.value, int(RpcErrc::NOT_FOUND));
  CHECK(std::string(missing.header.status.category_name) == "RPC");
  CHECK_EQ(missing.header.session_id.v_, 5u);
  CHECK(!missing.header.GetString(0).empty());
  disp.RegisterFunction(function_id_t{2}, [](int32_t) -> int32_t { throw std::runtime_error("kaput"); }, data::string("thrower"));
  auto thrown = disp.Dispatch(RpcRequestBuilder{}.PrepareRequest({{}, {}, function_id_t{2}}, int32_t(1)));
  CHECK_EQ(thrown.header.status.value, int(RpcErrc::INTERNAL));
  CHECK(thrown.header.GetString(0) == "kaput");
  auto wrong = disp.Dispatch(RpcRequestBuilder{}.PrepareRequest({{}, {}, function_id_t{2}}, 2.5));
  CHECK(!wrong.header.status.ok());
  // header, builder, string, vector, tensor meta and payload by reference
  disp.RegisterFunction(
      function_id_t{3},
      [](const RpcRequestHeader& req, const data::string& s, const data::vector<float>& v, const TensorMeta& m, UcxBuffer& buf,
         const RpcResponseBuilder& b) {
        float sum = 0;
        for (float x : v) sum += x;
        static_cast<char*>(buf.data())[0] = 'Z';
        return b.PrepareResponse(req.session_id, req.request_id, data::string(s.str() + "!"), sum, int64_t(m.shape[0]));
      },
      data::string("mixed"));
  TensorMeta m;
  m.ndim = 1;
  m.shape = {16};
  m.strides = {1};
  UcxBuffer buf(mr, ucx_memory_type::HOST, 16);
  auto [req, payload] = RpcRequestBuilder{}.PrepareRequest({session_id_t{8}, request_id_t{9}, function_id_t{3}}, data::string("hey"),
                                                          data::vector<float>{1.f, 2.f}, m, std::move(buf));
  CHECK(RpcDispatcher::ValidateTensorPayloadConstraints(req.params, payload).ok());
  auto res = disp.Dispatch(req, payload);
  CHECK(res.header.status.ok());
  CHECK(res.header.GetString(0) == "hey!");
  CHECK_EQ(res.header.GetPrimitive<float>(1), 3.f);
  CHECK_EQ(res.header.GetPrimitive<int64_t>(2), 16);
  CHECK_EQ(static_cast<char*>(std::get<UcxBuffer>(payload).data())[0], 'Z');
  // payload by value needs DispatchMove; payload returned in a tuple
  disp.RegisterFunction(function_id_t{4}, [&mr](UcxBuffer in) {
    UcxBufferVec out(mr, ucx_memory_type::HOST, std::vector<size_t>{in.size(), 4});
    return std::tuple<int32_t, UcxBufferVec>(int32_t(in.size()), std::move(out));
  }, data::string("consume"));
  UcxBuffer b2(mr, ucx_memory_type::HOST, 32);
  auto r4req = RpcRequestBuilder{}.PrepareRequest({{}, {}, function_id_t{4}});
  CHECK(!disp.Dispatch(r4req, b2).header.status.ok());
  auto r4 = disp.DispatchMove<UcxBufferVec>(r4req, std::move(b2));
  CHECK_EQ(r4.header.GetPrimitive<int32_t>(0), 32);
  CHECK_EQ(r4.payload.size(), 2u);
  auto sig = disp.GetSignature(function_id_t{4});
  CHECK(sig->input_payload_type == PayloadType::UCX_BUFFER && sig->return_payload_type == PayloadType::UCX_BUFFER_VEC);
  // mismatching metadata is caught
  TensorMeta big = m;
  big.shape = {1 << 20};
  data::vector<ParamMeta> ps;
  ps.emplace_back(big);
  CHECK(!RpcDispatcher::ValidateTensorPayloadConstraints(ps, payload).ok());
  // dynamic registration
  disp.RegisterFunction(function_id_t{5}, data::string("dyn"), {ParamType::PRIMITIVE_INT32}, {ParamType::PRIMITIVE_INT32}, PayloadType::NO_PAYLOAD,
                        PayloadType::NO_PAYLOAD, [](const RpcRequestHeader& rq, RpcContextPtr, const RpcResponseBuilder& b) -> DynamicRpcResult {
                          return {b.PrepareResponse(rq.session_id, rq.request_id, int32_t(rq.GetPrimitive<int32_t>(0) * 2)), ReturnedPayload{}};
                        });
  CHECK_EQ(disp.Dispatch(RpcRequestBuilder{}.PrepareRequest({{}, {}, function_id_t{5}}, int32_t(21))).header.GetPrimitive<int32_t>(0), 42);
  CHECK_EQ(disp.FunctionCount(), 4u);
  static_assert(accepts_every_payload_v<decltype([](auto&&) {})>);
}

// Natural call: the registered native callables fetched back and called with plain arguments.
EUX_TEST(get_caller_natural_syntax) {
  DefaultUcxMemoryResourceManager mr;
  RpcDispatcher d("natural");
  d.RegisterFunction(function_id_t{1}, [](int a, int b) { return a + b; }, "add");
  d.RegisterFunction(function_id_t{2}, [] {}, "no_op");
  d.RegisterFunction(function_id_t{3}, [] { return std::tuple<int, data::string, float>(123, data::string("hello"), 3.14f); }, "multi");
  d.RegisterFunction(function_id_t{4}, [&mr] { return UcxBufferVec(mr, ucx_memory_type::HOST, std::vector<size_t>{128, 256}); }, "vec");
  d.RegisterFunction(function_id_t{5}, [](const UcxBufferVec& v) { return uint64_t(v.total_size()); }, "sum");
  d.RegisterFunction(function_id_t{6}, [&mr] { return std::tuple<int, UcxBufferVec>(456, UcxBufferVec(mr, ucx_memory_type::HOST, std::vector<size_t>{16, 32})); }, "multi_payload");
  d.RegisterFunction(function_id_t{7}, []() -> void { throw std::runtime_error("Something went wrong"); }, "boom");
  d.RegisterFunction(function_id_t{8}, [](UcxBuffer b) { return uint64_t(b.size()); }, "consume");

  CHECK_EQ((*d.GetCaller<int(int, int)>(function_id_t{1}))(20, 22), 42);
  (*d.GetCaller<void()>(function_id_t{2}))();
  auto [i, s, f] = (*d.GetCaller<std::tuple<int, data::string, float>()>(function_id_t{3}))();
  CHECK(i == 123 && s == "hello" && f == 3.14f);
  auto vec = (*d.GetCaller<UcxBufferVec()>(function_id_t{4}))();
  CHECK(vec.size() == 2 && vec[0].size == 128 && vec[1].size == 256);
  UcxBufferVec in(mr, ucx_memory_type::HOST, std::vector<size_t>{100, 200, 300});
  CHECK_EQ((*d.GetCaller<uint64_t(const UcxBufferVec&)>(function_id_t{5}))(in), uint64_t(600));
  CHECK_EQ(in.size(), 3u);  // passed by const reference: untouched
  auto [val, pv] = (*d.GetCaller<std::tuple<int, UcxBufferVec>()>(function_id_t{6}))();
  CHECK(val == 456 && pv.size() == 2 && pv[1].size == 32);
  // a by-value payload parameter takes the caller's buffer
  UcxBuffer gift(mr, ucx_memory_type::HOST, 77);
  CHECK_EQ((*d.GetCaller<uint64_t(UcxBuffer)>(function_id_t{8}))(std::move(gift)), uint64_t(77));
  // unknown id, wrong signature, and an exception that comes through as it is
  CHECK_THROWS(d.GetCaller<void()>(function_id_t{999}));
  CHECK_THROWS(d.GetCaller<int(int)>(function_id_t{1}));
  bool same_text = false;
  try {
    (*d.GetCaller<void()>(function_id_t{7}))();
  } catch (const std::runtime_error& e) {
    same_text = std::string(e.what()) == "Something went wrong";
  }
  CHECK(same_text);
  // the serialised path still works for the same registration
  auto resp = d.Dispatch(RpcRequestBuilder{}.PrepareRequest({session_id_t{1}, request_id_t{1}, function_id_t{1}}, int(2), int(3)));
  CHECK(resp.header.status.ok() && resp.header.GetPrimitive<int>(0) == 5);
}

EUX_TEST(async_dispatcher_senders) {
  ex::static_thread_pool pool(2);
  AsyncRpcDispatcher disp("async");
  disp.RegisterFunction(function_id_t{1}, [&](int32_t a, int32_t b) { return ex::on(pool.get_scheduler(), ex::just(a * b)); }, data::string("mul"));
  disp.RegisterFunction(function_id_t{2}, [](int32_t a) { return a + 1; }, data::string("inc"));
  disp.RegisterFunction(function_id_t{3}, [&](int32_t) { return ex::on(pool.get_scheduler(), ex::just_from([]() -> int32_t { throw RpcException(RpcErrc::FAILED_PRECONDITION, "nope"); })); },
                        data::string("fail"));
  RpcRequestBuilder rb;
  auto r1 = ex::sync_wait(disp.Dispatch(rb.PrepareRequest({{}, request_id_t{4}, function_id_t{1}}, int32_t(6), int32_t(7))));
  CHECK(r1 && r1->header.status.ok());
  CHECK_EQ(r1->header.GetPrimitive<int32_t>(0), 42);
  CHECK_EQ(r1->header.request_id.v_, 4u);
  auto r2 = ex::sync_wait(disp.Dispatch(Serialize(rb.PrepareRequest({{}, {}, function_id_t{2}}, int32_t(1)))));
  CHECK_EQ(r2->header.GetPrimitive<int32_t>(0), 2);
  auto r3 = ex::sync_wait(disp.Dispatch(rb.PrepareRequest({{}, {}, function_id_t{3}}, int32_t(1))));
  CHECK_EQ(r3->header.status.value, int(RpcErrc::FAILED_PRECONDITION));
  CHECK(r3->header.GetString(0) == "nope");
  auto r4 = ex::sync_wait(disp.Dispatch(rb.PrepareRequest({{}, {}, function_id_t{77}})));
  CHECK_EQ(r4->header.status.value, int(RpcErrc::NOT_FOUND));
}

// Fork/join across three simulated nodes: every effect is later than its cause.
EUX_TEST(hybrid_logical_clock_causality) {
  using eux::rpc::utils::HybridLogicalClock;
  HybridLogicalClock a(1000, 0), b(900, 5), c(1000, 7);
  a.TickLocal(1000);
  CHECK_EQ(a.PhysicalTimeMs(), 1000u);
  CHECK_EQ(a.LogicalCounter(), 1);
  a.TickLocal(1005);
  CHECK(a == HybridLogicalClock(1005, 0));
  HybridLogicalClock sent = a;
  b.Merge(sent, 950);  // b's wall clock is behind: it still moves past the sender
  CHECK(b > sent);
  c.Merge(sent, 1001);
  CHECK(c > sent);
  HybridLogicalClock join = b;
  join.Merge(c, 1002);
  CHECK(join > b && join > c);
  HybridLogicalClock x(5, 0xffff);
  x.TickLocal(5);  // counter exhausted: physical part advances
  CHECK(x == HybridLogicalClock(6, 0));
  CHECK_EQ(HybridLogicalClock(123, 45).Raw(), (123ull << 16) | 45);
  HybridLogicalClock now = HybridLogicalClock::Now(), later = now;
  later.TickLocal();
  CHECK(later > now);
}

// Every return kind a handler may have, through the serialised request and back through the response bytes.
EUX_TEST(return_kinds_and_response_wire_round_trip) {
  DefaultUcxMemoryResourceManager mr;
  RpcDispatcher d("kinds");
  int side_effect = 0;
  d.RegisterFunction(function_id_t{1}, [&](int32_t v) { side_effect = v; }, data::string("void_fn"));
  d.RegisterFunction(function_id_t{2}, [](double x) { return x * 0.5; }, data::string("half"));
  d.RegisterFunction(function_id_t{3}, [](int32_t a) { return std::tuple<int32_t, data::string, bool>(a + 1, data::string("ok"), true); }, data::string("triple"));
  d.RegisterFunction(function_id_t{4}, [](const RpcRequestHeader& rq, const RpcResponseBuilder& b) {
    return b.PrepareResponse(rq.session_id, rq.request_id, data::vector<int64_t>{1, 2, 3});
  }, data::string("header_only"));
  d.RegisterFunction(function_id_t{5}, [&mr](const RpcRequestHeader& rq, const RpcResponseBuilder& b) {
    UcxBuffer out(mr, ucx_memory_type::HOST, 24);
    std::memset(out.data(), 7, 24);
    return b.PrepareResponse(rq.session_id, rq.request_id, int32_t(24), std::move(out));
  }, data::string("header_and_payload"));
  d.RegisterFunction(function_id_t{6}, [&mr] { return UcxBuffer(mr, ucx_memory_type::HOST, 40); }, data::string("payload_only"));
  RpcRequestBuilder rb;
  auto call = [&](uint32_t fid, auto... args) {
    return d.Dispatch(Serialize(rb.PrepareRequest({session_id_t{3}, request_id_t{fid * 10}, function_id_t{fid}}, args...)));
  };
  auto r1 = call(1, int32_t(17));
  CHECK(r1.header.status.ok() && r1.header.results.empty() && side_effect == 17);
  CHECK(std::holds_alternative<std::monostate>(r1.payload));
  CHECK_EQ(call(2, 5.0).header.GetPrimitive<double>(0), 2.5);
  auto r3 = call(3, int32_t(9));
  CHECK_EQ(r3.header.results.size(), 3u);
  CHECK(r3.header.GetPrimitive<int32_t>(0) == 10 && r3.header.GetString(1) == "ok" && r3.header.GetPrimitive<bool>(2));
  auto r4 = call(4);
  CHECK((r4.header.GetVector<int64_t>(0) == data::vector<int64_t>{1, 2, 3}));
  CHECK_EQ(r4.header.request_id.v_, 40u);
  auto r5 = call(5);
  CHECK_EQ(r5.header.GetPrimitive<int32_t>(0), 24);
  CHECK_EQ(std::get<UcxBuffer>(r5.payload).size(), 24u);
  CHECK_EQ(static_cast<unsigned char*>(std::get<UcxBuffer>(r5.payload).data())[23], 7);
  CHECK_EQ(std::get<UcxBuffer>(call(6).payload).size(), 40u);
  // the response header through its wire form, in all three serialising overloads
  byte_buf bytes = RpcDispatcher::SerializeResponse(r3.header);
  byte_buf bytes2;
  RpcDispatcher::SerializeResponse(r3.header, bytes2);
  CHECK(bytes == bytes2);
  RpcResponseHeader back = RpcDispatcher::DeserializeResponse(bytes.data(), bytes.size());
  CHECK(back.session_id.v_ == 3 && back.request_id.v_ == 30 && back.status.ok());
  CHECK(back.GetPrimitive<int32_t>(0) == 10 && back.GetString(1) == "ok" && back.GetPrimitive<bool>(2));
  eux::ucxx::UcxHeader hdr(mr, bytes.size());
  std::memcpy(hdr.data(), bytes.data(), bytes.size());
  RpcResponseHeader back2 = RpcDispatcher::DeerializeResponse(std::move(hdr));
  CHECK(back2.GetString(1) == "ok");
  // an error response keeps its category and text on the wire
  RpcResponseHeader err = RpcResponseBuilder{}.PrepareError(session_id_t{1}, request_id_t{2}, make_error_code(RpcErrc::UNAVAILABLE), "try later");
  byte_buf eb = RpcDispatcher::SerializeResponse(err);
  RpcResponseHeader eback = RpcDispatcher::DeserializeResponse(eb.data(), eb.size());
  CHECK(!eback.status.ok());
  CHECK_EQ(eback.status.value, int(RpcErrc::UNAVAILABLE));
  CHECK(std::string(eback.status.category_name) == "RPC" && eback.GetString(0) == "try later");
}

// The function table: queries, removal, names, member functions, ad-hoc calls.
EUX_TEST(registry_queries_and_adhoc) {
  struct Counter {
    int total = 0;
    int add(int v) { return total += v; }
  } counter;
  RpcDispatcher d("table");
  CHECK_EQ(d.FunctionCount(), 0u);
  CHECK(!d.IsRegistered(function_id_t{1}));
  CHECK(!d.GetSignature(function_id_t{1}).has_value());
  CHECK(d.RegisterFunction(function_id_t{1}, &Counter::add, &counter, data::string("counter.add")));
  CHECK(d.RegisterFunction(function_id_t{2}, [](const data::vector<double>& v) { return double(v.size()); }, data::string("len")));
  CHECK(d.IsRegistered(function_id_t{1}) && d.IsRegistered(function_id_t{2}));
  CHECK_EQ(d.FunctionCount(), 2u);
  RpcRequestBuilder rb;
  CHECK_EQ(d.Dispatch(rb.PrepareRequest({{}, {}, function_id_t{1}}, int(5))).header.GetPrimitive<int>(0), 5);
  CHECK_EQ(d.Dispatch(rb.PrepareRequest({{}, {}, function_id_t{1}}, int(6))).header.GetPrimitive<int>(0), 11);
  CHECK_EQ(counter.total, 11);
  auto by_name = d.GetSignature("len");
  CHECK(by_name.has_value() && by_name->id.v_ == 2);
  CHECK((by_name->param_types == data::vector<ParamType>{ParamType::VECTOR_FLOAT64}));
  CHECK(!d.GetSignature("nothing").has_value());
  auto blob = d.GetAllSignatures();
  auto sigs = RpcDispatcher::DeserializeSignatures(blob.data(), blob.size());
  CHECK_EQ(sigs.size(), 2u);
  bool seen_add = false, seen_len = false;
  for (auto& sg : sigs) {
    seen_add = seen_add || (sg.function_name == "counter.add" && sg.id.v_ == 1 && sg.instance_name == "table");
    seen_len = seen_len || (sg.function_name == "len" && sg.return_types == data::vector<ParamType>{ParamType::PRIMITIVE_FLOAT64});
  }
  CHECK(seen_add && seen_len);
  CHECK(d.UnregisterFunction(function_id_t{1}));
  CHECK(!d.UnregisterFunction(function_id_t{1}));
  CHECK_EQ(d.FunctionCount(), 1u);
  CHECK_EQ(d.Dispatch(rb.PrepareRequest({{}, {}, function_id_t{1}}, int(1))).header.status.value, int(RpcErrc::NOT_FOUND));
  // a callable that was never registered, filled from the same header
  auto adhoc = d.DispatchAdhoc([](int32_t a, const data::string& s) { return data::string(s.str() + std::to_string(a)); },
                               rb.PrepareRequest({session_id_t{9}, request_id_t{8}, function_id_t{777}}, int32_t(4), data::string("n=")));
  CHECK(adhoc.header.status.ok() && adhoc.header.GetString(0) == "n=4");
  CHECK_EQ(adhoc.header.session_id.v_, 9u);
  CHECK_EQ(d.FunctionCount(), 1u);
}

// Every allocation made on behalf of a call is returned: a memory manager that counts.
EUX_TEST(dispatch_returns_all_memory) {
  struct Tracking : DefaultUcxMemoryResourceManager {
    std::atomic<long> live{0}, total{0};
    void* allocate(ucx_memory_type_t t, size_t n, size_t a = 8) override {
      ++live, ++total;
      return DefaultUcxMemoryResourceManager::allocate(t, n, a);
    }
    void deallocate(ucx_memory_type_t t, void* p, size_t n, size_t a = 8) override {
      if (p) --live;
      DefaultUcxMemoryResourceManager::deallocate(t, p, n, a);
    }
  } mr;
  {
    RpcDispatcher d("mem");
    d.RegisterFunction(function_id_t{1}, [&mr](const TensorMeta& m, const UcxBuffer& in) {
      UcxBufferVec out(mr, ucx_memory_type::HOST, std::vector<size_t>{in.size(), in.size() / 2});
      return std::tuple<int64_t, UcxBufferVec>(m.shape[0], std::move(out));
    }, data::string("split"));
    d.RegisterFunction(function_id_t{2}, [](UcxBufferVec taken) { return uint64_t(taken.size()); }, data::string("take"));
    TensorMeta m;
    m.ndim = 1;
    m.shape = {64};
    m.strides = {1};
    for (int round = 0; round < 50; ++round) {
      UcxBuffer in(mr, ucx_memory_type::HOST, 64);
      auto r = d.Dispatch(RpcRequestBuilder{}.PrepareRequest({{}, request_id_t{uint32_t(round)}, function_id_t{1}}, m), in);
      CHECK(r.header.status.ok());
      CHECK_EQ(std::get<UcxBufferVec>(r.payload).size(), 2u);
      auto r2 = d.DispatchMove(RpcRequestBuilder{}.PrepareRequest({{}, {}, function_id_t{2}}), std::move(std::get<UcxBufferVec>(r.payload)));
      CHECK_EQ(r2.header.GetPrimitive<uint64_t>(0), 2u);
      // a failing call must not keep anything either
      UcxBuffer unused(mr, ucx_memory_type::HOST, 8);
      CHECK(!d.Dispatch(RpcRequestBuilder{}.PrepareRequest({{}, {}, function_id_t{404}}), unused).header.status.ok());
    }
  }
  CHECK(mr.total.load() >= 200);
  CHECK_EQ(mr.live.load(), 0);
}

// The clock a request carries and the clock of its response, across a chain of services:
// A calls B, B calls C and D (fork), joins their answers and replies. Every effect is later than its cause.
EUX_TEST(hlc_causality_through_dispatch_chain) {
  using eux::rpc::utils::HybridLogicalClock;
  struct Node {
    HybridLogicalClock clock;
    RpcDispatcher disp;
    uint64_t wall;
    explicit Node(const char* name, uint64_t wall_ms) : clock(wall_ms, 0), disp(name), wall(wall_ms) {}
    HybridLogicalClock tick() {
      clock.TickLocal(wall);
      return clock;
    }
    HybridLogicalClock observe(HybridLogicalClock remote) {
      clock.Merge(remote, wall);
      return clock;
    }
  };
  // wall clocks disagree on purpose: C is 40 ms behind, D 15 ms ahead
  Node a("a", 10'000), b("b", 10'003), c("c", 9'960), dnode("d", 10'015);
  auto leaf = [](Node& n) {
    return [&n](const RpcRequestHeader& rq, int32_t v) {
      n.observe(rq.hlc);
      RpcResponseBuilder rb(n.tick());
      return rb.PrepareResponse(rq.session_id, rq.request_id, int32_t(v * 2));
    };
  };
  c.disp.RegisterFunction(function_id_t{1}, leaf(c), data::string("leaf"));
  dnode.disp.RegisterFunction(function_id_t{1}, leaf(dnode), data::string("leaf"));
  std::vector<uint64_t> order;  // raw clocks in causal order of one path
  b.disp.RegisterFunction(function_id_t{1}, [&](const RpcRequestHeader& rq, int32_t v) {
    order.push_back(b.observe(rq.hlc).Raw());
    RpcRequestBuilder rb;
    auto to_c = rb.PrepareRequest({rq.session_id, request_id_t{1}, function_id_t{1}, b.tick()}, v);
    auto to_d = rb.PrepareRequest({rq.session_id, request_id_t{2}, function_id_t{1}, b.tick()}, int32_t(v + 1));
    CHECK(to_d.hlc > to_c.hlc);
    auto from_c = c.disp.Dispatch(Serialize(to_c));
    auto from_d = dnode.disp.Dispatch(Serialize(to_d));
    CHECK(from_c.header.hlc > to_c.hlc);
    CHECK(from_d.header.hlc > to_d.hlc);
    b.observe(from_c.header.hlc);
    auto joined = b.observe(from_d.header.hlc);
    CHECK(joined > from_c.header.hlc && joined > from_d.header.hlc);
    order.push_back(joined.Raw());
    RpcResponseBuilder out(b.tick());
    return out.PrepareResponse(rq.session_id, rq.request_id, int32_t(from_c.header.GetPrimitive<int32_t>(0) + from_d.header.GetPrimitive<int32_t>(0)));
  }, data::string("fan_out"));
  HybridLogicalClock sent = a.tick();
  order.push_back(sent.Raw());
  auto reply = b.disp.Dispatch(Serialize(RpcRequestBuilder{}.PrepareRequest({session_id_t{1}, request_id_t{7}, function_id_t{1}, sent}, int32_t(5))));
  CHECK(reply.header.status.ok());
  CHECK_EQ(reply.header.GetPrimitive<int32_t>(0), 10 + 12);
  CHECK(reply.header.hlc > sent);
  order.push_back(reply.header.hlc.Raw());
  order.push_back(a.observe(reply.header.hlc).Raw());
  for (size_t i = 1; i < order.size(); ++i) CHECK(order[i] > order[i - 1]);
  // the node whose wall clock is behind never issued a stamp earlier than what it had seen
  CHECK(c.clock > sent);
  // hlc travels in the wire image
  auto req = RpcRequestBuilder{}.PrepareRequest({session_id_t{1}, request_id_t{1}, function_id_t{1}, HybridLogicalClock(123456, 7), workflow_id_t{44}}, int32_t(1));
  auto round = Deserialize<RpcRequestHeader>(Serialize(req));
  CHECK(round.hlc == HybridLogicalClock(123456, 7));
  CHECK_EQ(round.workflow_id.v_, 44u);
}

// Ordering, packing and merge rules of the clock on their own.
EUX_TEST(hybrid_logical_clock_rules) {
  using eux::rpc::utils::HybridLogicalClock;
  HybridLogicalClock z;
  CHECK_EQ(z.Raw(), 0u);
  HybridLogicalClock p(77, 3);
  CHECK(p.PhysicalTimeMs() == 77 && p.LogicalCounter() == 3);
  CHECK(HybridLogicalClock(p.Raw()) == p);
  CHECK(HybridLogicalClock(77, 4) > p && HybridLogicalClock(78, 0) > HybridLogicalClock(77, 0xffff));
  CHECK(p != HybridLogicalClock(77, 4));
  // local tick: wall clock ahead -> adopt it, counter 0; not ahead -> counter + 1
  HybridLogicalClock l(100, 9);
  l.TickLocal(150);
  CHECK(l == HybridLogicalClock(150, 0));
  l.TickLocal(150);
  CHECK(l == HybridLogicalClock(150, 1));
  l.TickLocal(120);  // the wall clock went backwards: the stamp does not
  CHECK(l == HybridLogicalClock(150, 2));
  // merge: the largest of local, remote and wall wins; ties on the physical part take the larger counter + 1
  HybridLogicalClock m(200, 5);
  m.Merge(HybridLogicalClock(200, 9), 100);
  CHECK(m == HybridLogicalClock(200, 10));
  m.Merge(HybridLogicalClock(150, 99), 100);  // an older remote: only the local counter moves
  CHECK(m == HybridLogicalClock(200, 11));
  m.Merge(HybridLogicalClock(300, 4), 100);  // a newer remote
  CHECK(m == HybridLogicalClock(300, 5));
  m.Merge(HybridLogicalClock(250, 0), 400);  // the wall clock is ahead of both
  CHECK(m == HybridLogicalClock(400, 0));
  m.Merge(m.Raw());  // raw form, real wall clock: never goes back
  CHECK(m.PhysicalTimeMs() >= 400);
  HybridLogicalClock r;
  r.AssignRaw((55ull << 16) | 6);
  CHECK(r == HybridLogicalClock(55, 6));
  // a long run of ticks under a frozen wall clock stays strictly increasing through the counter wrap
  HybridLogicalClock f(1, 0xfff0);
  uint64_t prev = f.Raw();
  for (int i = 0; i < 64; ++i) {
    f.TickLocal(1);
    CHECK(f.Raw() > prev);
    prev = f.Raw();
  }
  CHECK(f.PhysicalTimeMs() == 2);
}

EUX_TEST_MAIN()
