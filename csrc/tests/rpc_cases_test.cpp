// rpc_core, one behaviour per case: the dispatcher's argument and return kinds, its error answers, the
// builders, the status type and the hybrid logical clock. The behaviours are the ones the reference
// exercises in rpc_core/rpc_dispatcher_test.cpp:201-1425, async_rpc_dispatcher_test.cpp,
// rpc_request_builder_test.cpp, rpc_response_builder_test.cpp and utils/hybrid_logical_clock_test.cpp;
// the cases are written against this implementation's own types.
#include <cstring>
#include <string>

#include "check.hpp"
#include "eux/exec/contexts.hpp"
#include "eux/rpc/async_rpc_dispatcher.hpp"

using namespace eux::rpc;
using eux::rpc::utils::HybridLogicalClock;
using eux::ucxx::DefaultUcxMemoryResourceManager;
using eux::ucxx::UcxBuffer;
using eux::ucxx::UcxBufferVec;
using eux::ucxx::UcxHeader;
namespace ex = eux::exec;

namespace {
RpcRequestBuilderOptions opt(uint32_t fn, uint32_t session = 1, uint32_t request = 1) {
  return {session_id_t{session}, request_id_t{request}, function_id_t{fn}};
}
int32_t add(int32_t a, int32_t b) { return a + b; }
struct Calculator {
  int32_t base = 100;
  int32_t plus(int32_t x) { return base + x; }
};
}  // namespace

// ---- dispatcher: registration and lookups --------------------------------------------------------
EUX_TEST(registration_rejects_a_taken_id) {
  RpcDispatcher d("svc");
  CHECK(d.RegisterFunction(function_id_t{1}, &add, data::string("add")));
  CHECK(!d.RegisterFunction(function_id_t{1}, &add, data::string("add_again")));
  CHECK(d.IsRegistered(function_id_t{1}) && !d.IsRegistered(function_id_t{2}));
  CHECK_EQ(d.FunctionCount(), 1u);
}

EUX_TEST(signature_is_derived_from_the_callable) {
  RpcDispatcher d("svc");
  d.RegisterFunction(function_id_t{7}, [](int64_t, double, const data::string&, bool) -> float { return 0.f; }, data::string("mixed"));
  auto sig = d.GetSignature(function_id_t{7});
  CHECK(sig.has_value());
  CHECK((sig->param_types == data::vector<ParamType>{ParamType::PRIMITIVE_INT64, ParamType::PRIMITIVE_FLOAT64, ParamType::STRING, ParamType::PRIMITIVE_BOOL}));
  CHECK((sig->return_types == data::vector<ParamType>{ParamType::PRIMITIVE_FLOAT32}));
  CHECK(sig->function_name == "mixed" && sig->instance_name == "svc" && sig->id.v_ == 7u);
  CHECK(sig->input_payload_type == PayloadType::NO_PAYLOAD && sig->return_payload_type == PayloadType::NO_PAYLOAD);
  CHECK(!d.GetSignature(function_id_t{8}).has_value());
}

// ---- dispatcher: argument kinds ----------------------------------------------------------------------
EUX_TEST(dispatch_simple_function_from_bytes_and_from_header) {
  RpcDispatcher d("svc");
  d.RegisterFunction(function_id_t{1}, &add, data::string("add"));
  auto req = RpcRequestBuilder{}.PrepareRequest(opt(1, 11, 22), int32_t(40), int32_t(2));
  auto from_bytes = d.Dispatch<std::monostate>(Serialize(req));
  auto from_header = d.Dispatch(req);
  for (auto* r : {&from_bytes.header, &from_header.header}) {
    CHECK(r->status.ok());
    CHECK_EQ(r->GetPrimitive<int32_t>(0), 42);
    CHECK(r->session_id.v_ == 11u && r->request_id.v_ == 22u);
  }
}

EUX_TEST(dispatch_void_function_returns_no_results) {
  RpcDispatcher d("svc");
  int calls = 0;
  d.RegisterFunction(function_id_t{2}, [&calls](int32_t n) { calls += n; }, data::string("bump"));
  auto r = d.Dispatch(RpcRequestBuilder{}.PrepareRequest(opt(2), int32_t(5)));
  CHECK(r.header.status.ok());
  CHECK_EQ(r.header.results.size(), 0u);
  CHECK_EQ(calls, 5);
}

EUX_TEST(dispatch_string_function) {
  RpcDispatcher d("svc");
  d.RegisterFunction(function_id_t{3}, [](const data::string& who) { return data::string("Hello, " + who.str() + "!"); }, data::string("greet"));
  auto r = d.Dispatch(RpcRequestBuilder{}.PrepareRequest(opt(3), data::string("a rather long name that does not fit the short-string form")));
  CHECK(r.header.status.ok());
  CHECK(r.header.GetString(0) == "Hello, a rather long name that does not fit the short-string form!");
}

EUX_TEST(dispatch_vector_function) {
  RpcDispatcher d("svc");
  d.RegisterFunction(function_id_t{4}, [](const data::vector<int32_t>& v) {
    data::vector<int32_t> out;
    for (auto x : v) out.push_back(x * 2);
    return out;
  }, data::string("double_all"));
  auto r = d.Dispatch(RpcRequestBuilder{}.PrepareRequest(opt(4), data::vector<int32_t>{1, 2, 3}));
  CHECK(r.header.status.ok());
  CHECK((r.header.GetVector<int32_t>(0) == data::vector<int32_t>{2, 4, 6}));
}

EUX_TEST(dispatch_member_function_through_a_lambda) {
  RpcDispatcher d("svc");
  Calculator calc;
  d.RegisterFunction(function_id_t{5}, [&calc](int32_t x) { return calc.plus(x); }, data::string("plus"));
  calc.base = 7;
  CHECK_EQ(d.Dispatch(RpcRequestBuilder{}.PrepareRequest(opt(5), int32_t(3))).header.GetPrimitive<int32_t>(0), 10);
}

EUX_TEST(handler_may_read_the_request_header) {
  RpcDispatcher d("svc");
  d.RegisterFunction(function_id_t{6}, [](const RpcRequestHeader& h, int32_t x) { return int64_t(h.session_id.v_) * 1000 + h.workflow_id.v_ + x; },
                     data::string("echo_ids"));
  auto req = RpcRequestBuilder{}.PrepareRequest({session_id_t{9}, request_id_t{1}, function_id_t{6}, {}, utils::workflow_id_t{50}}, int32_t(4));
  CHECK_EQ(d.Dispatch(req).header.GetPrimitive<int64_t>(0), 9054);
}

EUX_TEST(tensor_metadata_is_a_parameter_kind) {
  RpcDispatcher d("svc");
  d.RegisterFunction(function_id_t{8}, [](const TensorMeta& m) { return int64_t(utils::CalculateTensorSize(m)); }, data::string("nbytes"));
  TensorMeta m;
  m.ndim = 2;
  m.dtype = {kDLFloat, 32, 1};
  m.shape = {3, 5};
  m.strides = {5, 1};
  auto r = d.Dispatch(RpcRequestBuilder{}.PrepareRequest(opt(8), m));
  CHECK_EQ(r.header.GetPrimitive<int64_t>(0), 60);
  auto sig = d.GetSignature(function_id_t{8});
  CHECK((sig->param_types == data::vector<ParamType>{ParamType::TENSOR_META}));
}

EUX_TEST(payload_by_reference_is_seen_in_place) {
  DefaultUcxMemoryResourceManager mr;
  RpcDispatcher d("svc");
  d.RegisterFunction(function_id_t{9}, [](UcxBuffer& b) {
    auto* p = static_cast<unsigned char*>(b.data());
    for (size_t i = 0; i < b.size(); ++i) p[i] = static_cast<unsigned char>(p[i] + 1);
    return uint64_t(b.size());
  }, data::string("inc_bytes"));
  UcxBuffer buf(mr, ucx_memory_type::HOST, 8);
  std::memset(buf.data(), 7, 8);
  PayloadVariant pv(std::move(buf));
  auto r = d.Dispatch(RpcRequestBuilder{}.PrepareRequest(opt(9)), pv);
  CHECK(r.header.status.ok());
  CHECK_EQ(r.header.GetPrimitive<uint64_t>(0), uint64_t(8));
  CHECK_EQ(static_cast<unsigned char*>(std::get<UcxBuffer>(pv).data())[3], 8);
  CHECK(d.GetSignature(function_id_t{9})->input_payload_type == PayloadType::UCX_BUFFER);
}

EUX_TEST(payload_by_rvalue_reference_and_by_value_is_handed_over_whole) {
  // both forms take the payload over; the function must see the caller's bytes, not a moved-from temporary
  DefaultUcxMemoryResourceManager mr;
  RpcDispatcher d("svc");
  d.RegisterFunction(function_id_t{1}, [](UcxBuffer&& b) { return std::tuple<uint64_t, UcxBuffer>(b.size(), std::move(b)); }, data::string("take_rref"));
  d.RegisterFunction(function_id_t{2}, [](UcxBuffer b) { return std::tuple<uint64_t, UcxBuffer>(b.size(), std::move(b)); }, data::string("take_value"));
  d.RegisterFunction(function_id_t{3}, [](const RpcRequestHeader&, PayloadVariant&& v) { return uint64_t(std::get<UcxBuffer>(v).size()); }, data::string("take_variant"));
  for (uint32_t id : {1u, 2u}) {
    UcxBuffer buf(mr, ucx_memory_type::HOST, 24);
    std::memset(buf.data(), int(id), 24);
    auto r = d.DispatchMove(RpcRequestBuilder{}.PrepareRequest(opt(id)), std::move(buf));
    CHECK(r.header.status.ok());
    CHECK_EQ(r.header.GetPrimitive<uint64_t>(0), uint64_t(24));
    CHECK_EQ(std::get<UcxBuffer>(r.payload).size(), size_t(24));
    CHECK_EQ(static_cast<unsigned char*>(std::get<UcxBuffer>(r.payload).data())[23], id);
  }
  PayloadVariant pv(UcxBuffer(mr, ucx_memory_type::HOST, 5));
  auto r3 = d.DispatchMove(RpcRequestBuilder{}.PrepareRequest(opt(3)), std::move(pv));
  CHECK(r3.header.status.ok());
  CHECK_EQ(r3.header.GetPrimitive<uint64_t>(0), uint64_t(5));
  // without permission to move, a taking function is refused instead of being handed a copy
  UcxBuffer keep(mr, ucx_memory_type::HOST, 8);
  auto refused = d.Dispatch(RpcRequestBuilder{}.PrepareRequest(opt(1)), keep);
  CHECK_EQ(refused.header.status.value, int(RpcErrc::INVALID_ARGUMENT));
  CHECK_EQ(keep.size(), size_t(8));
}

EUX_TEST(buffer_vector_payload_and_returned_buffer_vector) {
  DefaultUcxMemoryResourceManager mr;
  RpcDispatcher d("svc");
  d.RegisterFunction(function_id_t{10}, [&mr](const UcxBufferVec& in) {
    std::vector<size_t> sizes;
    for (size_t i = 0; i < in.size(); ++i) sizes.push_back(in[i].size * 2);
    return UcxBufferVec(mr, ucx_memory_type::HOST, sizes);
  }, data::string("twice_as_large"));
  PayloadVariant pv(UcxBufferVec(mr, ucx_memory_type::HOST, std::vector<size_t>{4, 10}));
  auto r = d.Dispatch<UcxBufferVec>(RpcRequestBuilder{}.PrepareRequest(opt(10)), pv);
  CHECK(r.header.status.ok());
  CHECK(r.payload.size() == 2 && r.payload[0].size == 8 && r.payload[1].size == 20);
  auto sig = d.GetSignature(function_id_t{10});
  CHECK(sig->input_payload_type == PayloadType::UCX_BUFFER_VEC && sig->return_payload_type == PayloadType::UCX_BUFFER_VEC);
}

// ---- dispatcher: return kinds -------------------------------------------------------------------------
EUX_TEST(tuple_return_becomes_several_results) {
  RpcDispatcher d("svc");
  d.RegisterFunction(function_id_t{11}, [](int32_t x) { return std::tuple<int32_t, data::string, double>(x, data::string("s" + std::to_string(x)), x / 2.0); },
                     data::string("triple"));
  auto r = d.Dispatch(RpcRequestBuilder{}.PrepareRequest(opt(11), int32_t(5)));
  CHECK_EQ(r.header.results.size(), 3u);
  CHECK_EQ(r.header.GetPrimitive<int32_t>(0), 5);
  CHECK(r.header.GetString(1) == "s5");
  CHECK_EQ(r.header.GetPrimitive<double>(2), 2.5);
  CHECK((d.GetSignature(function_id_t{11})->return_types == data::vector<ParamType>{ParamType::PRIMITIVE_INT32, ParamType::STRING, ParamType::PRIMITIVE_FLOAT64}));
}

EUX_TEST(handler_may_return_a_whole_response_header) {
  RpcDispatcher d("svc");
  d.RegisterFunction(function_id_t{12}, [](const RpcRequestHeader& rq, const RpcResponseBuilder& b) {
    RpcResponseHeader h = b.PrepareResponse(rq.session_id, rq.request_id, int32_t(1), int32_t(2));
    h.workflow_id = utils::workflow_id_t{77};
    return h;
  }, data::string("manual"));
  auto r = d.Dispatch(RpcRequestBuilder{}.PrepareRequest(opt(12, 3, 4)));
  CHECK(r.header.status.ok());
  CHECK(r.header.results.size() == 2 && r.header.workflow_id.v_ == 77u && r.header.session_id.v_ == 3u && r.header.request_id.v_ == 4u);
}

EUX_TEST(handler_may_return_a_status_of_its_own) {
  RpcDispatcher d("svc");
  d.RegisterFunction(function_id_t{13}, [](const RpcRequestHeader& rq, const RpcResponseBuilder& b) {
    return b.PrepareError(rq.session_id, rq.request_id, make_error_code(RpcErrc::PERMISSION_DENIED), "not for you");
  }, data::string("deny"));
  auto r = d.Dispatch(RpcRequestBuilder{}.PrepareRequest(opt(13)));
  CHECK_EQ(r.header.status.value, int(RpcErrc::PERMISSION_DENIED));
  CHECK(r.header.GetString(0) == "not for you");
  std::error_code ec = r.header.status;
  CHECK(ec == make_error_code(RpcErrc::PERMISSION_DENIED));
}

// ---- dispatcher: errors -----------------------------------------------------------------------------------
EUX_TEST(unknown_function_is_answered_with_not_found) {
  RpcDispatcher d("svc");
  auto r = d.Dispatch(RpcRequestBuilder{}.PrepareRequest(opt(404, 7, 8)));
  CHECK_EQ(r.header.status.value, int(RpcErrc::NOT_FOUND));
  CHECK(r.header.session_id.v_ == 7u && r.header.request_id.v_ == 8u);
  CHECK(r.header.GetString(0).str().find("404") != std::string::npos);
}

EUX_TEST(wrong_argument_type_and_count_are_refused) {
  RpcDispatcher d("svc");
  d.RegisterFunction(function_id_t{1}, &add, data::string("add"));
  for (auto req : {RpcRequestBuilder{}.PrepareRequest(opt(1, 110), int32_t(1), 2.5), RpcRequestBuilder{}.PrepareRequest(opt(1, 110), int32_t(1)),
                   RpcRequestBuilder{}.PrepareRequest(opt(1, 110), data::string("not a number"), int32_t(1))}) {
    auto r = d.Dispatch<std::monostate>(Serialize(req));
    CHECK(!r.header.status.ok());
    CHECK(std::string(r.header.status.category_name) == "RPC");
    CHECK_EQ(r.header.session_id.v_, 110u);
    CHECK(!r.header.GetString(0).empty());  // says what was wrong
  }
}

EUX_TEST(rpc_exception_keeps_its_code_and_text) {
  RpcDispatcher d("svc");
  d.RegisterFunction(function_id_t{14}, [](int32_t) -> int32_t { throw RpcException(RpcErrc::RESOURCE_EXHAUSTED, "queue is full"); }, data::string("full"));
  auto r = d.Dispatch(RpcRequestBuilder{}.PrepareRequest(opt(14), int32_t(0)));
  CHECK_EQ(r.header.status.value, int(RpcErrc::RESOURCE_EXHAUSTED));
  CHECK(std::string(r.header.status.category_name) == "RPC");
  CHECK(r.header.GetString(0) == "queue is full");
}

EUX_TEST(garbage_bytes_do_not_reach_a_handler) {
  RpcDispatcher d("svc");
  bool called = false;
  d.RegisterFunction(function_id_t{1}, [&called](int32_t) { called = true; }, data::string("f"));
  bool refused = false;
  try {
    byte_buf junk(7, uint8_t(0x5a));
    refused = !d.Dispatch<std::monostate>(std::move(junk)).header.status.ok();
  } catch (const std::exception&) {
    refused = true;  // the image is checked while it is read: too short to be a header
  }
  CHECK(refused && !called);
}

// ---- dynamic registration and the response wire form --------------------------------------------
EUX_TEST(dynamic_function_sees_params_and_payload) {
  DefaultUcxMemoryResourceManager mr;
  RpcDispatcher d("svc");
  d.RegisterFunction(function_id_t{20}, data::string("dyn"), {ParamType::PRIMITIVE_INT32, ParamType::STRING}, {ParamType::STRING}, PayloadType::UCX_BUFFER,
                     PayloadType::NO_PAYLOAD, [](const RpcRequestHeader& rq, RpcContextPtr ctx, const RpcResponseBuilder& b) -> DynamicRpcResult {
                       const UcxBuffer* in = ctx.get<UcxBuffer>();
                       const size_t n = in ? in->size() : 0;
                       return {b.PrepareResponse(rq.session_id, rq.request_id,
                                                 data::string(rq.GetString(1).str() + ":" + std::to_string(rq.GetPrimitive<int32_t>(0)) + ":" + std::to_string(n))),
                               ReturnedPayload{}};
                     });
  PayloadVariant pv(UcxBuffer(mr, ucx_memory_type::HOST, 33));
  auto r = d.Dispatch(RpcRequestBuilder{}.PrepareRequest(opt(20), int32_t(4), data::string("k")), pv);
  CHECK(r.header.status.ok());
  CHECK(r.header.GetString(0) == "k:4:33");
  auto sig = d.GetSignature(function_id_t{20});
  CHECK(sig->function_name == "dyn" && sig->input_payload_type == PayloadType::UCX_BUFFER);
}

EUX_TEST(response_serialises_into_a_caller_supplied_buffer) {
  RpcResponseHeader h = RpcResponseBuilder{}.PrepareResponse(session_id_t{5}, request_id_t{6}, int32_t(7), data::string("a string long enough to live outside the short form"));
  const size_t need = GetSerializedSize(h);
  std::vector<uint8_t> buf(need);
  FixedBufferWriter w(buf.data(), buf.size());
  CHECK_EQ(RpcDispatcher::SerializeResponse(h, w), need);
  CHECK(std::memcmp(buf.data(), RpcDispatcher::SerializeResponse(h).data(), need) == 0);
  std::vector<uint8_t> small(need - 1);
  FixedBufferWriter tight(small.data(), small.size());
  CHECK_THROWS(RpcDispatcher::SerializeResponse(h, tight));
  // no results at all: still a complete image
  RpcResponseHeader empty = RpcResponseBuilder{}.PrepareResponse(session_id_t{1}, request_id_t{2});
  auto bytes = RpcDispatcher::SerializeResponse(empty);
  auto back = Deserialize<RpcResponseHeader>(bytes.data(), bytes.size());
  CHECK(back.results.size() == 0 && back.session_id.v_ == 1u && back.request_id.v_ == 2u && back.status.ok());
}

EUX_TEST(deserialised_response_owns_the_received_header_bytes) {
  DefaultUcxMemoryResourceManager mr;
  RpcResponseHeader h = RpcResponseBuilder{}.PrepareResponse(session_id_t{3}, request_id_t{4}, data::vector<double>{1.5, 2.5}, data::string("tail"));
  auto bytes = Serialize(h);
  UcxHeader wire(mr, bytes.size());
  std::memcpy(wire.data(), bytes.data(), bytes.size());
  RpcResponseHeader back = RpcDispatcher::DeerializeResponse(std::move(wire));
  CHECK(back.session_id.v_ == 3u && back.request_id.v_ == 4u);
  CHECK((back.GetVector<double>(0) == data::vector<double>{1.5, 2.5}));
  CHECK(back.GetString(1) == "tail");
}

// ---- builders ----------------------------------------------------------------------------------------------
EUX_TEST(request_builder_packs_every_scalar_kind) {
  auto req = RpcRequestBuilder{}.PrepareRequest(opt(1), true, int8_t(-1), int16_t(-2), int32_t(-3), int64_t(-4), uint8_t(1), uint16_t(2), uint32_t(3),
                                                uint64_t(4), 1.5f, 2.5);
  const ParamType want[] = {ParamType::PRIMITIVE_BOOL,  ParamType::PRIMITIVE_INT8,   ParamType::PRIMITIVE_INT16,  ParamType::PRIMITIVE_INT32,
                            ParamType::PRIMITIVE_INT64, ParamType::PRIMITIVE_UINT8,  ParamType::PRIMITIVE_UINT16, ParamType::PRIMITIVE_UINT32,
                            ParamType::PRIMITIVE_UINT64, ParamType::PRIMITIVE_FLOAT32, ParamType::PRIMITIVE_FLOAT64};
  CHECK_EQ(req.params.size(), 11u);
  for (size_t i = 0; i < 11; ++i) CHECK(req.params[i].type == want[i]);
  CHECK(req.GetPrimitive<bool>(0) && req.GetPrimitive<int64_t>(4) == -4 && req.GetPrimitive<uint64_t>(8) == 4u && req.GetPrimitive<double>(10) == 2.5);
}

EUX_TEST(request_builder_separates_the_payload) {
  DefaultUcxMemoryResourceManager mr;
  UcxBuffer buf(mr, ucx_memory_type::HOST, 64);
  void* where = buf.data();
  auto [req, payload] = RpcRequestBuilder{}.PrepareRequest(opt(2), int32_t(9), std::move(buf), data::string("after"));
  CHECK_EQ(req.params.size(), 2u);  // the payload is not a parameter
  CHECK(req.GetString(1) == "after");
  CHECK(std::holds_alternative<UcxBuffer>(payload) && std::get<UcxBuffer>(payload).data() == where);
}

EUX_TEST(request_builder_checks_against_a_signature) {
  RpcDispatcher d("svc");
  d.RegisterFunction(function_id_t{1}, &add, data::string("add"));
  auto sig = *d.GetSignature(function_id_t{1});
  RpcRequestBuilder rb;
  CHECK_THROWS(rb.PrepareRequest(sig, {}, int32_t(1)));
  CHECK_THROWS(rb.PrepareRequest(sig, {}, int64_t(1), int64_t(2)));
  auto ok = rb.PrepareRequest(sig, {session_id_t{4}}, int32_t(1), int32_t(2));
  CHECK(ok.function_id.v_ == 1u && ok.session_id.v_ == 4u);
}

EUX_TEST(request_builder_takes_prepared_params) {
  data::vector<ParamMeta> ps;
  ps.emplace_back(int32_t(5));
  ps.emplace_back(data::string("five"));
  auto req = RpcRequestBuilder{}.PrepareRequest(opt(3), std::move(ps));
  CHECK(req.params.size() == 2 && req.GetPrimitive<int32_t>(0) == 5 && req.GetString(1) == "five");
}

EUX_TEST(response_builder_forms) {
  DefaultUcxMemoryResourceManager mr;
  RpcResponseBuilder b;
  auto none = b.PrepareResponse(session_id_t{1}, request_id_t{2});
  CHECK(none.results.size() == 0 && none.status.ok());
  auto some = b.PrepareResponse(session_id_t{1}, request_id_t{2}, int32_t(3), data::vector<uint8_t>{1, 2}, data::string("x"));
  CHECK(some.results.size() == 3 && some.results[1].type == ParamType::VECTOR_UINT8);
  auto [h, payload] = b.PrepareResponse(session_id_t{1}, request_id_t{2}, int32_t(3), UcxBuffer(mr, ucx_memory_type::HOST, 12));
  CHECK(h.results.size() == 1 && std::holds_alternative<UcxBuffer>(payload) && std::get<UcxBuffer>(payload).size() == 12);
  auto err = b.PrepareError(session_id_t{1}, request_id_t{2}, make_error_code(RpcErrc::UNAVAILABLE), "gone");
  CHECK(!err.status.ok() && err.GetString(0) == "gone");
}

// ---- RpcStatus ---------------------------------------------------------------------------------------------
EUX_TEST(status_default_is_ok) {
  RpcStatus s;
  CHECK(s.ok() && s.value == 0);
  std::error_code ec = s;
  CHECK(!ec);
}

EUX_TEST(status_converts_to_and_from_error_codes) {
  RpcStatus s(make_error_code(RpcErrc::DEADLINE_EXCEEDED));
  CHECK(!s.ok() && std::string(s.category_name) == "RPC");
  std::error_code ec = s;
  CHECK(ec == make_error_code(RpcErrc::DEADLINE_EXCEEDED));
  CHECK(!s.GetErrorMessage().empty());
  RpcStatus g(std::make_error_code(std::errc::timed_out));
  std::error_code back = g;
  CHECK(back == std::make_error_code(std::errc::timed_out));
}

EUX_TEST(status_of_a_third_party_category) {
  struct Cat final : std::error_category {
    const char* name() const noexcept override { return "storage-engine"; }
    std::string message(int v) const override { return v == 3 ? "disk full" : "?"; }
  };
  static Cat cat;
  RpcStatus before(std::error_code(3, cat));
  CHECK(std::string(before.category_name) == "storage-engine");
  // unknown on this side until registered: the number survives, the meaning does not
  CHECK(static_cast<std::error_code>(before).category() == std::generic_category());
  RpcCategoryRegistry::GetInstance().RegisterCategory(cat);
  std::error_code ec = before;
  CHECK(&ec.category() == &cat && ec.message() == "disk full");
  CHECK(before.GetErrorMessage() == "disk full");
}

// ---- async dispatcher ---------------------------------------------------------------------------------
EUX_TEST(async_handler_value_error_and_void) {
  ex::static_thread_pool pool(2);
  AsyncRpcDispatcher d("async");
  int side = 0;
  d.RegisterFunction(function_id_t{1}, [&](int32_t a) { return ex::on(pool.get_scheduler(), ex::just(a * 3)); }, data::string("triple"));
  d.RegisterFunction(function_id_t{2}, [&](int32_t a) { return ex::on(pool.get_scheduler(), ex::just_from([&side, a] { side = a; })); }, data::string("store"));
  d.RegisterFunction(function_id_t{3}, [](int32_t) -> int32_t { throw RpcException(RpcErrc::ABORTED, "stop"); }, data::string("abort"));
  RpcRequestBuilder rb;
  auto r1 = ex::sync_wait(d.Dispatch(rb.PrepareRequest(opt(1), int32_t(4))));
  CHECK(r1 && r1->header.GetPrimitive<int32_t>(0) == 12);
  auto r2 = ex::sync_wait(d.Dispatch(rb.PrepareRequest(opt(2), int32_t(9))));
  CHECK(r2 && r2->header.status.ok() && r2->header.results.size() == 0 && side == 9);
  auto r3 = ex::sync_wait(d.Dispatch(rb.PrepareRequest(opt(3), int32_t(0))));
  CHECK(r3 && r3->header.status.value == int(RpcErrc::ABORTED) && r3->header.GetString(0) == "stop");
  auto r4 = ex::sync_wait(d.Dispatch(rb.PrepareRequest(opt(99))));
  CHECK(r4 && r4->header.status.value == int(RpcErrc::NOT_FOUND));
}

// Every kind of return value the synchronous dispatcher takes, through the asynchronous one, plain and as the
// value of a sender. The wire's own containers (string, vector) have a nested value_type like a sender has: they
// are values all the same.
EUX_TEST(async_handlers_return_every_kind_of_value) {
  DefaultUcxMemoryResourceManager mr;
  AsyncRpcDispatcher d("async");
  TensorMeta m;
  m.ndim = 2;
  m.dtype = {kDLFloat, 32, 1};
  m.shape = {2, 3};
  m.strides = {3, 1};
  d.RegisterFunction(function_id_t{1}, [](const data::string& s) { return data::string(s.str() + "!"); }, data::string("string"));
  d.RegisterFunction(function_id_t{2}, [](int32_t n) {
    data::vector<double> v;
    for (int32_t i = 0; i < n; ++i) v.push_back(i * 0.5);
    return v;
  }, data::string("doubles"));
  d.RegisterFunction(function_id_t{3}, [](const data::vector<bool>& v) {
    data::vector<bool> out;
    for (auto b : v) out.push_back(!bool(b));
    return out;
  }, data::string("flip"));
  d.RegisterFunction(function_id_t{4}, [m](int32_t) { return m; }, data::string("meta"));
  d.RegisterFunction(function_id_t{5}, [m](int32_t n) { return TensorMetaVec(size_t(n), m); }, data::string("metas"));
  d.RegisterFunction(function_id_t{6}, [](int32_t x) { return std::tuple<data::string, int64_t, bool>(data::string("t"), int64_t(x) * 2, x > 0); }, data::string("tuple"));
  d.RegisterFunction(function_id_t{7}, [](int32_t x) { return x > 3; }, data::string("bool"));
  d.RegisterFunction(function_id_t{8}, [](const data::string& s) { return ex::just(data::string(s.str() + "?")); }, data::string("later_string"));
  d.RegisterFunction(function_id_t{9}, [](int32_t n) { return ex::just(data::vector<int64_t>(size_t(n), int64_t(7))); }, data::string("later_vector"));
  d.RegisterFunction(function_id_t{10}, [&mr, m](int32_t) {
    UcxBuffer out(mr, ucx_memory_type::HOST, 24);
    std::memset(out.data(), 5, 24);
    return std::tuple<TensorMeta, UcxBuffer>(m, std::move(out));
  }, data::string("tensor"));
  d.RegisterFunction(function_id_t{11}, [](const RpcRequestHeader& rq, const RpcResponseBuilder& b) { return b.PrepareResponse(rq.session_id, rq.request_id, int32_t(1), data::string("two")); },
                     data::string("header"));
  RpcRequestBuilder rb;
  auto call = [&](uint32_t fn, auto&&... args) { return ex::sync_wait(d.Dispatch(rb.PrepareRequest(opt(fn), std::forward<decltype(args)>(args)...))); };
  auto r1 = call(1, data::string("hi"));
  CHECK(r1 && r1->header.status.ok() && r1->header.GetString(0) == "hi!");
  auto r2 = call(2, int32_t(3));
  CHECK(r2 && (r2->header.GetVector<double>(0) == data::vector<double>{0.0, 0.5, 1.0}));
  auto r3 = call(3, data::vector<bool>{true, false, true});
  CHECK(r3 && (r3->header.GetVector<bool>(0) == data::vector<bool>{false, true, false}));
  auto r4 = call(4, int32_t(0));
  CHECK(r4 && r4->header.GetTensor(0) == m);
  auto r5 = call(5, int32_t(3));
  CHECK(r5 && r5->header.GetTensorVec(0).size() == 3u);
  auto r6 = call(6, int32_t(21));
  CHECK(r6 && r6->header.results.size() == 3u && r6->header.GetString(0) == "t" && r6->header.GetPrimitive<int64_t>(1) == 42 && r6->header.GetPrimitive<bool>(2));
  auto r7 = call(7, int32_t(4));
  CHECK(r7 && r7->header.GetPrimitive<bool>(0));
  auto r8 = call(8, data::string("well"));
  CHECK(r8 && r8->header.GetString(0) == "well?");
  auto r9 = call(9, int32_t(2));
  CHECK(r9 && (r9->header.GetVector<int64_t>(0) == data::vector<int64_t>{7, 7}));
  auto r10 = call(10, int32_t(0));
  CHECK(r10 && r10->header.GetTensor(0) == m && std::get<UcxBuffer>(r10->payload).size() == 24u);
  auto r11 = call(11);
  CHECK(r11 && r11->header.GetPrimitive<int32_t>(0) == 1 && r11->header.GetString(1) == "two");
  auto sig = d.GetSignature(function_id_t{1});
  CHECK(sig && (sig->return_types == data::vector<ParamType>{ParamType::STRING}));
  sig = d.GetSignature(function_id_t{9});
  CHECK(sig && (sig->return_types == data::vector<ParamType>{ParamType::VECTOR_INT64}));
}

// ... and every kind of argument: by value, by reference, the request itself, the builder, payloads taken over.
EUX_TEST(async_handlers_take_every_kind_of_argument) {
  DefaultUcxMemoryResourceManager mr;
  AsyncRpcDispatcher d("async");
  d.RegisterFunction(function_id_t{1}, [](bool b, int8_t a, uint16_t c, int64_t e, float f, double g) { return int64_t(b) + a + c + e + int64_t(f) + int64_t(g); },
                     data::string("numbers"));
  d.RegisterFunction(function_id_t{2}, [](const data::string& s, const data::vector<int32_t>& v) { return int64_t(s.size() + v.size()); }, data::string("by_reference"));
  d.RegisterFunction(function_id_t{3}, [](data::string s, data::vector<uint8_t> v) { return int64_t(s.size() * 10 + v.size()); }, data::string("by_value"));
  d.RegisterFunction(function_id_t{4}, [](const RpcRequestHeader& rq, const TensorMetaVec& metas, UcxBufferVec& bufs, const RpcResponseBuilder& b) {
    return b.PrepareResponse(rq.session_id, rq.request_id, int64_t(metas.size()), int64_t(bufs.size()), int64_t(bufs[1].size));
  }, data::string("vec"));
  d.RegisterFunction(function_id_t{5}, [](const TensorMeta& m, UcxBuffer buf) { return int64_t(utils::CalculateTensorSize(m) + buf.size()); }, data::string("taken"));
  d.RegisterFunction(function_id_t{6}, [](int32_t k, PayloadVariant&& any) { return int64_t(k) + int64_t(any.index()); }, data::string("variant"));
  RpcRequestBuilder rb;
  auto r1 = ex::sync_wait(d.Dispatch(rb.PrepareRequest(opt(1), true, int8_t(-2), uint16_t(300), int64_t(1) << 40, 2.5f, 7.9)));
  CHECK(r1 && r1->header.status.ok() && r1->header.GetPrimitive<int64_t>(0) == 1 - 2 + 300 + (int64_t(1) << 40) + 2 + 7);
  auto r2 = ex::sync_wait(d.Dispatch(rb.PrepareRequest(opt(2), data::string("abc"), data::vector<int32_t>{1, 2})));
  CHECK(r2 && r2->header.GetPrimitive<int64_t>(0) == 5);
  auto r3 = ex::sync_wait(d.Dispatch(rb.PrepareRequest(opt(3), data::string("ab"), data::vector<uint8_t>{1, 2, 3})));
  CHECK(r3 && r3->header.GetPrimitive<int64_t>(0) == 23);
  TensorMeta m;
  m.ndim = 1;
  m.dtype = {kDLUInt, 8, 1};
  m.shape = {4};
  m.strides = {1};
  {
    auto [req, payload] = rb.PrepareRequest(opt(4), TensorMetaVec{m, m}, UcxBufferVec(mr, ucx_memory_type::HOST, std::vector<size_t>{4, 6}));
    auto r = ex::sync_wait(d.Dispatch(req, std::move(payload)));
    CHECK(r && r->header.status.ok() && r->header.GetPrimitive<int64_t>(0) == 2 && r->header.GetPrimitive<int64_t>(1) == 2 && r->header.GetPrimitive<int64_t>(2) == 6);
  }
  {
    auto [req, payload] = rb.PrepareRequest(opt(5), m, UcxBuffer(mr, ucx_memory_type::HOST, 4));
    auto r = ex::sync_wait(d.Dispatch(req, std::move(payload)));
    CHECK(r && r->header.status.ok() && r->header.GetPrimitive<int64_t>(0) == 8);
  }
  {
    auto [req, payload] = rb.PrepareRequest(opt(6), int32_t(10), UcxBuffer(mr, ucx_memory_type::HOST, 4));
    auto r = ex::sync_wait(d.Dispatch(req, std::move(payload)));
    CHECK(r && r->header.status.ok() && r->header.GetPrimitive<int64_t>(0) == 11);
  }
  // a description that does not fit its payload never reaches the function
  {
    TensorMeta big = m;
    big.shape = {400};
    auto [req, payload] = rb.PrepareRequest(opt(5), big, UcxBuffer(mr, ucx_memory_type::HOST, 4));
    auto r = ex::sync_wait(d.Dispatch(req, std::move(payload)));
    CHECK(r && r->header.status.value == int(RpcErrc::INVALID_ARGUMENT));
  }
}

EUX_TEST(async_handler_with_payload_in_and_out) {
  DefaultUcxMemoryResourceManager mr;
  ex::static_thread_pool pool(1);
  AsyncRpcDispatcher d("async");
  d.RegisterFunction(function_id_t{1}, [&](const TensorMeta& m, UcxBuffer& in) {
    UcxBuffer out(mr, ucx_memory_type::HOST, in.size());
    std::memcpy(out.data(), in.data(), in.size());
    static_cast<char*>(out.data())[0] = 'R';
    return ex::on(pool.get_scheduler(), ex::just(std::tuple<TensorMeta, UcxBuffer>(m, std::move(out))));
  }, data::string("copy"));
  TensorMeta m;
  m.ndim = 1;
  m.dtype = {kDLUInt, 8, 1};
  m.shape = {4};
  m.strides = {1};
  UcxBuffer in(mr, ucx_memory_type::HOST, 4);
  std::memcpy(in.data(), "abcd", 4);
  auto [req, payload] = RpcRequestBuilder{}.PrepareRequest(opt(1), m, std::move(in));
  auto r = ex::sync_wait(d.Dispatch(req, std::move(payload)));
  CHECK(r && r->header.status.ok());
  CHECK(std::holds_alternative<UcxBuffer>(r->payload));
  CHECK(std::memcmp(std::get<UcxBuffer>(r->payload).data(), "Rbcd", 4) == 0);
  CHECK(r->header.results.size() == 1 && r->header.results[0].type == ParamType::TENSOR_META);
}

// ---- hybrid logical clock ---------------------------------------------------------------------------
EUX_TEST(hlc_default_is_zero) {
  HybridLogicalClock c;
  CHECK(c.Raw() == 0 && c.PhysicalTimeMs() == 0 && c.LogicalCounter() == 0);
}
EUX_TEST(hlc_tick_advances_with_physical_time) {
  HybridLogicalClock c(1000, 5);
  c.TickLocal(2000);
  CHECK(c.PhysicalTimeMs() == 2000 && c.LogicalCounter() == 0);
}
EUX_TEST(hlc_tick_counts_when_physical_time_stalls) {
  HybridLogicalClock c(1000, 5);
  c.TickLocal(1000);
  CHECK(c.PhysicalTimeMs() == 1000 && c.LogicalCounter() == 6);
  c.TickLocal(900);  // a clock that went backwards does not pull the timestamp back
  CHECK(c.PhysicalTimeMs() == 1000 && c.LogicalCounter() == 7);
}
EUX_TEST(hlc_merge_takes_the_largest_physical_part) {
  HybridLogicalClock local(1000, 3), remote(1500, 9);
  local.Merge(remote, 1200);
  CHECK(local.PhysicalTimeMs() == 1500 && local.LogicalCounter() == 10);
}
EUX_TEST(hlc_merge_tie_uses_the_larger_counter) {
  HybridLogicalClock local(1000, 3), remote(1000, 9);
  local.Merge(remote, 1000);
  CHECK(local.PhysicalTimeMs() == 1000 && local.LogicalCounter() == 10);
}
EUX_TEST(hlc_merge_older_remote_keeps_local) {
  HybridLogicalClock local(1000, 3), remote(500, 60);
  local.Merge(remote, 400);
  CHECK(local.PhysicalTimeMs() == 1000 && local.LogicalCounter() == 4);
}
EUX_TEST(hlc_merge_newer_wall_clock_resets_the_counter) {
  HybridLogicalClock local(1000, 3);
  local.Merge(HybridLogicalClock(1200, 8).Raw(), uint64_t(5000));
  CHECK(local.PhysicalTimeMs() == 5000 && local.LogicalCounter() == 0);
}
EUX_TEST(hlc_bump_wraps_and_assign_overwrites) {
  HybridLogicalClock c;
  c.Assign(77, 0xffff);
  CHECK(c.PhysicalTimeMs() == 77 && c.LogicalCounter() == 0xffff);
  c.BumpLogicalCounter();
  CHECK(c.PhysicalTimeMs() == 77 && c.LogicalCounter() == 0);
  c.AssignRaw((uint64_t(123) << 16) | 45);
  CHECK(c.PhysicalTimeMs() == 123 && c.LogicalCounter() == 45);
  CHECK(c.ToString() == "123.45");
}
EUX_TEST(hlc_now_and_monotonic_merges) {
  HybridLogicalClock a = HybridLogicalClock::Now();
  CHECK(a.PhysicalTimeMs() > 1'600'000'000'000ull);
  HybridLogicalClock prev = a;
  for (int i = 0; i < 1000; ++i) {
    a.Merge(prev);
    CHECK(a > prev);
    prev = a;
  }
  HybridLogicalClock b = a;
  b.TickLocal();
  CHECK(b > a);
}

EUX_TEST_MAIN()
