// RpcDispatcher: a registry of callables addressed by function id. A request
// header (or its serialised bytes) plus an optional payload is turned into a
// call: every argument of the registered callable is filled by its type from
// the header's parameters, the request itself, a response builder or the
// payload; the return value becomes a response header plus an optional payload
// (reference: rpc_core/rpc_dispatcher.hpp:242-1089).
#pragma once

#include <typeindex>
#include <algorithm>
#include <functional>
#include <memory>
#include <mutex>
#include <optional>
#include <shared_mutex>
#include <string>
#include <unordered_map>

#include "eux/rpc/rpc_request_builder.hpp"
#include "eux/rpc/rpc_response_builder.hpp"
#include "eux/rpc/utils/cista_serialize_helper.hpp"

namespace eux::rpc {

template <class ReturnedPayloadT>
struct RpcInvokeResult {
  RpcResponseHeader header;
  ReturnedPayloadT payload;
};

// The payload handed to a call: a non-owning view of the caller's object. When
// `movable` the callee may move out of it (DispatchMove).
struct RpcContextPtr {
  void* ptr = nullptr;
  PayloadType kind = PayloadType::NO_PAYLOAD;
  bool is_variant = false;  // ptr is a PayloadVariant*
  bool movable = false;
  template <class T>
  static RpcContextPtr of(T& obj, bool movable) {
    using D = std::remove_cvref_t<T>;
    if constexpr (std::is_same_v<D, PayloadVariant>) return {&obj, payload_type_of(obj), true, movable};
    else if constexpr (is_payload_v<D>) return {&obj, payload_type_of<D>(), false, movable};
    else return {};
  }
  template <class P>
  P* get() const {  // P = UcxBuffer or UcxBufferVec; nullptr when the kinds differ
    if (!ptr || kind != payload_type_of<P>()) return nullptr;
    if (is_variant) return std::get_if<P>(static_cast<PayloadVariant*>(ptr));
    return static_cast<P*>(ptr);
  }
};

using DynamicRpcResult = std::pair<RpcResponseHeader, ReturnedPayload>;
using DynamicRpcFunction = std::function<DynamicRpcResult(const RpcRequestHeader&, RpcContextPtr, const RpcResponseBuilder&)>;

namespace detail {

inline RpcResponseHeader error_header(const RpcRequestHeader& req, const RpcResponseBuilder& b, std::error_code ec, std::string_view what) {
  return b.PrepareError(req.session_id, req.request_id, ec, what);
}

// ---- argument extraction by type ----
template <class T>
decltype(auto) extract_arg(const RpcRequestHeader& req, RpcContextPtr ctx, const RpcResponseBuilder& builder, size_t& idx) {
  using D = std::remove_cvref_t<T>;
  if constexpr (std::is_same_v<D, RpcRequestHeader>) {
    return (req);
  } else if constexpr (std::is_same_v<D, RpcResponseBuilder>) {
    return (builder);
  } else if constexpr (is_payload_v<D>) {
    D* p = ctx.template get<D>();
    if (!p) throw RpcException(RpcErrc::INVALID_ARGUMENT, "the call needs a payload of another kind than the one supplied");
    if constexpr (std::is_lvalue_reference_v<T>) {
      return (*p);
    } else {  // by value or by rvalue reference: the function takes it over
      if (!ctx.movable) throw RpcException(RpcErrc::INVALID_ARGUMENT, "the function takes its payload by value; dispatch it with DispatchMove");
      // `T&&` must refer to the caller's object, which outlives the call: a temporary made here would be
      // gone before the function runs
      if constexpr (std::is_rvalue_reference_v<T>) return std::move(*p);
      else return D(std::move(*p));
    }
  } else if constexpr (is_payload_variant_v<D>) {
    if (!ctx.ptr) throw RpcException(RpcErrc::INVALID_ARGUMENT, "the call needs a payload");
    if (ctx.is_variant) {
      auto* v = static_cast<PayloadVariant*>(ctx.ptr);
      if constexpr (std::is_lvalue_reference_v<T>) return (*v);
      else if constexpr (std::is_rvalue_reference_v<T>) return std::move(*v);
      else return PayloadVariant(std::move(*v));
    } else {
      throw RpcException(RpcErrc::INVALID_ARGUMENT, "the function takes a PayloadVariant; pass one");
    }
  } else if constexpr (std::is_same_v<D, TensorMeta>) {
    return (req.GetTensor(idx++));
  } else if constexpr (std::is_same_v<D, TensorMetaVec>) {
    return (req.GetTensorVec(idx++));
  } else if constexpr (std::is_same_v<D, data::string>) {
    return (req.GetString(idx++));
  } else if constexpr (std::is_same_v<D, std::string>) {
    return std::string(req.GetString(idx++).str());
  } else if constexpr (std::is_same_v<D, std::string_view>) {
    return req.GetString(idx++).view();
  } else if constexpr (std::is_enum_v<D>) {
    return static_cast<D>(req.template GetPrimitive<std::underlying_type_t<D>>(idx++));
  } else if constexpr (std::is_arithmetic_v<D>) {
    return req.template GetPrimitive<D>(idx++);
  } else if constexpr (is_strong<D>::value) {
    return D(req.template GetPrimitive<typename D::value_t>(idx++));
  } else if constexpr (is_data_vector<D>::value) {
    using E0 = typename D::value_type;
    using E = std::conditional_t<std::is_same_v<E0, data::bool_t>, bool, E0>;
    return (req.template GetVector<E>(idx++));
  } else {
    static_assert(!std::is_same_v<T, T>, "unsupported argument type for an RPC function");
  }
}

// ---- result packing ----
template <class R>
void pack_one(RpcResponseHeader& h, ReturnedPayload& payload, R&& r) {
  using D = std::remove_cvref_t<R>;
  if constexpr (is_payload_v<D>) payload = std::move(r);
  else if constexpr (is_payload_variant_v<D>) payload = std::move(r);
  else h.results.emplace_back(std::forward<R>(r));
}

template <class T>
struct is_header_pair : std::false_type {};
template <class B>
struct is_header_pair<std::pair<RpcResponseHeader, B>> : std::true_type {};

template <class Ret>
DynamicRpcResult pack_result(const RpcRequestHeader& req, const RpcResponseBuilder& b, Ret&& ret) {
  using D = std::remove_cvref_t<Ret>;
  ReturnedPayload payload;
  if constexpr (std::is_same_v<D, RpcResponseHeader>) {
    return {std::forward<Ret>(ret), std::move(payload)};
  } else if constexpr (is_header_pair<D>::value) {
    pack_one(ret.first, payload, std::move(ret.second));
    return {std::move(ret.first), std::move(payload)};
  } else if constexpr (is_tuple<D>::value) {
    RpcResponseHeader h = b.PrepareResponse(req.session_id, req.request_id);
    std::apply([&](auto&&... e) { (pack_one(h, payload, std::move(e)), ...); }, std::move(ret));
    return {std::move(h), std::move(payload)};
  } else {
    RpcResponseHeader h = b.PrepareResponse(req.session_id, req.request_id);
    pack_one(h, payload, std::forward<Ret>(ret));
    return {std::move(h), std::move(payload)};
  }
}

template <class Tuple>
struct signature_of_args;
template <class... A>
struct signature_of_args<std::tuple<A...>> {
  static void fill(RpcFunctionSignature& s) {
    ((is_wire_param_v<A> ? s.param_types.push_back(get_param_type<A>()) : void()), ...);
    s.input_payload_type = payload_finder<A...>::type;
    if constexpr ((is_payload_variant_v<A> || ...)) s.input_payload_type = PayloadType::UCX_BUFFER;
  }
};
template <class Ret>
void fill_return_signature(RpcFunctionSignature& s) {
  using D = std::remove_cvref_t<Ret>;
  if constexpr (std::is_void_v<D>) {
  } else if constexpr (is_tuple<D>::value) {
    [&]<class... E>(std::type_identity<std::tuple<E...>>) {
      ((is_wire_param_v<E> ? s.return_types.push_back(get_param_type<E>()) : void()), ...);
      s.return_payload_type = payload_finder<E...>::type;
    }(std::type_identity<D>{});
  } else if constexpr (is_pair<D>::value) {
    s.return_payload_type = payload_type_of<typename D::second_type>();
  } else if constexpr (is_payload_v<D>) {
    s.return_payload_type = payload_type_of<D>();
  } else if constexpr (is_wire_param_v<D>) {
    s.return_types.push_back(get_param_type<D>());
  }
}

}  // namespace detail

// ---- natural call (reference: GetCaller under EUX_RPC_ENABLE_NATURAL_CALL, rpc_core/rpc_dispatcher.hpp:335-673) ----
// A registered native callable can be fetched back and called with ordinary C++ arguments, without a
// request header in between: `(*dispatcher.GetCaller<int(int, int)>(id))(20, 22)`.
namespace detail {
template <class R, class ArgsTuple>
struct canon_fn;
template <class R, class... A>
struct canon_fn<R, std::tuple<A...>> {
  using type = std::function<R(std::remove_cvref_t<A>&...)>;  // every argument by lvalue reference to its decayed type
};
// hands the canonical lvalue on the way the declared parameter wants it: by reference as it is, by value as an rvalue
template <class Decl, class T>
constexpr decltype(auto) pass_as(T& v) {
  if constexpr (std::is_lvalue_reference_v<Decl>) return (v);
  else return std::move(v);
}
}  // namespace detail

template <class Sig>
class NaturalCaller;
template <class R, class... A>
class NaturalCaller<R(A...)> {
 public:
  using canon_type = typename detail::canon_fn<R, std::tuple<A...>>::type;
  explicit NaturalCaller(std::shared_ptr<canon_type> fn) : fn_(std::move(fn)) {}
  R operator()(A... a) const { return (*fn_)(const_cast<std::remove_cvref_t<A>&>(a)...); }

 private:
  std::shared_ptr<canon_type> fn_;
};

class RpcDispatcher {
 public:
  explicit RpcDispatcher(std::string instance_name = "default") : instance_name_(std::move(instance_name)) {}

  const std::string& instance_name() const { return instance_name_; }

  // Wrap any callable (function, lambda, functor, std::function) into the type-erased form.
  template <class F>
  static DynamicRpcFunction MakeRpcWrapper(F&& f) {
    using Traits = function_traits<std::remove_cvref_t<F>>;
    using Args = typename Traits::args_tuple;
    using Ret = typename Traits::return_type;
    return [fn = std::forward<F>(f)](const RpcRequestHeader& req, RpcContextPtr ctx, const RpcResponseBuilder& b) mutable -> DynamicRpcResult {
      try {
        return invoke_with_args<Ret, Args>(fn, req, ctx, b, std::make_index_sequence<std::tuple_size_v<Args>>{});
      } catch (const RpcException& e) {
        return {detail::error_header(req, b, e.code(), e.what()), ReturnedPayload{}};
      } catch (const std::system_error& e) {
        return {detail::error_header(req, b, e.code(), e.what()), ReturnedPayload{}};
      } catch (const std::exception& e) {
        return {detail::error_header(req, b, make_error_code(RpcErrc::INTERNAL), e.what()), ReturnedPayload{}};
      }
    };
  }
  // Member function bound to an object.
  template <class C, class R, class... A>
  static DynamicRpcFunction MakeRpcWrapper(R (C::*mf)(A...), C* obj) {
    return MakeRpcWrapper(std::function<R(A...)>([obj, mf](A... a) -> R { return (obj->*mf)(std::forward<A>(a)...); }));
  }

  template <class F>
  bool RegisterFunction(function_id_t id, F&& f, const data::string& name = {}) {
    using Traits = function_traits<std::remove_cvref_t<F>>;
    RpcFunctionSignature sig;
    sig.instance_name = data::string(instance_name_);
    sig.id = id;
    sig.function_name = name;
    detail::signature_of_args<typename Traits::args_tuple>::fill(sig);
    detail::fill_return_signature<typename Traits::return_type>(sig);
    using Callable = std::remove_cvref_t<F>;
    if constexpr (std::is_copy_constructible_v<Callable>) {
      // one copy serves the serialised path, the other the natural call
      auto [native, tag] = make_native<typename Traits::return_type, typename Traits::args_tuple>(Callable(f));
      return insert(id, std::move(sig), MakeRpcWrapper(std::forward<F>(f)), std::move(native), tag);
    } else {
      return insert(id, std::move(sig), MakeRpcWrapper(std::forward<F>(f)));
    }
  }
  // The registered native callable as something callable with ordinary arguments. Throws
  // std::runtime_error when the id is unknown, when the function was registered in its dynamic
  // (type-erased) form, or when `Sig` differs from the registered signature in more than
  // const / reference qualifiers. Exceptions of the callable reach the caller unchanged.
  template <class Sig>
  std::shared_ptr<NaturalCaller<Sig>> GetCaller(function_id_t id) const {
    std::shared_ptr<Entry> e;
    {
      std::shared_lock lk(mu_);
      auto it = functions_.find(id);
      if (it != functions_.end()) e = it->second;
    }
    if (!e) throw std::runtime_error("GetCaller: function " + std::to_string(id.v_) + " is not registered");
    using Canon = typename NaturalCaller<Sig>::canon_type;
    if (!e->native || e->native_type != std::type_index(typeid(Canon)))
      throw std::runtime_error("GetCaller: function " + std::to_string(id.v_) + " has no native form with this signature");
    return std::make_shared<NaturalCaller<Sig>>(std::static_pointer_cast<Canon>(e->native));
  }
  template <class C, class R, class... A>
  bool RegisterFunction(function_id_t id, R (C::*mf)(A...), C* obj, const data::string& name = {}) {
    return RegisterFunction(id, std::function<R(A...)>([obj, mf](A... a) -> R { return (obj->*mf)(std::forward<A>(a)...); }), name);
  }
  // Dynamic registration: the signature is given, the callable is already type-erased.
  bool RegisterFunction(function_id_t id, const data::string& name, const data::vector<ParamType>& param_types,
                        const data::vector<ParamType>& return_types, PayloadType input_payload_type,
                        PayloadType return_payload_type, DynamicRpcFunction&& fn) {
    RpcFunctionSignature sig;
    sig.instance_name = data::string(instance_name_);
    sig.id = id;
    sig.function_name = name;
    sig.param_types = param_types;
    sig.return_types = return_types;
    sig.input_payload_type = input_payload_type;
    sig.return_payload_type = return_payload_type;
    return insert(id, std::move(sig), std::move(fn));
  }
  bool UnregisterFunction(function_id_t id) {
    std::unique_lock lk(mu_);
    return functions_.erase(id) != 0;
  }

  bool IsRegistered(function_id_t id) const {
    std::shared_lock lk(mu_);
    return functions_.count(id) != 0;
  }
  size_t FunctionCount() const {
    std::shared_lock lk(mu_);
    return functions_.size();
  }
  std::optional<RpcFunctionSignature> GetSignature(function_id_t id) const {
    std::shared_lock lk(mu_);
    auto it = functions_.find(id);
    if (it == functions_.end()) return std::nullopt;
    return it->second->signature;
  }
  std::optional<RpcFunctionSignature> GetSignature(std::string_view name) const {
    std::shared_lock lk(mu_);
    for (auto& [id, e] : functions_)
      if (e->signature.function_name.view() == name) return e->signature;
    return std::nullopt;
  }
  // Serialised vector<RpcFunctionSignature>, for service discovery.
  byte_buf GetAllSignatures() const {
    data::vector<RpcFunctionSignature> all;
    {
      std::shared_lock lk(mu_);
      for (auto& [id, e] : functions_) all.push_back(e->signature);
    }
    std::sort(all.begin(), all.end(), [](auto& a, auto& b) { return a.id.v_ < b.id.v_; });
    return Serialize(all);
  }
  static data::vector<RpcFunctionSignature> DeserializeSignatures(const void* p, size_t n) {
    return Deserialize<data::vector<RpcFunctionSignature>>(p, n);
  }

  // ---- dispatch ----
  // Untyped: the returned payload is the variant.
  RpcInvokeResult<ReturnedPayload> Dispatch(const RpcRequestHeader& req, const RpcResponseBuilder& b = RpcResponseBuilder{}) {
    return to_result(InvokeFunction(req, RpcContextPtr{}, b));
  }
  template <class Input>
    requires(is_payload_v<Input> || is_payload_variant_v<Input>)
  RpcInvokeResult<ReturnedPayload> Dispatch(const RpcRequestHeader& req, Input& input, const RpcResponseBuilder& b = RpcResponseBuilder{}) {
    return to_result(InvokeFunction(req, RpcContextPtr::of(input, false), b));
  }
  template <class Input>
    requires(is_payload_v<Input> || is_payload_variant_v<Input>)
  RpcInvokeResult<ReturnedPayload> DispatchMove(const RpcRequestHeader& req, Input&& input, const RpcResponseBuilder& b = RpcResponseBuilder{}) {
    std::remove_cvref_t<Input> owned(std::move(input));  // lives on this frame for the whole (synchronous) call
    return to_result(InvokeFunction(req, RpcContextPtr::of(owned, true), b));
  }
  RpcInvokeResult<ReturnedPayload> Dispatch(byte_buf&& request_buffer) {
    return Dispatch(Deserialize<RpcRequestHeader>(request_buffer));
  }
  template <class Input>
    requires(is_payload_v<Input> || is_payload_variant_v<Input>)
  RpcInvokeResult<ReturnedPayload> Dispatch(byte_buf&& request_buffer, Input& input) {
    return Dispatch(Deserialize<RpcRequestHeader>(request_buffer), input);
  }
  template <class Input>
    requires(is_payload_v<Input> || is_payload_variant_v<Input>)
  RpcInvokeResult<ReturnedPayload> DispatchMove(byte_buf&& request_buffer, Input&& input) {
    return DispatchMove(Deserialize<RpcRequestHeader>(request_buffer), std::move(input));
  }
  // Typed: the caller names the payload type it expects back (std::monostate = none).
  template <class RetPayload, class... Rest>
  RpcInvokeResult<RetPayload> Dispatch(const RpcRequestHeader& req, Rest&&... rest) {
    return typed<RetPayload>(Dispatch(req, std::forward<Rest>(rest)...));
  }
  template <class RetPayload, class... Rest>
  RpcInvokeResult<RetPayload> Dispatch(byte_buf&& buf, Rest&&... rest) {
    return typed<RetPayload>(Dispatch(std::move(buf), std::forward<Rest>(rest)...));
  }
  template <class RetPayload, class... Rest>
  RpcInvokeResult<RetPayload> DispatchMove(const RpcRequestHeader& req, Rest&&... rest) {
    return typed<RetPayload>(DispatchMove(req, std::forward<Rest>(rest)...));
  }
  template <class RetPayload, class... Rest>
  RpcInvokeResult<RetPayload> DispatchMove(byte_buf&& buf, Rest&&... rest) {
    return typed<RetPayload>(DispatchMove(std::move(buf), std::forward<Rest>(rest)...));
  }
  // Call a function that is not registered, with the same argument filling.
  template <class F>
  RpcInvokeResult<ReturnedPayload> DispatchAdhoc(F&& f, const RpcRequestHeader& req, RpcContextPtr ctx = {},
                                                 const RpcResponseBuilder& b = RpcResponseBuilder{}) {
    auto fn = MakeRpcWrapper(std::forward<F>(f));
    return to_result(fn(req, ctx, b));
  }

  // The core: find and call. Also used by the asynchronous front ends.
  DynamicRpcResult InvokeFunction(const RpcRequestHeader& req, RpcContextPtr ctx, const RpcResponseBuilder& b) {
    std::shared_ptr<Entry> e;
    {
      std::shared_lock lk(mu_);
      auto it = functions_.find(req.function_id);
      if (it != functions_.end()) e = it->second;
    }
    if (!e)
      return {detail::error_header(req, b, make_error_code(RpcErrc::NOT_FOUND), "function " + std::to_string(req.function_id.v_) + " is not registered"),
              ReturnedPayload{}};
    if (!TensorsFitPayload(req.params, ctx.get<ucxx::UcxBuffer>(), ctx.get<ucxx::UcxBufferVec>()))
      return {detail::error_header(req, b, make_error_code(RpcErrc::INVALID_ARGUMENT), "the tensor metadata describes more bytes than the payload holds"),
              ReturnedPayload{}};
    return e->fn(req, ctx, b);
  }

  // What a handler may take for granted about a call that carries both tensor descriptions and a payload: every
  // described tensor lies inside the payload (one description: inside the buffer, or the vector's first segment;
  // several: one segment each, or back to back in one buffer). The descriptions come from the caller, so this is
  // checked before any handler runs. A call without a payload, or without descriptions, passes: nothing to compare.
  static bool TensorsFitPayload(const data::vector<ParamMeta>& params, const ucxx::UcxBuffer* buf, const ucxx::UcxBufferVec* vec) {
    if (!buf && !vec) return true;
    const TensorMeta* one = nullptr;
    const TensorMetaVec* many = nullptr;
    for (auto& p : params) {
      if (p.type == ParamType::TENSOR_META) one = std::get_if<TensorMeta>(&p.value), many = nullptr;
      else if (p.type == ParamType::TENSOR_META_VEC) many = std::get_if<TensorMetaVec>(&p.value), one = nullptr;
    }
    if (one) {
      const size_t need = utils::TensorPayloadBytes(*one);
      if (buf) return need <= buf->size();
      return vec->size() >= 1 && need <= (*vec)[0].size;
    }
    if (many) {
      if (vec) {
        if (vec->size() < many->size()) return false;
        for (size_t i = 0; i < many->size(); ++i)
          if (utils::TensorPayloadBytes((*many)[i]) > (*vec)[i].size) return false;
        return true;
      }
      size_t total = 0;
      for (auto& m : *many) {
        const size_t n = utils::TensorPayloadBytes(m);
        if (n > buf->size() - std::min(total, buf->size())) return false;  // also what overflows the sum
        total += n;
      }
      return true;
    }
    return true;
  }

  // ---- response (de)serialisation helpers ----
  static byte_buf SerializeResponse(const RpcResponseHeader& h) { return Serialize(h); }
  static size_t SerializeResponse(const RpcResponseHeader& h, FixedBufferWriter& w) { return SerializeInto(w, h); }
  static void SerializeResponse(const RpcResponseHeader& h, byte_buf& out) { out = Serialize(h); }
  // (spelled as in the reference, rpc_dispatcher.hpp:312)
  static RpcResponseHeader DeerializeResponse(ucxx::UcxHeader&& header) {
    ucxx::UcxHeader owned(std::move(header));
    return Deserialize<RpcResponseHeader>(owned.data(), owned.size());
  }
  static RpcResponseHeader DeserializeResponse(const void* p, size_t n) { return Deserialize<RpcResponseHeader>(p, n); }
  static RpcRequestHeader DeserializeRequest(const void* p, size_t n) { return Deserialize<RpcRequestHeader>(p, n); }

  // A tensor-carrying call is consistent when the metadata in the header agrees
  // with the payload: one TENSOR_META for a buffer of at least that many bytes,
  // a TENSOR_META_VEC whose entries match the buffer vector one to one.
  static RpcStatus ValidateTensorPayloadConstraints(const data::vector<ParamMeta>& params, const PayloadVariant& payload) {
    const TensorMeta* one = nullptr;
    const TensorMetaVec* many = nullptr;
    for (auto& p : params) {
      if (p.type == ParamType::TENSOR_META) {
        if (one || many) return RpcStatus(make_error_code(RpcErrc::INVALID_ARGUMENT));
        one = &std::get<TensorMeta>(p.value);
      } else if (p.type == ParamType::TENSOR_META_VEC) {
        if (one || many) return RpcStatus(make_error_code(RpcErrc::INVALID_ARGUMENT));
        many = &std::get<TensorMetaVec>(p.value);
      }
    }
    if (one) {
      const auto* b = std::get_if<ucxx::UcxBuffer>(&payload);
      if (!b || b->size() < utils::CalculateTensorSize(*one)) return RpcStatus(make_error_code(RpcErrc::INVALID_ARGUMENT));
    } else if (many) {
      if (const auto* v = std::get_if<ucxx::UcxBufferVec>(&payload)) {
        if (v->size() != many->size()) return RpcStatus(make_error_code(RpcErrc::INVALID_ARGUMENT));
        for (size_t i = 0; i < many->size(); ++i)
          if ((*v)[i].size < utils::CalculateTensorSize((*many)[i])) return RpcStatus(make_error_code(RpcErrc::INVALID_ARGUMENT));
      } else if (const auto* b = std::get_if<ucxx::UcxBuffer>(&payload)) {
        size_t total = 0;
        for (auto& m : *many) total += utils::CalculateTensorSize(m);
        if (b->size() < total) return RpcStatus(make_error_code(RpcErrc::INVALID_ARGUMENT));
      } else {
        return RpcStatus(make_error_code(RpcErrc::INVALID_ARGUMENT));
      }
    }
    return RpcStatus{};
  }

 private:
  struct Entry {
    RpcFunctionSignature signature;
    DynamicRpcFunction fn;
    std::shared_ptr<void> native;                         // canon_fn of the registered callable, if it has one
    std::type_index native_type = std::type_index(typeid(void));
  };
  template <class R, class ArgsTuple, class Callable>
  static std::pair<std::shared_ptr<void>, std::type_index> make_native(Callable&& c) {
    return make_native_impl<R>(std::forward<Callable>(c), static_cast<ArgsTuple*>(nullptr));
  }
  template <class R, class Callable, class... A>
  static std::pair<std::shared_ptr<void>, std::type_index> make_native_impl(Callable&& c, std::tuple<A...>*) {
    using Canon = typename detail::canon_fn<R, std::tuple<A...>>::type;
    auto shared = std::make_shared<std::remove_cvref_t<Callable>>(std::forward<Callable>(c));
    auto canon = std::make_shared<Canon>([shared](std::remove_cvref_t<A>&... a) -> R { return (*shared)(detail::pass_as<A>(a)...); });
    return {std::static_pointer_cast<void>(canon), std::type_index(typeid(Canon))};
  }
  bool insert(function_id_t id, RpcFunctionSignature&& sig, DynamicRpcFunction&& fn, std::shared_ptr<void> native = nullptr,
              std::type_index native_type = std::type_index(typeid(void))) {
    auto e = std::make_shared<Entry>(Entry{std::move(sig), std::move(fn), std::move(native), native_type});
    std::unique_lock lk(mu_);
    return functions_.emplace(id, std::move(e)).second;
  }
  template <class Ret, class Args, class Fn, size_t... I>
  static DynamicRpcResult invoke_with_args(Fn& fn, const RpcRequestHeader& req, RpcContextPtr ctx, const RpcResponseBuilder& b,
                                           std::index_sequence<I...>) {
    size_t idx = 0;
    // braced initialisation fixes the evaluation order, so parameters are consumed left to right
    if constexpr (std::is_void_v<Ret>) {
      std::tuple<std::tuple_element_t<I, Args>...> args{detail::extract_arg<std::tuple_element_t<I, Args>>(req, ctx, b, idx)...};
      std::apply([&](auto&&... a) { fn(std::forward<decltype(a)>(a)...); }, std::move(args));
      return {b.PrepareResponse(req.session_id, req.request_id), ReturnedPayload{}};
    } else {
      std::tuple<std::tuple_element_t<I, Args>...> args{detail::extract_arg<std::tuple_element_t<I, Args>>(req, ctx, b, idx)...};
      return detail::pack_result(req, b, std::apply([&](auto&&... a) -> Ret { return fn(std::forward<decltype(a)>(a)...); }, std::move(args)));
    }
  }
  static RpcInvokeResult<ReturnedPayload> to_result(DynamicRpcResult&& r) { return {std::move(r.first), std::move(r.second)}; }
  template <class RetPayload>
  static RpcInvokeResult<RetPayload> typed(RpcInvokeResult<ReturnedPayload>&& r) {
    if constexpr (std::is_same_v<RetPayload, ReturnedPayload>) {
      return std::move(r);
    } else if constexpr (std::is_same_v<RetPayload, std::monostate>) {
      return {std::move(r.header), std::monostate{}};
    } else {
      if (auto* p = std::get_if<RetPayload>(&r.payload)) return RpcInvokeResult<RetPayload>{std::move(r.header), std::move(*p)};
      if (r.header.status.ok()) throw RpcException(RpcErrc::INTERNAL, "the function returned another payload kind than the caller expects");
      throw RpcException(static_cast<std::error_code>(r.header.status),
                         r.header.results.empty() ? std::string() : std::string(r.header.GetString(0).str()));
    }
  }

  std::string instance_name_;
  mutable std::shared_mutex mu_;
  std::unordered_map<function_id_t, std::shared_ptr<Entry>> functions_;
};

}  // namespace eux::rpc
