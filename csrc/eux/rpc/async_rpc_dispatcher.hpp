// AsyncRpcDispatcher: the same registry as RpcDispatcher, but a handler may
// return a sender; dispatching yields a type-erased sender of the invoke result
// (reference: rpc_core/async_rpc_dispatcher.hpp:146-768).
#pragma once

#include "eux/exec/async_scope.hpp"
#include "eux/rpc/rpc_dispatcher.hpp"

namespace eux::rpc {

using AsyncInvokeSender = exec::any_sender_of<RpcInvokeResult<ReturnedPayload>>;
// Type-erased asynchronous function: starts the call, returns a sender of its result. The
// payload (if any) is moved in, so it stays alive for as long as the sender runs.
using DynamicAsyncRpcFunction = std::function<AsyncInvokeSender(const RpcRequestHeader&, PayloadVariant&&, const RpcResponseBuilder&)>;

class AsyncRpcDispatcher {
 public:
  explicit AsyncRpcDispatcher(std::string instance_name = "default") : instance_name_(std::move(instance_name)) {}
  const std::string& instance_name() const { return instance_name_; }

  // A handler's return type is taken for a sender when it has the mark of one (a nested value_type) and is not
  // one of the wire's own containers, which carry the same mark (data::string, data::vector<T>).
  template <class T>
  static constexpr bool returns_sender_v = exec::sender<T> && !is_wire_param_v<T> && !is_data_vector<std::remove_cvref_t<T>>::value &&
                                           !std::is_same_v<std::remove_cvref_t<T>, data::string> && !is_payload_v<std::remove_cvref_t<T>>;

  // f(args...) -> value | sender of value. Arguments are filled as in RpcDispatcher.
  template <class F>
  bool RegisterFunction(function_id_t id, F&& f, const data::string& name = {}) {
    using Traits = function_traits<std::remove_cvref_t<F>>;
    using Ret = typename Traits::return_type;
    RpcFunctionSignature sig;
    sig.instance_name = data::string(instance_name_);
    sig.id = id;
    sig.function_name = name;
    detail::signature_of_args<typename Traits::args_tuple>::fill(sig);
    if constexpr (returns_sender_v<Ret>) detail::fill_return_signature<exec::value_t<Ret>>(sig);
    else detail::fill_return_signature<Ret>(sig);
    return insert(id, std::move(sig), MakeAsyncWrapper(std::forward<F>(f)));
  }
  bool RegisterFunction(function_id_t id, const data::string& name, const data::vector<ParamType>& param_types,
                        const data::vector<ParamType>& return_types, PayloadType input_payload_type,
                        PayloadType return_payload_type, DynamicAsyncRpcFunction&& fn) {
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
  byte_buf GetAllSignatures() const {
    data::vector<RpcFunctionSignature> all;
    {
      std::shared_lock lk(mu_);
      for (auto& [id, e] : functions_) all.push_back(e->signature);
    }
    std::sort(all.begin(), all.end(), [](auto& a, auto& b) { return a.id.v_ < b.id.v_; });
    return Serialize(all);
  }

  // Start the call; the payload is consumed.
  AsyncInvokeSender Dispatch(const RpcRequestHeader& req, PayloadVariant&& payload = {}, const RpcResponseBuilder& b = RpcResponseBuilder{}) {
    return InvokeAsyncFunction(req, std::move(payload), b);
  }
  AsyncInvokeSender Dispatch(byte_buf&& request_buffer, PayloadVariant&& payload = {}) {
    return InvokeAsyncFunction(Deserialize<RpcRequestHeader>(request_buffer), std::move(payload), RpcResponseBuilder{});
  }
  AsyncInvokeSender InvokeAsyncFunction(const RpcRequestHeader& req, PayloadVariant&& payload, const RpcResponseBuilder& b) {
    std::shared_ptr<Entry> e;
    {
      std::shared_lock lk(mu_);
      auto it = functions_.find(req.function_id);
      if (it != functions_.end()) e = it->second;
    }
    if (!e) {
      RpcInvokeResult<ReturnedPayload> r{
          detail::error_header(req, b, make_error_code(RpcErrc::NOT_FOUND), "function " + std::to_string(req.function_id.v_) + " is not registered"),
          ReturnedPayload{}};
      return AsyncInvokeSender(exec::just(std::move(r)));
    }
    if (!RpcDispatcher::TensorsFitPayload(req.params, std::get_if<ucxx::UcxBuffer>(&payload), std::get_if<ucxx::UcxBufferVec>(&payload))) {
      RpcInvokeResult<ReturnedPayload> r{
          detail::error_header(req, b, make_error_code(RpcErrc::INVALID_ARGUMENT), "the tensor metadata describes more bytes than the payload holds"),
          ReturnedPayload{}};
      return AsyncInvokeSender(exec::just(std::move(r)));
    }
    return e->fn(req, std::move(payload), b);
  }

  template <class F>
  static DynamicAsyncRpcFunction MakeAsyncWrapper(F&& f) {
    using Traits = function_traits<std::remove_cvref_t<F>>;
    using Args = typename Traits::args_tuple;
    using Ret = typename Traits::return_type;
    return [fn = std::forward<F>(f)](const RpcRequestHeader& req, PayloadVariant&& payload, const RpcResponseBuilder& b) mutable -> AsyncInvokeSender {
      // request, builder and payload must outlive the asynchronous call
      struct State {
        RpcRequestHeader req;
        RpcResponseBuilder b;
        PayloadVariant payload;
      };
      auto st = std::make_shared<State>(State{req, b, std::move(payload)});
      auto fail = [st](std::error_code ec, std::string_view what) {
        return RpcInvokeResult<ReturnedPayload>{detail::error_header(st->req, st->b, ec, what), ReturnedPayload{}};
      };
      try {
        RpcContextPtr ctx = RpcContextPtr::of(st->payload, true);
        if constexpr (returns_sender_v<Ret>) {
          size_t idx = 0;
          auto snd = call(fn, st->req, ctx, st->b, idx, static_cast<Args*>(nullptr), std::make_index_sequence<std::tuple_size_v<Args>>{});
          using V = exec::value_t<Ret>;
          auto on_error = [fail](std::exception_ptr ep) {
            try {
              std::rethrow_exception(ep);
            } catch (const RpcException& e) {
              return fail(e.code(), e.what());
            } catch (const std::system_error& e) {
              return fail(e.code(), e.what());
            } catch (const std::exception& e) {
              return fail(make_error_code(RpcErrc::INTERNAL), e.what());
            } catch (...) {
              return fail(make_error_code(RpcErrc::UNKNOWN), "unknown error");
            }
          };
          auto on_done = [fail] { return fail(make_error_code(RpcErrc::CANCELLED), "the handler was cancelled"); };
          if constexpr (std::is_void_v<V>) {
            return AsyncInvokeSender(exec::upon_done(
                exec::upon_error(exec::then(std::move(snd),
                                            [st] {
                                              return RpcInvokeResult<ReturnedPayload>{st->b.PrepareResponse(st->req.session_id, st->req.request_id), {}};
                                            }),
                                 on_error),
                on_done));
          } else {
            return AsyncInvokeSender(exec::upon_done(
                exec::upon_error(exec::then(std::move(snd),
                                            [st](V v) {
                                              auto r = detail::pack_result(st->req, st->b, std::move(v));
                                              return RpcInvokeResult<ReturnedPayload>{std::move(r.first), std::move(r.second)};
                                            }),
                                 on_error),
                on_done));
          }
        } else {
          auto sync = RpcDispatcher::MakeRpcWrapper(fn);
          auto r = sync(st->req, ctx, st->b);
          return AsyncInvokeSender(exec::just(RpcInvokeResult<ReturnedPayload>{std::move(r.first), std::move(r.second)}));
        }
      } catch (const RpcException& e) {
        return AsyncInvokeSender(exec::just(fail(e.code(), e.what())));
      } catch (const std::exception& e) {
        return AsyncInvokeSender(exec::just(fail(make_error_code(RpcErrc::INTERNAL), e.what())));
      }
    };
  }

 private:
  struct Entry {
    RpcFunctionSignature signature;
    DynamicAsyncRpcFunction fn;
  };
  bool insert(function_id_t id, RpcFunctionSignature&& sig, DynamicAsyncRpcFunction&& fn) {
    auto e = std::make_shared<Entry>(Entry{std::move(sig), std::move(fn)});
    std::unique_lock lk(mu_);
    return functions_.emplace(id, std::move(e)).second;
  }
  template <class Fn, class... A, size_t... I>
  static auto call(Fn& fn, const RpcRequestHeader& req, RpcContextPtr ctx, const RpcResponseBuilder& b, size_t& idx, std::tuple<A...>*,
                   std::index_sequence<I...>) {
    std::tuple<A...> args{detail::extract_arg<A>(req, ctx, b, idx)...};
    return std::apply([&](auto&&... a) { return fn(std::forward<decltype(a)>(a)...); }, std::move(args));
  }
  std::string instance_name_;
  mutable std::shared_mutex mu_;
  std::unordered_map<function_id_t, std::shared_ptr<Entry>> functions_;
};

}  // namespace eux::rpc
