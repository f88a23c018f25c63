// Python bindings, part 2: memory managers and the AxonRuntime class with its
// asyncio integration (reference: axon/python/src/bindings_runtime.cpp,
// async_bridge.hpp, bindings_runtime_wrapper.cpp, memory_policy_helpers.cpp).
//
// Threads: Python calls arrive on the asyncio thread with the GIL. Completions
// come from the runtime's C++ threads; they are turned into closures that the
// wake manager runs on the asyncio thread, where futures are resolved and
// Python handlers are started as tasks.
#include <cuda_runtime_api.h>

#include <atomic>
#include <optional>
#include <unordered_map>

#include "eux/ucxx/nvtx_range.hpp"
#include "bindings_common.hpp"
#include "eux/ucxx/cuda/ucx_cuda_context.hpp"
#include "eux/ucxx/cuda/ucx_cuda_memory_manager.hpp"
#include "eux/axon/services/peer_memory_service.hpp"
#include "eux/axon/services/remote_gemm_service.hpp"

namespace eux::python {

namespace ex = eux::exec;
using axon::ClientMemoryPolicy;
using axon::InvokeResult;
using axon::ServerMemoryPolicy;
using rpc::PayloadVariant;
using ucxx::UcxBuffer;
using ucxx::UcxBufferVec;

namespace {

std::shared_ptr<ucxx::UcxMemoryResourceManager>& default_manager() {
  static std::shared_ptr<ucxx::UcxMemoryResourceManager> mr = std::make_shared<ucxx::DefaultUcxMemoryResourceManager>();
  return mr;
}

std::chrono::milliseconds parse_timeout(py::handle t) {
  if (t.is_none()) return std::chrono::milliseconds(300);
  if (py::isinstance<py::int_>(t)) return std::chrono::milliseconds(t.cast<int64_t>());           // int: milliseconds
  if (py::isinstance<py::float_>(t)) return std::chrono::milliseconds(int64_t(t.cast<double>() * 1000.0));  // float: seconds
  if (py::hasattr(t, "total_seconds")) return std::chrono::milliseconds(int64_t(t.attr("total_seconds")().cast<double>() * 1000.0));
  throw py::type_error("timeout must be int (ms), float (s), datetime.timedelta or None");
}

// payload argument of invoke_raw / result of a Python handler -> PayloadVariant. With `metas`, the
// metadata of every tensor that is imported is appended there (one __dlpack__ call per tensor serves
// both the bytes and the description).
// The stream on which the producer of a device tensor would launch its next kernel, as far as this layer can
// know it: a torch tensor's is torch's current stream on that device; anything else is taken to work on the
// legacy default stream (0), with which every blocking stream synchronises.
uintptr_t producer_stream(py::handle obj, int device) { return torch_current_stream(obj, device); }

PayloadVariant payload_from_python(ucxx::UcxMemoryResourceManager& mr, py::handle obj, rpc::TensorMetaVec* metas = nullptr, int wire_dtype = 0) {
  if (obj.is_none()) return {};
  if (py::isinstance<PyBuffer>(obj)) {
    auto& b = obj.cast<PyBuffer&>();
    if (!b.buf) return {};
    // a view that keeps the shared buffer alive
    auto keep = b.buf;
    return UcxBuffer(mr, keep->type(), keep->data(), keep->size(), nullptr, true, [keep](void*) mutable { keep.reset(); });
  }
  if (py::isinstance<PyBufferVec>(obj)) {
    auto keep = obj.cast<PyBufferVec&>().vec;
    if (!keep) return {};
    return UcxBufferVec(mr, keep->type(), std::vector<ucx_buffer_t>(keep->buffers()), nullptr, true, [keep](void*) mutable { keep.reset(); });
  }
  if (py::isinstance<py::list>(obj) || py::isinstance<py::tuple>(obj)) {
    std::vector<ImportedTensor> ts;
    py::handle first_cuda;
    int cuda_device = -1;
    for (auto item : obj) {
      ts.push_back(import_tensor(item));
      if (metas) metas->push_back(ts.back().meta);
      if (cuda_device < 0 && ts.back().meta.device.device_type == kDLCUDA) {
        cuda_device = ts.back().meta.device.device_id;
        first_cuda = item;
      }
    }
    auto vec = to_ucx_buffer_vec(mr, std::move(ts));
    if (cuda_device >= 0) vec.set_send_attr(make_send_attr(nullptr, cuda_device, producer_stream(first_cuda, cuda_device)));
    return vec;
  }
  ImportedTensor t = import_tensor(obj, /*allow_strided=*/true, wire_dtype);
  if (metas) metas->push_back(t.meta);
  std::shared_ptr<const ucxx::UcxSendAttr> attr;
  if (t.meta.device.device_type == kDLCUDA && t.nbytes > 0)
    attr = make_send_attr(&t, t.meta.device.device_id, producer_stream(obj, t.meta.device.device_id));
  auto buf = to_ucx_buffer(mr, std::move(t));
  buf.set_send_attr(std::move(attr));
  return buf;
}

// The tensor description(s) go last in the parameter list, where the receiver looks first:
// 1: one TENSOR_META, 2: one TENSOR_META_VEC.
void append_tensor_metas(rpc::data::vector<rpc::ParamMeta>& params, rpc::TensorMetaVec&& metas, int add_meta) {
  if (add_meta == 1 && metas.size() == 1) {
    params.push_back(rpc::ParamMeta(rpc::ParamType::TENSOR_META, rpc::ParamValue(std::in_place_type<rpc::TensorMeta>, std::move(metas[0]))));
  } else if (add_meta != 0) {
    params.push_back(rpc::ParamMeta(rpc::ParamType::TENSOR_META_VEC, rpc::ParamValue(std::in_place_type<rpc::TensorMetaVec>, std::move(metas))));
  }
}

// Buffers handed to Python may outlive the runtime that received them (a result tensor kept
// after `stop()`), and they return their bytes to the memory resource: each one keeps it alive.
py::object payload_to_python(PayloadVariant&& p, int device_id, std::shared_ptr<ucxx::UcxMemoryResourceManager> mr) {
  if (auto* b = std::get_if<UcxBuffer>(&p))
    return py::cast(PyBuffer{std::shared_ptr<UcxBuffer>(new UcxBuffer(std::move(*b)), [mr](UcxBuffer* x) { delete x; }), device_id});
  if (auto* v = std::get_if<UcxBufferVec>(&p))
    return py::cast(PyBufferVec{std::shared_ptr<UcxBufferVec>(new UcxBufferVec(std::move(*v)), [mr](UcxBufferVec* x) { delete x; }), device_id});
  return py::none();
}

std::string error_text(const std::exception_ptr& e) {
  try {
    std::rethrow_exception(e);
  } catch (const std::exception& ex) {
    return ex.what();
  } catch (...) {
    return "unknown error";
  }
}

}  // namespace

class PyAxonRuntime {
 public:
  PyAxonRuntime(const std::string& worker_name, size_t thread_pool_size, py::object timeout, py::object device,
                std::shared_ptr<ucxx::UcxMemoryResourceManager> mr)
      : name_(worker_name) {
    std::unique_ptr<ucxx::UcxAutoDeviceContext> dev;
    if (!device.is_none()) {
      std::string kind = py::hasattr(device, "kind") ? device.attr("kind").cast<std::string>() : std::string(py::str(device));
      int index = py::hasattr(device, "index") ? device.attr("index").cast<int>() : 0;
      if (kind == "cuda") {
        device_id_ = index;
        is_cuda_ = true;
        dev = std::make_unique<ucxx::UcxAutoCudaDeviceContext>(index);
        if (!mr) {
          ucxx::UcxCudaMemoryResourceManager::Options opt;
          opt.device = index;
          mr = std::make_shared<ucxx::UcxCudaMemoryResourceManager>(opt);
        }
      } else if (kind != "cpu") {
        throw py::value_error("this build drives cpu and cuda devices; got '" + kind + "'");
      }
    }
    mr_ = mr ? mr : default_manager();
    if (thread_pool_size == 0) thread_pool_size = axon::AxonWorker::DefaultThreadPoolSize();
    rt_ = std::make_unique<axon::AxonRuntime>(worker_name, thread_pool_size, parse_timeout(timeout), std::move(dev), mr_);
  }
  ~PyAxonRuntime() {
    try {
      stop();
    } catch (...) {
    }
  }

  // ---- lifecycle ----
  void attach_loop() {
    py::object asyncio = py::module_::import("asyncio");
    py::object loop;
    try {
      loop = asyncio.attr("get_running_loop")();
    } catch (py::error_already_set&) {
      // outside a running loop (registration before the program's loop exists): use the thread's
      // current loop if it is usable, otherwise wait for the next call made from inside a loop
      try {
        loop = asyncio.attr("get_event_loop")();
      } catch (py::error_already_set&) {
        return;
      }
      if (loop.attr("is_closed")().cast<bool>()) return;
    }
    wake_.attach(loop);
  }
  void start() {
    attach_loop();
    open_gate();
    throw_if(rt_->Start());
  }
  void start_server() {
    attach_loop();
    open_gate();
    throw_if(rt_->StartServer());
  }
  void start_client() {
    attach_loop();
    throw_if(rt_->StartClient());
  }
  // No call reaches the event loop from here on; those already queued for it are answered now (on this thread,
  // which is the loop's), because the code that follows blocks this thread until every call has an answer.
  void close_gate() {
    {
      std::lock_guard lk(gate_mu_);
      stopping_ = true;
    }
    wake_.process_queue();
  }
  void open_gate() {
    std::lock_guard lk(gate_mu_);
    stopping_ = false;
  }
  void stop() {
    if (!rt_) return;
    close_gate();
    // handlers that are still awaiting are answered with CANCELLED and their tasks cancelled
    auto running = std::move(running_tasks_);
    running_tasks_.clear();
    for (auto& [id, t] : running) {
      t.answer_cancelled();
      try {
        t.task.attr("cancel")();
      } catch (py::error_already_set&) {
      }
    }
    running.clear();
    {
      py::gil_scoped_release nogil;  // worker threads may be waiting for the GIL to finish their callbacks
      rt_->Stop();
      ex::sync_wait(scope_.cleanup());
    }
    wake_.process_queue();
    wake_.detach();
  }
  void stop_server() {
    close_gate();
    auto running = std::move(running_tasks_);
    running_tasks_.clear();
    for (auto& [id, t] : running) {
      t.answer_cancelled();
      try {
        t.task.attr("cancel")();
      } catch (py::error_already_set&) {
      }
    }
    running.clear();
    py::gil_scoped_release nogil;
    rt_->StopServer();
  }
  void stop_client() {
    py::gil_scoped_release nogil;
    rt_->StopClient();
  }
  py::bytes get_local_address() {
    auto a = rt_->GetLocalAddress();
    return py::bytes(reinterpret_cast<const char*>(a.data()), a.size());
  }
  py::bytes get_local_signatures() {
    auto b = rt_->GetLocalSignatures();
    return py::bytes(reinterpret_cast<const char*>(b.data()), b.size());
  }
  bool register_endpoint_signatures(const std::string& worker_name, py::bytes data) {
    std::string s = data;
    return rt_->RegisterEndpointSignatures(worker_name, s.data(), s.size());
  }
  void set_timeout(py::object t) { rt_->SetTimeout(parse_timeout(t)); }
  void set_reject_messages(bool r) { rt_->SetRejectMessages(r); }
  std::string worker_name() const { return name_; }
  py::dict transport_stats() {
    const auto s = rt_->worker().GetTransportStats();
    py::dict d;
    d["frames_refused"] = s.frames_refused;
    d["regions_ignored"] = s.regions_ignored;
    d["device_pulls"] = s.device_pulls;
    d["device_staged"] = s.device_staged;
    d["truncated"] = s.truncated;
    d["device_eager_sent"] = s.device_eager_sent;
    d["device_eager_recv"] = s.device_eager_recv;
    d["device_pushes"] = s.device_pushes;
    d["device_push_recv"] = s.device_push_recv;
    d["kernel_launches"] = s.kernel_launches;
    d["device_gathers"] = s.device_gathers;
    d["device_packs"] = s.device_packs;
    d["sends_held"] = s.sends_held;
    d["vmm_fds_sent"] = s.vmm_fds_sent;
    d["vmm_fds_recv"] = s.vmm_fds_recv;
    return d;
  }
  size_t stored_request_count() { return rt_->worker().GetStorage().size(); }
  std::string save_stored_requests(const std::string& dir, const std::string& prefix) {
    py::gil_scoped_release nogil;
    return rt_->worker().GetStorage().save(*mr_, dir, prefix);
  }
  size_t load_stored_requests(const std::string& path) {
    py::gil_scoped_release nogil;
    return rt_->worker().GetStorage().load(*mr_, path);
  }
  // Python handlers run on the event loop, so re-processing must not block it: the work runs on a
  // helper thread and the caller awaits the returned future.
  py::object process_stored_requests();

  // ---- futures ----
  // Run `sender`; resolve a new asyncio future with `convert(value)` on the loop thread.
  template <class Sender, class Convert>
  py::object future_from(Sender&& sender, Convert convert) {
    attach_loop();
    py::object fut = wake_.loop().attr("create_future")();
    auto fut_box = gil_shared(fut);  // destroyed on the loop thread, under the GIL
    auto settle = [this, fut_box](std::function<void(py::object&)> fn) {
      ucxx::nvtx_mark("axon.python.result_queued");
      wake_.enqueue([fut_box, fn = std::move(fn)] {
        ucxx::NvtxRange range("axon.python.result_on_loop");
        py::object f = *fut_box;
        if (!f.attr("done")().cast<bool>()) fn(f);
      });
    };
    using V = ex::value_t<Sender>;
    auto on_value = [settle, convert](V v) mutable {
      auto box = std::make_shared<V>(std::move(v));
      settle([box, convert](py::object& f) mutable {
        try {
          f.attr("set_result")(convert(std::move(*box)));
        } catch (py::error_already_set& e) {
          f.attr("set_exception")(e.value());
        } catch (const std::exception& e) {
          f.attr("set_exception")(py::module_::import("builtins").attr("RuntimeError")(e.what()));
        }
      });
    };
    auto on_error = [settle](std::exception_ptr e) {
      std::string text = error_text(e);
      settle([text](py::object& f) { f.attr("set_exception")(py::module_::import("builtins").attr("RuntimeError")(text)); });
    };
    auto on_done = [settle] { settle([](py::object& f) { f.attr("cancel")(); }); };
    {
      py::gil_scoped_release nogil;
      scope_.spawn_detached(ex::upon_done(ex::upon_error(ex::then(std::forward<Sender>(sender), std::move(on_value)), std::move(on_error)), std::move(on_done)));
    }
    return fut;
  }

  py::object connect_endpoint_async(py::object address, const std::string& worker_name) {
    std::string bytes = py::isinstance<py::bytes>(address) ? std::string(address.cast<py::bytes>()) : std::string(py::bytes(py::bytearray(address)));
    std::vector<std::byte> addr(bytes.size());
    std::memcpy(addr.data(), bytes.data(), bytes.size());
    return future_from(rt_->ConnectEndpointAsync(std::move(addr), worker_name), [](uint64_t conn) -> py::object { return py::int_(conn); });
  }

  // ---- memory policy from Python ----
  // callable(list[TensorMeta]) -> tensor | list[tensor]; the returned objects are remembered so the
  // caller gets the very same objects back once the data has landed in them.
  ServerMemoryPolicy server_policy(py::object policy) {
    ServerMemoryPolicy p;
    if (policy.is_none()) return p;
    p.on_host = false;
    // Called on the context's own thread (with the GIL taken there) instead of on a pool thread: waking a
    // pool thread and bouncing back costs about 100 us per message, the call itself a few. The loop
    // thread holds the GIL only while Python code runs, and while it does no handler could run either.
    p.provider_inline = true;
    auto fn = gil_shared(policy);
    auto* mr = mr_.get();
    // The policy runs on a pool thread whose current CUDA device is the default one; tensor
    // libraries refuse to export a tensor of another device, so the thread adopts the runtime's.
    const int cuda_dev = is_cuda_ ? device_id_ : -1;
    p.buffer_provider = [fn, mr, cuda_dev](rpc::utils::TensorMetaSpan metas) -> UcxBuffer {
      if (cuda_dev >= 0) cudaSetDevice(cuda_dev);
      py::gil_scoped_acquire gil;
      py::list lst;
      for (auto& m : metas) lst.append(py::cast(m));
      py::object out = (*fn)(lst);
      if (py::isinstance<py::list>(out) || py::isinstance<py::tuple>(out)) out = py::reinterpret_borrow<py::sequence>(out)[0];
      if (auto direct = receive_buffer_of(*mr, out)) return std::move(*direct);
      ImportedTensor t = import_tensor(out);
      remember_owner(t.data, out);
      return to_ucx_buffer(*mr, std::move(t));
    };
    p.buffer_vec_provider = [fn, mr, cuda_dev](rpc::utils::TensorMetaSpan metas) -> UcxBufferVec {
      if (cuda_dev >= 0) cudaSetDevice(cuda_dev);
      py::gil_scoped_acquire gil;
      py::list lst;
      for (auto& m : metas) lst.append(py::cast(m));
      py::object out = (*fn)(lst);
      std::vector<ImportedTensor> ts;
      if (py::isinstance<py::list>(out) || py::isinstance<py::tuple>(out)) {
        for (auto item : out) {
          ts.push_back(import_tensor(item));
          remember_owner(ts.back().data, py::reinterpret_borrow<py::object>(item));
        }
      } else {
        ts.push_back(import_tensor(out));
        remember_owner(ts.back().data, out);
      }
      return to_ucx_buffer_vec(*mr, std::move(ts));
    };
    return p;
  }
  // A tensor that says where it is (torch: data_ptr(), numel(), element_size(), is_contiguous(), is_cuda)
  // becomes a receive buffer without a DLPack export: the export of a CUDA tensor orders streams and
  // builds a capsule, tens of microseconds that a buffer about to be overwritten does not need.
  static std::optional<UcxBuffer> receive_buffer_of(ucxx::UcxMemoryResourceManager& mr, py::object& out) {
    if (!py::hasattr(out, "data_ptr") || !py::hasattr(out, "element_size") || !py::hasattr(out, "is_contiguous")) return std::nullopt;
    try {
      if (!out.attr("is_contiguous")().cast<bool>()) return std::nullopt;
      void* data = reinterpret_cast<void*>(out.attr("data_ptr")().cast<uintptr_t>());
      const size_t bytes = out.attr("numel")().cast<size_t>() * out.attr("element_size")().cast<size_t>();
      const bool on_gpu = py::hasattr(out, "is_cuda") && out.attr("is_cuda").cast<bool>();
      remember_owner(data, out);
      auto keep = gil_shared(out);
      UcxBuffer buf(mr, on_gpu ? ucx_memory_type::CUDA : ucx_memory_type::HOST, data, bytes, nullptr, true,
                    [keep](void*) mutable { keep.reset(); });
      if (on_gpu && bytes) {
        // memory fresh from the tensor library's allocator may still be in use by work queued on its stream
        // before it was handed out: the transport writes it after that work (an event on that stream)
        int device = 0;
        try {
          device = out.attr("device").attr("index").cast<int>();
        } catch (const std::exception&) {
          PyErr_Clear();
        }
        buf.set_send_attr(make_send_attr(nullptr, device, producer_stream(out, device)));
      }
      return buf;
    } catch (py::error_already_set&) {
      return std::nullopt;  // not that kind of object after all: the DLPack road
    }
  }

  ClientMemoryPolicy client_policy(py::object policy, bool want_vec) {
    ClientMemoryPolicy c;
    c.want_vec = want_vec;
    if (policy.is_none()) return c;
    ServerMemoryPolicy s = server_policy(policy);
    c.on_host = false;
    c.buffer_provider = std::move(s.buffer_provider);
    c.buffer_vec_provider = std::move(s.buffer_vec_provider);
    c.provider_inline = s.provider_inline;  // as on the server: called on the context's thread, no hand-over to the pool and back
    return c;
  }

  // ---- invoke ----
  // `transform(response_header, payload)`, when given, runs on the loop thread and its result (or
  // the exception it raises) settles the future: one loop iteration instead of a chained future.
  // `add_meta` (1: TENSOR_META, 2: TENSOR_META_VEC): describe the payload tensors in the header here.
  py::object invoke_raw(const std::string& worker_name, rpc::RpcRequestHeader header, py::object payload, py::object memory_policy,
                        bool response_as_list, py::object transform, int add_meta, int wire_dtype) {
    rpc::TensorMetaVec metas;
    PayloadVariant p = payload_from_python(*mr_, payload, add_meta ? &metas : nullptr, wire_dtype);
    if (add_meta) append_tensor_metas(header.params, std::move(metas), add_meta);
    ClientMemoryPolicy pol = client_policy(memory_policy, response_as_list);
    if (response_as_list && !memory_policy.is_none()) pol.buffer_provider = nullptr;
    const int dev = device_id_;
    auto mr = mr_;
    std::shared_ptr<py::object> tf = transform.is_none() ? nullptr : gil_shared(transform);
    return future_from(rt_->InvokeRpc(std::string_view(worker_name), std::move(header), std::move(p), std::move(pol)),
                       [dev, mr, tf](InvokeResult r) -> py::object {
                         py::object payload_obj = payload_to_python(std::move(r.payload), dev, mr);
                         if (tf) return (*tf)(py::cast(std::move(r.header)), payload_obj);
                         return py::make_tuple(py::cast(std::move(r.header)), payload_obj);
                       });
  }

  // ---- remote GEMM service (see eux/axon/services/remote_gemm_service.hpp) ----
  axon::services::RemoteGemmService& gemm_service() {
    if (!gemm_) {
      auto cuda_mr = std::dynamic_pointer_cast<ucxx::UcxCudaMemoryResourceManager>(mr_);
      if (!cuda_mr) throw std::runtime_error("the remote GEMM service needs a runtime on a cuda device");
      gemm_ = std::make_unique<axon::services::RemoteGemmService>(rt_->worker(), cuda_mr);
    }
    return *gemm_;
  }
  void gemm_add_weight(uint32_t weight_id, uintptr_t w_t, int n, int k, int format, int max_m, uintptr_t w_scale) {
    axon::services::GemmWeight w;
    w.w_t = reinterpret_cast<const void*>(w_t);
    w.w_scale = reinterpret_cast<const void*>(w_scale);
    w.n = n;
    w.k = k;
    w.format = static_cast<axon::services::GemmFormat>(format);
    w.max_m = max_m;
    auto& svc = gemm_service();
    svc.AddWeight(weight_id, w);
    if (!svc.Register()) throw std::runtime_error("the remote GEMM function could not be registered");
  }
  uint64_t gemm_launches() { return gemm_ ? gemm_->launches() : 0; }
  std::array<uint64_t, 3> gemm_progress() { return gemm_ ? gemm_->progress() : std::array<uint64_t, 3>{0, 0, 0}; }
  py::object remote_gemm(const std::string& worker_name, uint32_t weight_id, int m, uintptr_t x, size_t x_bytes, uintptr_t y, size_t y_bytes,
                         uintptr_t xs, size_t xs_bytes) {
    return future_from(gemm_service().Call(worker_name, weight_id, m, reinterpret_cast<const void*>(x), x_bytes, reinterpret_cast<void*>(y),
                                           y_bytes, reinterpret_cast<const void*>(xs), xs_bytes),
                       [](int32_t status) -> py::object { return py::int_(status); });
  }

  // ---- symmetric peer memory (see eux/axon/services/peer_memory_service.hpp) ----
  void peer_memory_init(int rank, int world) {
    auto cuda_mr = std::dynamic_pointer_cast<ucxx::UcxCudaMemoryResourceManager>(mr_);
    if (!cuda_mr) throw std::runtime_error("peer memory needs a runtime on a cuda device");
    peer_mem_ = std::make_unique<axon::services::PeerMemoryService>(rt_->worker(), cuda_mr, rank, world);
    if (!peer_mem_->Register()) throw std::runtime_error("the peer-memory function could not be registered");
  }
  axon::services::PeerMemoryService& peer_memory() {
    if (!peer_mem_) throw std::runtime_error("call peer_memory_init(rank, world) first");
    return *peer_mem_;
  }
  uintptr_t peer_memory_alloc(uint32_t tag, size_t nbytes) { return reinterpret_cast<uintptr_t>(peer_memory().Allocate(tag, nbytes)); }
  py::object peer_memory_publish(const std::string& worker_name, uint32_t tag) {
    return future_from(peer_memory().Publish(worker_name, tag), [](int32_t v) -> py::object { return py::int_(v); });
  }
  int peer_memory_arrived(uint32_t tag) { return peer_memory().Arrived(tag); }
  std::vector<uintptr_t> peer_memory_resolve(uint32_t tag) { return peer_memory().Resolve(tag); }
  void peer_memory_free(uint32_t tag) { peer_memory().Free(tag); }

  // ---- server-side functions ----
  // `callable(header: RpcRequestHeader, payload) -> awaitable of (RpcResponseHeader | list of results, payload | None)`.
  bool register_function_raw(uint32_t function_id, const std::string& function_name, std::vector<rpc::ParamType> param_types,
                             std::vector<rpc::ParamType> return_types, rpc::PayloadType input_payload_type,
                             rpc::PayloadType return_payload_type, py::object callable, py::object memory_policy, py::object lifecycle_policy) {
    attach_loop();
    auto fn = gil_shared(std::move(callable));
    auto* self = this;
    rpc::DynamicAsyncRpcFunction handler = [self, fn](const rpc::RpcRequestHeader& req, PayloadVariant&& payload,
                                                     const rpc::RpcResponseBuilder& builder) -> rpc::AsyncInvokeSender {
      struct State {
        rpc::RpcRequestHeader req;
        rpc::RpcResponseBuilder builder;
        PayloadVariant payload;
      };
      auto st = std::make_shared<State>(State{req, builder, std::move(payload)});
      return rpc::AsyncInvokeSender(ex::create<rpc::RpcInvokeResult<rpc::ReturnedPayload>>([self, fn, st](auto handle) {
        // hop to the asyncio thread: start the coroutine as a task, finish the C++ call from its done-callback
        ucxx::nvtx_mark("axon.python.handler_queued");
        // A runtime that is stopping takes no more work onto the event loop: its stop() runs on the loop's thread
        // and waits there for every call to be answered, so a call that waited for the loop would wait for ever.
        // The gate is closed and the queue drained under one mutex, so that no call slips in between.
        std::unique_lock gate(self->gate_mu_);
        if (self->stopping_) {
          gate.unlock();
          handle.set_value(rpc::RpcInvokeResult<rpc::ReturnedPayload>{
              st->builder.PrepareError(st->req.session_id, st->req.request_id, rpc::make_error_code(rpc::RpcErrc::UNAVAILABLE), "the server is stopping"),
              rpc::ReturnedPayload{}});
          return;
        }
        self->wake_.enqueue([self, fn, st, handle]() mutable {
          ucxx::NvtxRange range("axon.python.handler_on_loop");
          // the call is answered exactly once: by the task's completion, or by stop() while it still runs
          auto settled = std::make_shared<std::atomic<bool>>(false);
          auto fail = [st, handle, settled](std::error_code ec, const std::string& what) mutable {
            if (settled->exchange(true)) return;
            py::gil_scoped_release nogil;
            handle.set_value(rpc::RpcInvokeResult<rpc::ReturnedPayload>{
                st->builder.PrepareError(st->req.session_id, st->req.request_id, ec, what), rpc::ReturnedPayload{}});
          };
          if (self->stopping_) {  // queued before the gate closed, run by stop()'s drain
            fail(rpc::make_error_code(rpc::RpcErrc::UNAVAILABLE), "the server is stopping");
            return;
          }
          try {
            py::object payload_obj = payload_to_python(std::move(st->payload), self->device_id_, self->mr_);
            py::object coro = (*fn)(py::cast(st->req), payload_obj);
            // The first step of the coroutine runs right here (eager start): a handler that awaits
            // nothing is finished when the constructor returns, and its reply leaves in this loop
            // iteration instead of two iterations later.
            py::object asyncio = py::module_::import("asyncio");
            py::object task;
            try {
              task = asyncio.attr("Task")(coro, py::arg("loop") = self->wake_.loop(), py::arg("eager_start") = true);
            } catch (py::error_already_set& e) {
              if (!e.matches(PyExc_TypeError)) throw;
              task = asyncio.attr("ensure_future")(coro, py::arg("loop") = self->wake_.loop());  // interpreters before 3.12
            }
            const uint64_t task_id = self->next_task_id_++;
            auto finish = py::cpp_function([self, st, handle, fail, settled, task_id](py::object t) mutable {
              self->running_tasks_.erase(task_id);
              try {
                if (settled->load()) return;  // stop() answered for this task
                if (t.attr("cancelled")().cast<bool>()) {
                  fail(rpc::make_error_code(rpc::RpcErrc::CANCELLED), "the handler task was cancelled");
                  return;
                }
                py::object exc = t.attr("exception")();
                if (!exc.is_none()) {
                  fail(rpc::make_error_code(rpc::RpcErrc::INTERNAL), std::string(py::str(py::type::of(exc).attr("__name__"))) + ": " + std::string(py::str(exc)));
                  return;
                }
                py::object res = t.attr("result")();
                py::object head = res, pay = py::none();
                int add_meta = 0;    // third element: describe the payload tensors in the header here (see invoke_raw)
                int wire_dtype = 0;  // fourth: the type in which a device tensor's elements travel
                if (py::isinstance<py::tuple>(res) && py::len(res) >= 2) {
                  auto tup = res.cast<py::tuple>();
                  head = tup[0];
                  pay = tup[1];
                  if (py::len(res) >= 3) add_meta = tup[2].cast<int>();
                  if (py::len(res) >= 4) wire_dtype = tup[3].cast<int>();
                }
                rpc::RpcResponseHeader h;
                if (py::isinstance<rpc::RpcResponseHeader>(head)) {
                  h = head.cast<rpc::RpcResponseHeader>();
                } else {
                  h = st->builder.PrepareResponse(st->req.session_id, st->req.request_id);
                  if (!head.is_none())
                    for (auto item : head) h.results.push_back(py::isinstance<rpc::ParamMeta>(item) ? item.cast<rpc::ParamMeta>() : python_to_param(item));
                }
                h.session_id = st->req.session_id;
                h.request_id = st->req.request_id;
                rpc::TensorMetaVec metas;
                PayloadVariant out = payload_from_python(*self->mr_, pay, add_meta ? &metas : nullptr, wire_dtype);
                if (add_meta) append_tensor_metas(h.results, std::move(metas), add_meta);
                if (settled->exchange(true)) return;
                py::gil_scoped_release nogil;
                handle.set_value(rpc::RpcInvokeResult<rpc::ReturnedPayload>{std::move(h), std::move(out)});
              } catch (py::error_already_set& e) {
                fail(rpc::make_error_code(rpc::RpcErrc::INTERNAL), e.what());
              } catch (const std::exception& e) {
                fail(rpc::make_error_code(rpc::RpcErrc::INTERNAL), e.what());
              }
            });
            if (task.attr("done")().cast<bool>()) {
              finish(task);
            } else {
              // still running (it awaits something): stop() must be able to answer for it, because a
              // stop() on the loop's thread cannot wait for a task that needs the loop
              self->running_tasks_.emplace(task_id, RunningTask{task, [fail]() mutable {
                fail(rpc::make_error_code(rpc::RpcErrc::CANCELLED), "the runtime stopped while the handler was running");
              }});
              task.attr("add_done_callback")(finish);
            }
          } catch (py::error_already_set& e) {
            fail(rpc::make_error_code(rpc::RpcErrc::INTERNAL), e.what());
          } catch (const std::exception& e) {
            fail(rpc::make_error_code(rpc::RpcErrc::INTERNAL), e.what());
          }
        });
      }));
    };
    axon::MessageLifecyclePolicy lc = axon::TransientPolicy{};
    if (!lifecycle_policy.is_none()) {
      auto lcf = gil_shared(lifecycle_policy);
      lc = axon::RetentionPolicy([lcf](std::shared_ptr<axon::utils::AxonRequest> req, axon::utils::AxonMessageID id) {
        py::gil_scoped_acquire gil;
        py::object r = (*lcf)(py::cast(req->header), id);
        if (py::isinstance<py::bool_>(r)) return r.cast<bool>() ? axon::LifecycleStatus::Preserve : axon::LifecycleStatus::Discard;
        return static_cast<axon::LifecycleStatus>(r.cast<int>());
      });
    }
    ServerMemoryPolicy mem = server_policy(memory_policy);
    mem.handler_inline = true;  // the handler above only queues the call for the event loop
    return rt_->RegisterFunction(rpc::function_id_t{function_id}, function_name, rpc::data::vector<rpc::ParamType>(param_types.begin(), param_types.end()),
                                 rpc::data::vector<rpc::ParamType>(return_types.begin(), return_types.end()), input_payload_type,
                                 return_payload_type, std::move(handler), std::move(mem), std::move(lc));
  }

 private:
  static void throw_if(std::error_code ec) {
    if (ec) throw std::runtime_error("axon: " + ec.message());
  }
  std::string name_;
  int device_id_ = 0;
  bool is_cuda_ = false;
  std::shared_ptr<ucxx::UcxMemoryResourceManager> mr_;
  PythonWakeManager wake_;
  std::mutex gate_mu_;      // see close_gate()
  bool stopping_ = false;
  struct RunningTask {
    py::object task;
    std::function<void()> answer_cancelled;
  };
  std::unordered_map<uint64_t, RunningTask> running_tasks_;  // touched on the loop thread only (under the GIL)
  uint64_t next_task_id_ = 1;
  ex::static_thread_pool helper_{1};
  ex::async_scope scope_;
  std::unique_ptr<axon::AxonRuntime> rt_;
  std::unique_ptr<axon::services::PeerMemoryService> peer_mem_;
  std::unique_ptr<axon::services::RemoteGemmService> gemm_;  // declared after rt_: destroyed before the worker it is registered on
};

py::object PyAxonRuntime::process_stored_requests() {
  auto* worker = &rt_->worker();
  return future_from(ex::on(helper_.get_scheduler(), ex::just_from([worker] { return worker->ProcessStoredRequests(); })),
                     [](size_t n) -> py::object { return py::int_(n); });
}

void bind_runtime(py::module_& m) {
  py::class_<ucxx::UcxMemoryResourceManager, std::shared_ptr<ucxx::UcxMemoryResourceManager>>(m, "UcxMemoryResourceManager");
  py::class_<ucxx::DefaultUcxMemoryResourceManager, ucxx::UcxMemoryResourceManager, std::shared_ptr<ucxx::DefaultUcxMemoryResourceManager>>(
      m, "DefaultUcxMemoryResourceManager")
      .def(py::init<>());
  py::class_<ucxx::UcxCudaMemoryResourceManager, ucxx::UcxMemoryResourceManager, std::shared_ptr<ucxx::UcxCudaMemoryResourceManager>>(
      m, "CudaMemoryResourceManager")
      .def(py::init([](int device, size_t arena_bytes) {
             ucxx::UcxCudaMemoryResourceManager::Options o;
             o.device = device;
             o.arena_bytes = arena_bytes;
             return std::make_shared<ucxx::UcxCudaMemoryResourceManager>(o);
           }),
           py::arg("device") = 0, py::arg("arena_bytes") = size_t(64) << 20)
      .def("pooled_bytes", &ucxx::UcxCudaMemoryResourceManager::pooled_bytes)
      .def("pooled_bytes_in_use", &ucxx::UcxCudaMemoryResourceManager::pooled_bytes_in_use);
  m.def("get_default_resource_manager", [] { return default_manager(); });
  m.def("_spin_for_wake", [](double seconds) {
    py::gil_scoped_release nogil;
    return spin_for_wake(std::chrono::nanoseconds(static_cast<int64_t>(seconds * 1e9)));
  }, "Spin without the GIL until a native thread has queued work for an event loop of this process, or the time is up.");
  m.def("get_device_context_handle", [](const std::string& kind) -> py::object {
    if (kind != "cuda") return py::none();
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) {
      cudaGetLastError();
      return py::none();
    }
    return py::int_(dev);
  }, "The CUDA device current on the calling thread, or None.");

  py::class_<PyAxonRuntime>(m, "AxonRuntime")
      .def(py::init<const std::string&, size_t, py::object, py::object, std::shared_ptr<ucxx::UcxMemoryResourceManager>>(), py::arg("worker_name"),
           py::arg("thread_pool_size") = 0, py::arg("timeout") = py::none(), py::arg("device") = py::none(), py::arg("resource_manager") = nullptr)
      .def("start", &PyAxonRuntime::start).def("start_server", &PyAxonRuntime::start_server).def("start_client", &PyAxonRuntime::start_client)
      .def("stop", &PyAxonRuntime::stop).def("stop_server", &PyAxonRuntime::stop_server).def("stop_client", &PyAxonRuntime::stop_client)
      .def("get_local_address", &PyAxonRuntime::get_local_address).def("get_local_signatures", &PyAxonRuntime::get_local_signatures)
      .def("register_endpoint_signatures", &PyAxonRuntime::register_endpoint_signatures)
      .def("connect_endpoint_async", &PyAxonRuntime::connect_endpoint_async, py::arg("ucp_address"), py::arg("worker_name"))
      .def("_register_native", &PyAxonRuntime::register_function_raw, py::arg("function_id"), py::arg("function_name"), py::arg("param_types"),
           py::arg("return_types"), py::arg("input_payload_type"), py::arg("return_payload_type"), py::arg("callable"),
           py::arg("memory_policy") = py::none(), py::arg("lifecycle_policy") = py::none())
      .def("_invoke_native", &PyAxonRuntime::invoke_raw, py::arg("worker_name"), py::arg("request_header"), py::arg("payload") = py::none(),
           py::arg("memory_policy") = py::none(), py::arg("response_as_list") = false, py::arg("transform") = py::none(),
           py::arg("add_meta") = 0, py::arg("wire_dtype") = 0)
      .def("_gemm_add_weight", &PyAxonRuntime::gemm_add_weight, py::arg("weight_id"), py::arg("w_t"), py::arg("n"), py::arg("k"), py::arg("format"),
           py::arg("max_m"), py::arg("w_scale") = 0)
      .def("_remote_gemm", &PyAxonRuntime::remote_gemm, py::arg("worker_name"), py::arg("weight_id"), py::arg("m"), py::arg("x"), py::arg("x_bytes"),
           py::arg("y"), py::arg("y_bytes"), py::arg("x_scale") = 0, py::arg("x_scale_bytes") = 0)
      .def("peer_memory_init", &PyAxonRuntime::peer_memory_init, py::arg("rank"), py::arg("world"))
      .def("peer_memory_alloc", &PyAxonRuntime::peer_memory_alloc, py::arg("tag"), py::arg("nbytes"))
      .def("peer_memory_publish", &PyAxonRuntime::peer_memory_publish, py::arg("worker_name"), py::arg("tag"))
      .def("peer_memory_arrived", &PyAxonRuntime::peer_memory_arrived, py::arg("tag"))
      .def("peer_memory_resolve", &PyAxonRuntime::peer_memory_resolve, py::arg("tag"))
      .def("peer_memory_free", &PyAxonRuntime::peer_memory_free, py::arg("tag"))
      .def("gemm_progress", &PyAxonRuntime::gemm_progress, "(launches issued, completions seen, kernel status word) of the remote-GEMM handler")
      .def("gemm_launches", &PyAxonRuntime::gemm_launches, "GEMM kernels launched by this runtime's remote-GEMM handler so far.")
      .def("set_timeout", &PyAxonRuntime::set_timeout).def("set_reject_messages", &PyAxonRuntime::set_reject_messages)
      .def_property_readonly("worker_name", &PyAxonRuntime::worker_name)
      .def("transport_stats", &PyAxonRuntime::transport_stats,
           "Counters of the transports under this runtime: device payloads pulled / pushed / sent eagerly / staged through the host, frames refused.")
      .def("stored_request_count", &PyAxonRuntime::stored_request_count)
      .def("save_stored_requests", &PyAxonRuntime::save_stored_requests, py::arg("directory"), py::arg("prefix") = "axon")
      .def("load_stored_requests", &PyAxonRuntime::load_stored_requests).def("process_stored_requests", &PyAxonRuntime::process_stored_requests);
}

}  // namespace eux::python
