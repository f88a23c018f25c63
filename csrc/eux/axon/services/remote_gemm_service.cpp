#include "eux/axon/services/remote_gemm_service.hpp"

#include <cuda_runtime_api.h>
#include <unistd.h>

#include <cstring>
#include <stdexcept>

#include "eux/axon/utils/hash.hpp"
#include "eux/ucxx/nvtx_range.hpp"
#include "eux/ucxx/transport.hpp"
#include "kernels/eux_kernels.h"

namespace eux::axon::services {

namespace ex = eux::exec;
using rpc::data::vector;
using ucxx::PeerRegionDesc;

namespace {
constexpr size_t kSchedWords = 64;

vector<uint8_t> desc_bytes(const PeerRegionDesc& d) {
  vector<uint8_t> v(sizeof(d));
  std::memcpy(v.data(), &d, sizeof(d));
  return v;
}
bool desc_from(const vector<uint8_t>& v, PeerRegionDesc* d) {
  if (v.size() != sizeof(*d)) return false;
  std::memcpy(d, v.data(), sizeof(*d));
  return true;
}
size_t x_elem_bytes(GemmFormat f) { return f == GemmFormat::kBf16 ? 2 : 1; }
size_t x_scale_bytes_for(GemmFormat f, int64_t m, int64_t k) {
  if (f == GemmFormat::kFp8Block) return size_t(m) * size_t(k / 128) * 4;
  if (f == GemmFormat::kMxFp8) return size_t(m) * size_t(k / 32);
  return 0;
}
}  // namespace

RemoteGemmService::RemoteGemmService(AxonWorker& worker, std::shared_ptr<ucxx::UcxCudaMemoryResourceManager> mr)
    : worker_(worker), mr_(std::move(mr)) {
  if (!mr_) throw std::invalid_argument("RemoteGemmService needs the CUDA memory resource manager of its worker");
}

RemoteGemmService::~RemoteGemmService() {
  if (registered_) worker_.UnregisterFunction(rpc::function_id_t{utils::FunctionIdFromName(kFunctionName, worker_.name())});
  if (stream_) {
    cudaSetDevice(mr_->device());
    cudaStreamSynchronize(static_cast<cudaStream_t>(stream_));
    cudaStreamDestroy(static_cast<cudaStream_t>(stream_));
  }
  for (auto& [id, r] : weights_) {
    try {
      if (r.x_stage) mr_->deallocate(ucx_memory_type::CUDA, r.x_stage, r.x_stage_bytes);
      if (r.xs_stage) mr_->deallocate(ucx_memory_type::CUDA, r.xs_stage, r.xs_stage_bytes);
      if (r.scratch) mr_->deallocate(ucx_memory_type::CUDA, r.scratch, r.scratch_bytes);
    } catch (...) {
    }
  }
  if (flag_host_) eux_host_free(flag_host_);
}

bool RemoteGemmService::EnsureDevice() {
  if (stream_) return true;
  cudaStream_t st = nullptr;
  if (cudaSetDevice(mr_->device()) != cudaSuccess || cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  void *h = nullptr, *d = nullptr;
  if (eux_host_alloc_mapped(&h, &d, 256) != 0) {
    cudaStreamDestroy(st);
    return false;
  }
  std::memset(h, 0, 256);
  // the handler launches on behalf of a peer: its kernels are loaded now, not by their first launch
  if (int rc = eux_gemm_preload(); rc != 0) {
    eux_host_free(h);
    cudaStreamDestroy(st);
    return false;
  }
  flag_host_ = static_cast<uint64_t*>(h);
  flag_dev_ = static_cast<uint64_t*>(d);
  stream_ = st;
  return true;
}

void RemoteGemmService::AddWeight(uint32_t weight_id, const GemmWeight& w) {
  if (!w.w_t || w.n <= 0 || w.k <= 0 || w.max_m <= 0 || w.max_m % 128 || (w.format != GemmFormat::kBf16 && !w.w_scale))
    throw std::invalid_argument("RemoteGemmService::AddWeight: incomplete weight description");
  std::lock_guard lk(mu_);
  if (!EnsureDevice()) throw std::runtime_error("RemoteGemmService: no CUDA device");
  if (weights_.count(weight_id)) throw std::invalid_argument("RemoteGemmService::AddWeight: the id is taken");
  Resident r;
  r.w = w;
  r.x_stage_bytes = size_t(w.max_m) * size_t(w.k) * x_elem_bytes(w.format);
  r.x_stage = mr_->allocate(ucx_memory_type::CUDA, r.x_stage_bytes);
  r.xs_stage_bytes = x_scale_bytes_for(w.format, w.max_m, w.k);
  if (r.xs_stage_bytes) r.xs_stage = mr_->allocate(ucx_memory_type::CUDA, r.xs_stage_bytes);
  r.scratch_bytes = (kSchedWords + size_t(w.max_m) / 128 + 64) * sizeof(uint32_t);
  r.scratch = static_cast<uint32_t*>(mr_->allocate(ucx_memory_type::CUDA, r.scratch_bytes));
  cudaSetDevice(mr_->device());
  if (cudaMemsetAsync(r.scratch, 0, r.scratch_bytes, static_cast<cudaStream_t>(stream_)) != cudaSuccess ||
      cudaStreamSynchronize(static_cast<cudaStream_t>(stream_)) != cudaSuccess)
    throw std::runtime_error("RemoteGemmService: could not clear the kernel's scratch");
  weights_.emplace(weight_id, r);
}

// One launch on the service's stream; the order of launches is the order in which the staging copy of
// X and the scratch words are reused, so no two kernels ever share them.
RemoteGemmService::Done RemoteGemmService::Launch(Resident& r, int32_t m, const void* x, void* y, const void* xs) {
  eux_gemm_desc d;
  std::memset(&d, 0, sizeof(d));
  d.x_src = x;
  d.x_stage = r.x_stage;
  d.w_t = r.w.w_t;
  d.y_dst = y;
  d.x_scale = static_cast<const float*>(xs);
  d.x_scale_stage = static_cast<float*>(r.xs_stage);
  d.w_scale = static_cast<const float*>(r.w.w_scale);
  d.M = m;
  d.N = r.w.n;
  d.K = r.w.k;
  d.fp8 = static_cast<int32_t>(r.w.format);
  d.sched = r.scratch;
  d.panel_flags = r.scratch + kSchedWords;
  d.done_flag = flag_dev_;
  d.done_value = ++seq_;
  d.wait_timeout_ns = 2'000'000'000ull;
  d.status = reinterpret_cast<uint32_t*>(flag_dev_ + 8);
  d.copy_ctas = 0;
  // pairs where M allows; X copied by the spare warps of every CTA; the flag is raised after a failed run too:
  // the call is answered with the kernel's status instead of running into the caller's deadline
  d.flags = EUX_GEMM_FLAG_CTA_PAIRS | EUX_GEMM_FLAG_COPY_WARPS | EUX_GEMM_FLAG_DONE_ALWAYS;
  cudaSetDevice(mr_->device());
  const int rc = eux_gemm_launch(&d, stream_);
  if (rc != 0) {
    --seq_;
    throw std::runtime_error(std::string("remote gemm launch failed: ") + eux_error_string(rc));
  }
  ++launches_;
  return {flag_host_, seq_, reinterpret_cast<const volatile uint32_t*>(flag_host_ + 8)};
}

bool RemoteGemmService::Register() {
  if (registered_) return true;
  auto* self = this;
  auto handler = [self](uint32_t weight_id, int32_t m, uint64_t caller_uid, const vector<uint8_t>& xd, const vector<uint8_t>& yd,
                        const vector<uint8_t>& xsd) {
    ucxx::NvtxRange range("axon.remote_gemm.handler");
    PeerRegionDesc x, y, xs;
    if (!desc_from(xd, &x) || !desc_from(yd, &y)) throw std::invalid_argument("remote gemm: malformed region descriptor");
    std::lock_guard lk(self->mu_);
    auto it = self->weights_.find(weight_id);
    if (it == self->weights_.end()) throw std::invalid_argument("remote gemm: unknown weight " + std::to_string(weight_id));
    Resident& r = it->second;
    const GemmWeight& w = r.w;
    if (m <= 0 || m > w.max_m) throw std::invalid_argument("remote gemm: M is beyond the staging buffer of this weight");
    if (x.length < size_t(m) * size_t(w.k) * x_elem_bytes(w.format) || y.length < size_t(m) * size_t(w.n) * 2)
      throw std::invalid_argument("remote gemm: the caller's regions are smaller than the operands");
    // the caller is this very process only if it presented the uid of a worker that lives here
    const bool same = ucxx::transport::is_live_local_uid(caller_uid);
    auto map = [&](const PeerRegionDesc& d) -> void* {
      void* p = self->mr_->import_region(d, same && d.pid == static_cast<uint32_t>(getpid()));
      if (!p) throw std::runtime_error("remote gemm: the caller's memory cannot be mapped on this GPU");
      return p;
    };
    const void* xp = map(x);
    void* yp = map(y);
    const void* xsp = nullptr;
    if (w.format != GemmFormat::kBf16) {
      if (!desc_from(xsd, &xs) || xs.length < x_scale_bytes_for(w.format, m, w.k))
        throw std::invalid_argument("remote gemm: this weight needs the scales of X");
      xsp = map(xs);
    }
    const Done done = self->Launch(r, m, xp, yp, xsp);
    auto sched = self->worker_.server_context()->get_scheduler();
    // no thread waits for the GPU: the server's loop completes the call when the kernel's flag shows up
    return ex::then(sched.schedule_when_flag(done.flag, done.seq), [done]() -> int32_t {
      ucxx::nvtx_mark("axon.remote_gemm.kernel_done");
      const uint32_t st = *done.status;
      if (st) *const_cast<volatile uint32_t*>(done.status) = 0;
      return static_cast<int32_t>(st);
    });
  };
  ServerMemoryPolicy mp;
  mp.handler_inline = true;  // a few driver calls and one launch: cheaper than waking a pool thread
  registered_ = worker_.RegisterFunction(rpc::function_id_t{utils::FunctionIdFromName(kFunctionName, worker_.name())}, handler, kFunctionName,
                                         std::move(mp), MessageLifecyclePolicy{});
  return registered_;
}

exec::any_sender_of<int32_t> RemoteGemmService::Call(std::string_view worker_name, uint32_t weight_id, int32_t m, const void* x, size_t x_bytes,
                                                     void* y, size_t y_bytes, const void* x_scale, size_t x_scale_bytes) {
  ucxx::NvtxRange range("axon.remote_gemm.call");
  PeerRegionDesc xd, yd, xsd;
  if (!mr_->export_region(x, x_bytes, &xd) || !mr_->export_region(y, y_bytes, &yd))
    throw std::invalid_argument("remote gemm: X and Y must be device memory that can be exported to the callee");
  vector<uint8_t> xs_bytes;
  if (x_scale) {
    if (!mr_->export_region(x_scale, x_scale_bytes, &xsd)) throw std::invalid_argument("remote gemm: the scales of X cannot be exported");
    xs_bytes = desc_bytes(xsd);
  }
  auto* ctx = worker_.client_context();
  const uint64_t uid = ctx ? ctx->worker().address().uid : 0;
  const rpc::function_id_t fid{utils::FunctionIdFromName(kFunctionName, std::string(worker_name))};
  auto call = worker_.InvokeRpc(worker_name, rpc::session_id_t{0}, fid, rpc::utils::workflow_id_t{0}, ClientMemoryPolicy{}, weight_id, m, uid,
                                desc_bytes(xd), desc_bytes(yd), std::move(xs_bytes));
  return exec::any_sender_of<int32_t>(ex::then(std::move(call), [](InvokeResult r) -> int32_t {
    if (!r.header.status.ok()) {
      std::string what = "remote gemm failed";
      for (auto& p : r.header.results)
        if (p.type == rpc::ParamType::STRING)
          if (auto* s = std::get_if<rpc::data::string>(&p.value)) what = std::string(s->data(), s->size());
      throw std::runtime_error(what);
    }
    for (auto& p : r.header.results)
      if (auto* prim = std::get_if<rpc::PrimitiveValue>(&p.value))
        if (auto* v = std::get_if<int32_t>(prim)) return *v;
    return 0;
  }));
}

}  // namespace eux::axon::services
