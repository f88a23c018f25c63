// Remote-GEMM as an Axon function: Y = X * W where W is resident on the callee and X, Y live in the
// caller's device memory. The request is a small active message that carries no payload to pull: it
// names the weight and describes the caller's X and Y regions (PeerRegionDesc, exported through the
// memory resource). The callee's handler maps the regions and launches the tcgen05/TMEM GEMM kernel
// with x_src / y_dst pointing into the caller's memory: the kernel streams X over NVLink panel by
// panel while its tensor cores already work on the panels that have arrived, and stores Y straight
// into the caller's buffer. The handler returns a sender that the server context completes when the
// kernel's completion flag (mapped pinned memory) shows up; the response is a status word.
//
// Three operand formats: bf16; e4m3 with fp32 block scales (1x128 on X, 128x128 on W); MXFP8
// (e4m3 with one UE8M0 scale per 32 elements of K on both operands, scaled by the tensor core).
//
// The reference has no GEMM; what it offers for this workload is "receive the tensor, call a
// library, send the result" (axon/src/axon_worker.cpp:1136-1219 receives into policy memory,
// :522-584 sends the response). This service is the fused replacement of that sequence.
#pragma once

#include <array>
#include <cstdint>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>

#include "eux/axon/axon_worker.hpp"
#include "eux/ucxx/cuda/ucx_cuda_memory_manager.hpp"

namespace eux::axon::services {

enum class GemmFormat : uint8_t {
  kBf16 = 0,      // X, Wt bf16
  kFp8Block = 1,  // e4m3; X scales fp32 [M, K/128], W scales fp32 [N/128, K/128]
  kMxFp8 = 2,     // e4m3; UE8M0 scale chunks (512 bytes per 128 rows x 128 elements of K) on both operands
};

struct GemmWeight {
  const void* w_t = nullptr;      // Wt[N, K] (K-major), resident device memory of the callee
  const void* w_scale = nullptr;  // kFp8Block: fp32 [N/128, K/128]; kMxFp8: scale chunks, K-step major
  int32_t n = 0, k = 0;
  GemmFormat format = GemmFormat::kBf16;
  int32_t max_m = 0;              // rows of X the staging buffer is sized for
};

class RemoteGemmService {
 public:
  static constexpr const char* kFunctionName = "eux.remote_gemm";

  // `mr` must be the worker's memory resource manager (staging buffers and scratch come from its pool).
  RemoteGemmService(AxonWorker& worker, std::shared_ptr<ucxx::UcxCudaMemoryResourceManager> mr);
  ~RemoteGemmService();
  RemoteGemmService(const RemoteGemmService&) = delete;

  // ---- callee ----
  // Make a weight callable under `weight_id` (allocates the staging copy of X and the kernel's scratch).
  void AddWeight(uint32_t weight_id, const GemmWeight& w);
  // Register the Axon function on the worker (once). The function id is the hash of the function and
  // worker names, so callers address it by name.
  bool Register();
  // Kernel launches made by this service's handler so far.
  uint64_t launches() const { return launches_.load(); }
  // (launches issued, completion sequence the kernels have reached, status word): for diagnostics
  std::array<uint64_t, 3> progress() const {
    return {seq_, flag_host_ ? *static_cast<volatile uint64_t*>(flag_host_) : 0, flag_host_ ? static_cast<uint64_t>(*reinterpret_cast<volatile uint32_t*>(flag_host_ + 8)) : 0};
  }

  // ---- caller ----
  // Y[m, N] = X[m, K] * W(weight_id) on worker `worker_name` (an endpoint of this worker's client side).
  // x, y (and x_scale for the fp8 formats) are device buffers of this process; they must stay valid
  // until the returned sender completes. The sender's value is the kernel's status word (0 = ok).
  exec::any_sender_of<int32_t> Call(std::string_view worker_name, uint32_t weight_id, int32_t m, const void* x, size_t x_bytes, void* y,
                                    size_t y_bytes, const void* x_scale = nullptr, size_t x_scale_bytes = 0);

 private:
  struct Resident {
    GemmWeight w;
    void* x_stage = nullptr;
    size_t x_stage_bytes = 0;
    void* xs_stage = nullptr;
    size_t xs_stage_bytes = 0;
    uint32_t* scratch = nullptr;  // [0..3] sched, [64..] panel flags
    size_t scratch_bytes = 0;
  };
  struct Done {
    const volatile uint64_t* flag;
    uint64_t seq;
    const volatile uint32_t* status;
  };
  Done Launch(Resident& r, int32_t m, const void* x, void* y, const void* xs);
  bool EnsureDevice();

  AxonWorker& worker_;
  std::shared_ptr<ucxx::UcxCudaMemoryResourceManager> mr_;
  std::mutex mu_;  // launches (their order on the stream is the order in which the staging buffers are reused)
  std::unordered_map<uint32_t, Resident> weights_;
  void* stream_ = nullptr;
  uint64_t* flag_host_ = nullptr;  // [0]: completion sequence; [8]: status word of the kernels (mapped pinned memory)
  uint64_t* flag_dev_ = nullptr;
  uint64_t seq_ = 0;
  std::atomic<uint64_t> launches_{0};
  bool registered_ = false;
};

}  // namespace eux::axon::services
