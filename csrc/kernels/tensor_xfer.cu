// Tensor send/recv data plane (the role UCX's cuda_ipc/cuda_copy transports
// play under ucp_am_send_nbx in the reference, ucx_context/ucx_connection.cpp:353-398,
// and the role of the divide-by-two "handler" kernel in
// ucx_context/ucx_am_context/ucx_am_context_test_cuda_helper.cu:27-78).
//
// One kernel does: (optional bounded acquire-wait on an arrival flag) ->
// strided gather / dense read of the source tensor -> elementwise handler ->
// dtype cast -> dense store into the destination (normally a slot of the
// peer's receive arena, mapped into this process) -> system-scope release of
// a sequence flag. Nothing is staged through the host.
#include "eux_bulk.cuh"
#include "eux_device.cuh"

namespace eux {

constexpr int kXferThreads = 512;

struct XferArgs {
  eux_xfer_desc d;
  uint32_t* counter;
};

template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static __device__ __forceinline__ float to(float v) { return v; }
  static __device__ __forceinline__ float from(float f) { return f; }
};
template <>
struct Elem<__half> {
  static __device__ __forceinline__ float to(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from(float f) { return __float2half_rn(f); }
};
template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from(float f) { return __float2bfloat16_rn(f); }
};
template <>
struct Elem<__nv_fp8_e4m3> {
  static __device__ __forceinline__ float to(__nv_fp8_e4m3 v) { return float(v); }
  static __device__ __forceinline__ __nv_fp8_e4m3 from(float f) { return __nv_fp8_e4m3(f); }
};

template <int BYTES>
struct PackT;
template <>
struct PackT<8> {
  using type = uint2;
};
template <>
struct PackT<16> {
  using type = uint4;
};

// Wait (bounded) for the arrival flag; every thread of the CTA learns the outcome.
__device__ __forceinline__ bool cta_wait_arrival(const eux_xfer_desc& d) {
  if (d.wait_flag == nullptr) return true;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    bool ok = wait_flag_ge(d.wait_flag, d.wait_value, d.wait_timeout_ns);
    if (!ok) set_status(d.status, EUX_ST_TIMEOUT, 1);
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

// All stores of this CTA are done; the last CTA of the grid publishes the flag, and only if no CTA
// of the grid gave up: every CTA runs its own bounded wait, so near the deadline one can time out (and
// skip its share of the copy) while the last one to arrive succeeded. The scratch word counts arrivals
// in its low 31 bits; a CTA that failed sets the top bit before it counts itself.
__device__ __forceinline__ void cta_publish(const eux_xfer_desc& d, uint32_t* counter, bool ok) {
  __syncthreads();
  if (threadIdx.x != 0) return;
  __threadfence_system();
  bool last = true;
  if (gridDim.x > 1) {
    if (!ok) atomicOr(counter, 0x80000000u);
    const uint32_t old = atomicAdd(counter, 1u);
    last = ((old & 0x7fffffffu) == gridDim.x - 1);
    if (old & 0x80000000u) ok = false;
    if (last) {
      *counter = 0;  // leave the scratch word clean for the next launch
      __threadfence();
    }
  }
  if (last && ok && d.flag) st_release_sys(d.flag, d.flag_value);
  if (last && ok && d.flag2) st_release_sys(d.flag2, d.flag2_value);
}

// Dense byte copy. A CTA works on one contiguous block at a time and the blocks are dealt
// round-robin to the CTAs, so that what a CTA has in flight stays inside a few DRAM pages.
// With 32-byte aligned buffers each thread moves two 32-byte vectors per block (measured best
// on B200: 3.31 TB/s each way for a local copy, above cudaMemcpy's 3.26; four or eight 16-byte
// accesses in flight per thread reach 3.17 and 3.01); otherwise four 16-byte vectors.
__device__ __forceinline__ void ld_v8(const void* p, uint32_t (&v)[8]) {
  asm volatile("ld.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "l"(p));
}
__device__ __forceinline__ void st_v8(void* p, const uint32_t (&v)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
               "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

// `cta` of `nctas` CTAs share the copy (the whole grid for one message, a single CTA for one
// descriptor of a batch).
template <bool V32>
__device__ __forceinline__ void copy_bytes_grid(const unsigned char* src, unsigned char* dst, uint64_t nbytes,
                                                uint32_t cta, uint32_t nctas) {
  const uint64_t tid = (uint64_t)cta * blockDim.x + threadIdx.x;
  const uint64_t nthreads = (uint64_t)nctas * blockDim.x;
  uint64_t done = 0;  // bytes handled by the blocked loops
  if (V32) {
    constexpr int U = 2;
    const uint64_t block_bytes = (uint64_t)blockDim.x * U * 32;
    const uint64_t nblocks = nbytes / block_bytes;
    for (uint64_t b = cta; b < nblocks; b += nctas) {
      const uint64_t off = b * block_bytes + (uint64_t)threadIdx.x * 32;
      uint32_t v[U][8];
#pragma unroll
      for (int j = 0; j < U; ++j) ld_v8(src + off + (uint64_t)j * blockDim.x * 32, v[j]);
#pragma unroll
      for (int j = 0; j < U; ++j) st_v8(dst + off + (uint64_t)j * blockDim.x * 32, v[j]);
    }
    done = nblocks * block_bytes;
  } else {
    constexpr int U = 4;
    const uint64_t block_bytes = (uint64_t)blockDim.x * U * 16;
    const uint64_t nblocks = nbytes / block_bytes;
    for (uint64_t b = cta; b < nblocks; b += nctas) {
      const uint64_t off = b * block_bytes + (uint64_t)threadIdx.x * 16;
      uint4 v[U];
#pragma unroll
      for (int j = 0; j < U; ++j) v[j] = ld_cg_u4(src + off + (uint64_t)j * blockDim.x * 16);
#pragma unroll
      for (int j = 0; j < U; ++j) st_u4(dst + off + (uint64_t)j * blockDim.x * 16, v[j]);
    }
    done = nblocks * block_bytes;
  }
  // what is left of the last block: 16-byte vectors, then single bytes
  const uint64_t nvec = (nbytes - done) >> 4;
  for (uint64_t i = tid; i < nvec; i += nthreads) st_u4(dst + done + i * 16, ld_cg_u4(src + done + i * 16));
  for (uint64_t b = done + (nvec << 4) + tid; b < nbytes; b += nthreads) dst[b] = src[b];
}

template <bool V32>
__global__ void __launch_bounds__(kXferThreads) xfer_bytes_kernel(XferArgs a) {
  const eux_xfer_desc& d = a.d;
  bool ok = cta_wait_arrival(d);
  if (ok) {
    const uint64_t nbytes = d.n_elems * (uint64_t)dtype_size(d.src_dtype);
    copy_bytes_grid<V32>(reinterpret_cast<const unsigned char*>(d.src), reinterpret_cast<unsigned char*>(d.dst), nbytes,
                         blockIdx.x, gridDim.x);
  }
  cta_publish(d, a.counter, ok);
}

// Dense byte copy on the bulk-copy engine: two threads per CTA drive a ring of shared-memory
// chunks (loads from the source with completion on an mbarrier, stores to the destination in
// bulk groups). The SMs issue almost no instructions, and the bytes in flight per CTA (the whole
// ring) do not depend on how many threads there are, which is what a source across NVLink needs.
constexpr int kBulkChunk = 16384;
constexpr int kBulkStages = 6;  // 96 KiB of ring per CTA: two CTAs per SM
constexpr int kBulkThreads = 128;
constexpr size_t kBulkSmem = (size_t)kBulkChunk * kBulkStages + 128;

__global__ void __launch_bounds__(kBulkThreads) xfer_bulk_kernel(XferArgs a) {
  extern __shared__ unsigned char xb_raw[];
  __shared__ uint64_t xb_bars[2 * kBulkStages];
  __shared__ int xb_abort;
  const eux_xfer_desc& d = a.d;
  bool ok = cta_wait_arrival(d);
  const uint32_t ring0 = smem_u32(reinterpret_cast<unsigned char*>(((uintptr_t)xb_raw + 127) & ~(uintptr_t)127));
  const uint32_t bar0 = smem_u32(xb_bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kBulkStages + s); };
  if (threadIdx.x == 0) {
    xb_abort = 0;
    for (int s = 0; s < kBulkStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  volatile int* abort = &xb_abort;
  const uint64_t nbytes = d.n_elems * (uint64_t)dtype_size(d.src_dtype);
  const uint64_t body = nbytes & ~(uint64_t)15;
  const uint64_t nchunks = (body + kBulkChunk - 1) / kBulkChunk;
  const unsigned char* src = reinterpret_cast<const unsigned char*>(d.src);
  unsigned char* dst = reinterpret_cast<unsigned char*>(d.dst);
  if (ok && threadIdx.x == 0) {
    uint32_t c = 0;
    for (uint64_t ch = blockIdx.x; ch < nchunks; ch += gridDim.x, ++c) {
      const int st = (int)(c % kBulkStages);
      if (!mbar_wait(empty_bar(st), ((c / kBulkStages) & 1u) ^ 1u, abort, d.wait_timeout_ns)) break;
      const uint64_t off = ch * kBulkChunk;
      const uint32_t n = (uint32_t)min((uint64_t)kBulkChunk, body - off);
      mbar_expect_tx(full_bar(st), n);
      bulk_g2s(ring0 + (uint32_t)st * kBulkChunk, src + off, n, full_bar(st));
    }
    if (*abort) {
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
  } else if (ok && threadIdx.x == 32) {
    uint32_t c = 0, released = 0;
    for (uint64_t ch = blockIdx.x; ch < nchunks; ch += gridDim.x, ++c) {
      const int st = (int)(c % kBulkStages);
      if (!mbar_wait(full_bar(st), (c / kBulkStages) & 1u, abort, d.wait_timeout_ns)) break;
      const uint64_t off = ch * kBulkChunk;
      const uint32_t n = (uint32_t)min((uint64_t)kBulkChunk, body - off);
      bulk_s2g(dst + off, ring0 + (uint32_t)st * kBulkChunk, n);
      bulk_commit();
      bulk_wait_read_1();
      for (; released < c; ++released) mbar_arrive(empty_bar((int)(released % kBulkStages)));
    }
    bulk_wait_all();  // the stores have been performed
    asm volatile("fence.proxy.async;" ::: "memory");
    if (*abort) set_status(d.status, EUX_ST_TIMEOUT, 2);
  } else if (ok && blockIdx.x == 0 && threadIdx.x >= 64 && threadIdx.x < 64 + (nbytes & 15)) {
    const uint64_t b = body + (threadIdx.x - 64);
    dst[b] = src[b];
  }
  __syncthreads();
  cta_publish(d, a.counter, ok && xb_abort == 0);
}

// Dense typed path: 8 elements per step, cast + handler fused.
template <typename S, typename D>
__device__ __forceinline__ void typed_body(const eux_xfer_desc& d) {
  const S* src = reinterpret_cast<const S*>(d.src);
  D* dst = reinterpret_cast<D*>(d.dst);
  const uint64_t n8 = d.n_elems >> 3;
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t nthreads = (uint64_t)gridDim.x * blockDim.x;
  const int op = d.op;
  const float arg = d.op_arg;
  using PS = typename PackT<(8 * sizeof(S) >= 32 ? 16 : 8 * sizeof(S))>::type;
  using PD = typename PackT<(8 * sizeof(D) >= 32 ? 16 : 8 * sizeof(D))>::type;
  constexpr int NS = 8 * sizeof(S) / sizeof(PS);
  constexpr int ND = 8 * sizeof(D) / sizeof(PD);
  for (uint64_t i = tid; i < n8; i += nthreads) {
    alignas(16) S sv[8];
    alignas(16) D dv[8];
#pragma unroll
    for (int k = 0; k < NS; ++k) reinterpret_cast<PS*>(sv)[k] = __ldcg(reinterpret_cast<const PS*>(src + i * 8) + k);
#pragma unroll
    for (int k = 0; k < 8; ++k) dv[k] = Elem<D>::from(apply_op(Elem<S>::to(sv[k]), op, arg));
#pragma unroll
    for (int k = 0; k < ND; ++k) reinterpret_cast<PD*>(dst + i * 8)[k] = reinterpret_cast<PD*>(dv)[k];
  }
  for (uint64_t e = (n8 << 3) + tid; e < d.n_elems; e += nthreads)
    dst[e] = Elem<D>::from(apply_op(Elem<S>::to(src[e]), op, arg));
}

template <typename S, typename D>
__global__ void __launch_bounds__(kXferThreads) xfer_typed_kernel(XferArgs a) {
  const eux_xfer_desc& d = a.d;
  bool ok = cta_wait_arrival(d);
  if (ok) typed_body<S, D>(d);
  cta_publish(d, a.counter, ok);
}

// One tensor-RPC echo step of a rank in a single launch: push the request into the partner's arena and
// publish its flag; as the partner's server, wait for its request, apply the handler and push the response
// back; as client again, wait for the response. Each phase is what xfer_bytes_kernel / xfer_typed_kernel
// do in a launch of their own. The partner runs the same kernel on its GPU at the same time; no CTA waits
// for a CTA of its own grid (a phase's flag is published by whichever CTA finishes it last), and the grid
// is at most one CTA per SM, so every CTA is resident. All tensors dense, 16-byte aligned, of one dtype.
struct RpcStepArgs {
  eux_xfer_desc req, resp, done;
  uint32_t* counter;  // three words
};
template <typename S>
__device__ __forceinline__ void rpc_phase(const eux_xfer_desc& d, uint32_t* counter) {
  bool ok = cta_wait_arrival(d);
  if (ok && d.n_elems) {
    if (d.op == EUX_OP_NONE) {
      const unsigned char* src = reinterpret_cast<const unsigned char*>(d.src);
      unsigned char* dst = reinterpret_cast<unsigned char*>(d.dst);
      const uint64_t nbytes = d.n_elems * (uint64_t)dtype_size(d.src_dtype);
      if (((((uintptr_t)src) | ((uintptr_t)dst)) & 31u) == 0) copy_bytes_grid<true>(src, dst, nbytes, blockIdx.x, gridDim.x);
      else copy_bytes_grid<false>(src, dst, nbytes, blockIdx.x, gridDim.x);
    } else
      typed_body<S, S>(d);
  }
  cta_publish(d, counter, ok);
}
template <typename S>
__global__ void __launch_bounds__(kXferThreads) xfer_rpc_step_kernel(RpcStepArgs a) {
  rpc_phase<S>(a.req, a.counter);
  rpc_phase<S>(a.resp, a.counter + 1);
  if (blockIdx.x == 0) {  // the completion: one CTA watches the response flag
    const bool ok = cta_wait_arrival(a.done);
    (void)ok;
  }
}

// Strided gather (and the catch-all for unaligned bases): one element per step.
__global__ void __launch_bounds__(kXferThreads) xfer_strided_kernel(XferArgs a) {
  const eux_xfer_desc& d = a.d;
  bool ok = cta_wait_arrival(d);
  if (ok) {
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nthreads = (uint64_t)gridDim.x * blockDim.x;
    const bool raw = (d.src_dtype == d.dst_dtype && d.op == EUX_OP_NONE) || d.src_dtype == EUX_DT_BYTES;
    const int esz = dtype_size(d.src_dtype);
    for (uint64_t e = tid; e < d.n_elems; e += nthreads) {
      uint64_t rem = e;
      int64_t off = 0;
      if (d.ndim == 0) {
        off = (int64_t)e;
      } else {
        for (int k = d.ndim - 1; k >= 0; --k) {
          uint64_t q = rem / (uint64_t)d.shape[k];
          off += (int64_t)(rem - q * (uint64_t)d.shape[k]) * d.stride[k];
          rem = q;
        }
      }
      if (raw) {
        const unsigned char* s = reinterpret_cast<const unsigned char*>(d.src) + off * esz;
        unsigned char* t = reinterpret_cast<unsigned char*>(d.dst) + e * esz;
        if (esz == 4) *reinterpret_cast<uint32_t*>(t) = *reinterpret_cast<const uint32_t*>(s);
        else if (esz == 2) *reinterpret_cast<uint16_t*>(t) = *reinterpret_cast<const uint16_t*>(s);
        else *t = *s;
      } else {
        store_from_float(d.dst, e, d.dst_dtype, apply_op(load_as_float(d.src, (uint64_t)off, d.src_dtype), d.op, d.op_arg));
      }
    }
  }
  cta_publish(d, a.counter, ok);
}

// One CTA per descriptor; meant for many small messages per launch.
__global__ void __launch_bounds__(256) xfer_batch_kernel(const eux_xfer_desc* descs, int n) {
  if ((int)blockIdx.x >= n) return;
  __shared__ eux_xfer_desc d;
  {
    const uint32_t* s = reinterpret_cast<const uint32_t*>(descs + blockIdx.x);
    uint32_t* t = reinterpret_cast<uint32_t*>(&d);
    for (int i = threadIdx.x; i < (int)(sizeof(eux_xfer_desc) / 4); i += blockDim.x) t[i] = s[i];
  }
  __syncthreads();
  bool ok = true;
  if (d.wait_flag) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
      bool w = wait_flag_ge(d.wait_flag, d.wait_value, d.wait_timeout_ns);
      if (!w) set_status(d.status, EUX_ST_TIMEOUT, 2);
      s_ok = w;
    }
    __syncthreads();
    ok = s_ok != 0;
  }
  if (ok) {
    const uint64_t esz = (uint64_t)dtype_size(d.src_dtype);
    const bool dense = d.ndim == 0;
    const bool raw = d.src_dtype == d.dst_dtype && d.op == EUX_OP_NONE;
    const bool al16 = ((((uintptr_t)d.src) | ((uintptr_t)d.dst)) & 15u) == 0;
    if (dense && raw && al16) {
      copy_bytes_grid<false>(reinterpret_cast<const unsigned char*>(d.src), reinterpret_cast<unsigned char*>(d.dst),
                             d.n_elems * esz, 0, 1);
    } else if (dense && al16 && d.src_dtype == EUX_DT_F32 && d.dst_dtype == EUX_DT_F32) {
      const float4* s = reinterpret_cast<const float4*>(d.src);
      float4* t = reinterpret_cast<float4*>(d.dst);
      const uint64_t n4 = d.n_elems >> 2;
      for (uint64_t i = threadIdx.x; i < n4; i += blockDim.x) {
        float4 v = __ldcg(s + i);
        v.x = apply_op(v.x, d.op, d.op_arg);
        v.y = apply_op(v.y, d.op, d.op_arg);
        v.z = apply_op(v.z, d.op, d.op_arg);
        v.w = apply_op(v.w, d.op, d.op_arg);
        t[i] = v;
      }
      for (uint64_t e = (n4 << 2) + threadIdx.x; e < d.n_elems; e += blockDim.x)
        reinterpret_cast<float*>(d.dst)[e] = apply_op(reinterpret_cast<const float*>(d.src)[e], d.op, d.op_arg);
    } else {
      for (uint64_t e = threadIdx.x; e < d.n_elems; e += blockDim.x) {
        uint64_t rem = e;
        int64_t off = dense ? (int64_t)e : 0;
        if (!dense)
          for (int k = d.ndim - 1; k >= 0; --k) {
            uint64_t q = rem / (uint64_t)d.shape[k];
            off += (int64_t)(rem - q * (uint64_t)d.shape[k]) * d.stride[k];
            rem = q;
          }
        if (raw) {
          const unsigned char* s = reinterpret_cast<const unsigned char*>(d.src) + off * esz;
          unsigned char* t = reinterpret_cast<unsigned char*>(d.dst) + e * esz;
          for (uint64_t b = 0; b < esz; ++b) t[b] = s[b];
        } else {
          store_from_float(d.dst, e, d.dst_dtype,
                           apply_op(load_as_float(d.src, (uint64_t)off, d.src_dtype), d.op, d.op_arg));
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && ok && d.flag) {
    __threadfence_system();
    st_release_sys(d.flag, d.flag_value);
  }
}

// ---------------------------------------------------------------------------
// Device-driven ping-pong: both GPUs run this kernel at the same time (one
// launch per GPU, never two on the same GPU). The initiator pushes its buffer
// into the peer's buffer and publishes seq; the echo side waits for seq,
// pushes the received bytes back and publishes seq on the initiator.
// initiator == 2 is a single-GPU loopback (no flags, peer_buf is local).
// ---------------------------------------------------------------------------
__device__ __forceinline__ bool grid_barrier(uint32_t* bar, uint32_t& gen, uint64_t timeout_ns) {
  __syncthreads();
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    __threadfence_system();
    gen += 1;
    atomicAdd(bar, 1u);
    s_ok = wait_u32_ge_gpu(bar, gen * gridDim.x, timeout_ns);
  }
  __syncthreads();
  return s_ok != 0;
}

__global__ void __launch_bounds__(kXferThreads) pingpong_kernel(eux_pingpong_desc d) {
  uint32_t gen = 0;
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t nthreads = (uint64_t)gridDim.x * blockDim.x;
  __shared__ int s_ok;
  bool alive = true;
  for (int it = 0; it < d.iters && alive; ++it) {
    const uint64_t seq = d.base_seq + 1 + (uint64_t)it;
    if (d.ts_out && tid == 0) d.ts_out[it] = globaltimer_ns();
    if (d.initiator == 0) {
      if (threadIdx.x == 0) s_ok = wait_flag_ge(d.local_flag, seq, d.wait_timeout_ns);
      __syncthreads();
      if (!s_ok) { alive = false; break; }
    }
    copy_bytes_grid<false>(reinterpret_cast<const unsigned char*>(d.local_buf), reinterpret_cast<unsigned char*>(d.peer_buf),
                           d.nbytes, blockIdx.x, gridDim.x);
    if (!grid_barrier(d.grid_bar, gen, d.wait_timeout_ns)) { alive = false; break; }
    if (d.initiator == 2) {
      copy_bytes_grid<false>(reinterpret_cast<const unsigned char*>(d.peer_buf), reinterpret_cast<unsigned char*>(d.local_buf),
                             d.nbytes, blockIdx.x, gridDim.x);
      if (!grid_barrier(d.grid_bar, gen, d.wait_timeout_ns)) { alive = false; break; }
      continue;
    }
    if (tid == 0) st_release_sys(d.peer_flag, seq);
    if (d.initiator == 1) {
      if (threadIdx.x == 0) s_ok = wait_flag_ge(d.local_flag, seq, d.wait_timeout_ns);
      __syncthreads();
      if (!s_ok) { alive = false; break; }
    }
  }
  if (!alive && threadIdx.x == 0) set_status(d.status, EUX_ST_TIMEOUT, 3);
  if (d.ts_out && tid == 0) d.ts_out[d.iters] = globaltimer_ns();
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t old = atomicAdd(d.grid_bar + 1, 1u);
    if (old == gridDim.x - 1) {
      d.grid_bar[0] = 0;
      d.grid_bar[1] = 0;
      __threadfence();
    }
  }
}

static int num_sms() {
  static int sms[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    sms[dev] = n;
  }
  return sms[dev];
}

template <typename S>
static int launch_typed(const XferArgs& a, int grid, cudaStream_t st) {
  switch (a.d.dst_dtype) {
    case EUX_DT_F32: xfer_typed_kernel<S, float><<<grid, kXferThreads, 0, st>>>(a); break;
    case EUX_DT_F16: xfer_typed_kernel<S, __half><<<grid, kXferThreads, 0, st>>>(a); break;
    case EUX_DT_BF16: xfer_typed_kernel<S, __nv_bfloat16><<<grid, kXferThreads, 0, st>>>(a); break;
    case EUX_DT_F8E4M3: xfer_typed_kernel<S, __nv_fp8_e4m3><<<grid, kXferThreads, 0, st>>>(a); break;
    default: return EUX_ERR_BAD_ARG;
  }
  return 0;
}

}  // namespace eux

using namespace eux;

extern "C" int eux_xfer_launch(const eux_xfer_desc* d, uint32_t* scratch_counter, int max_ctas, void* stream) {
  if (!d || !d->src || !d->dst || d->ndim < 0 || d->ndim > EUX_MAX_DIMS) return EUX_ERR_BAD_ARG;
  if (d->src_dtype == EUX_DT_BYTES && (d->dst_dtype != EUX_DT_BYTES || d->op != EUX_OP_NONE)) return EUX_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  XferArgs a{*d, scratch_counter};
  const int sms = num_sms();
  const bool ctas_given = max_ctas > 0;
  if (!ctas_given) max_ctas = 2 * sms;
  const uint64_t src_bytes = d->n_elems * (uint64_t)dtype_size(d->src_dtype);
  const bool raw = d->src_dtype == d->dst_dtype && d->op == EUX_OP_NONE;
  const uintptr_t al = ((uintptr_t)d->src) | ((uintptr_t)d->dst);
  int grid;
  if (d->ndim == 0 && raw && (al & 15u) == 0) {
    // 64 B per thread per step, one CTA per SM; small messages stay on one CTA (no counter traffic)
    if (!ctas_given) max_ctas = sms;
    uint64_t want = (src_bytes + (uint64_t)kXferThreads * 64 - 1) / ((uint64_t)kXferThreads * 64);
    grid = (int)(want < 1 ? 1 : (want > (uint64_t)max_ctas ? max_ctas : want));
    if (grid > 1 && !scratch_counter) return EUX_ERR_BAD_ARG;
    if ((al & 31u) == 0) xfer_bytes_kernel<true><<<grid, kXferThreads, 0, st>>>(a);
    else xfer_bytes_kernel<false><<<grid, kXferThreads, 0, st>>>(a);
  } else if (d->ndim == 0 && d->src_dtype != EUX_DT_BYTES && (al & 15u) == 0) {
    uint64_t want = (d->n_elems / 8 + kXferThreads - 1) / kXferThreads;
    grid = (int)(want < 1 ? 1 : (want > (uint64_t)max_ctas ? max_ctas : want));
    if (grid > 1 && !scratch_counter) return EUX_ERR_BAD_ARG;
    int rc = 0;
    switch (d->src_dtype) {
      case EUX_DT_F32: rc = launch_typed<float>(a, grid, st); break;
      case EUX_DT_F16: rc = launch_typed<__half>(a, grid, st); break;
      case EUX_DT_BF16: rc = launch_typed<__nv_bfloat16>(a, grid, st); break;
      case EUX_DT_F8E4M3: rc = launch_typed<__nv_fp8_e4m3>(a, grid, st); break;
      default: rc = EUX_ERR_BAD_ARG;
    }
    if (rc) return rc;
  } else {
    uint64_t want = (d->n_elems + kXferThreads * 4 - 1) / (kXferThreads * 4);
    grid = (int)(want < 1 ? 1 : (want > (uint64_t)max_ctas ? max_ctas : want));
    if (grid > 1 && !scratch_counter) return EUX_ERR_BAD_ARG;
    xfer_strided_kernel<<<grid, kXferThreads, 0, st>>>(a);
  }
  return (int)cudaGetLastError();
}

extern "C" int eux_xfer_rpc_step_launch(const eux_xfer_desc* req, const eux_xfer_desc* resp, const eux_xfer_desc* done,
                                        uint32_t* scratch3, int max_ctas, void* stream) {
  if (!req || !resp || !done || !scratch3 || !req->src || !req->dst || !resp->src || !resp->dst) return EUX_ERR_BAD_ARG;
  const eux_xfer_desc* ds[2] = {req, resp};
  for (const eux_xfer_desc* d : ds) {
    if (d->ndim != 0 || d->src_dtype != d->dst_dtype) return EUX_ERR_BAD_ARG;
    if ((((uintptr_t)d->src) | ((uintptr_t)d->dst)) & 15u) return EUX_ERR_BAD_ARG;
    if (d->op != EUX_OP_NONE && d->src_dtype == EUX_DT_BYTES) return EUX_ERR_BAD_ARG;
  }
  if (req->src_dtype != resp->src_dtype) return EUX_ERR_BAD_ARG;
  const int sms = num_sms();
  if (max_ctas <= 0 || max_ctas > sms) max_ctas = sms;  // every CTA resident: see the kernel
  const uint64_t bytes = req->n_elems * (uint64_t)dtype_size(req->src_dtype);
  const uint64_t want = (bytes + (uint64_t)kXferThreads * 64 - 1) / ((uint64_t)kXferThreads * 64);
  const int grid = (int)(want < 1 ? 1 : (want > (uint64_t)max_ctas ? max_ctas : want));
  RpcStepArgs a{*req, *resp, *done, scratch3};
  a.done.n_elems = 0;
  cudaStream_t st = (cudaStream_t)stream;
  switch (req->src_dtype) {
    case EUX_DT_F32: xfer_rpc_step_kernel<float><<<grid, kXferThreads, 0, st>>>(a); break;
    case EUX_DT_F16: xfer_rpc_step_kernel<__half><<<grid, kXferThreads, 0, st>>>(a); break;
    case EUX_DT_BF16: xfer_rpc_step_kernel<__nv_bfloat16><<<grid, kXferThreads, 0, st>>>(a); break;
    case EUX_DT_F8E4M3: xfer_rpc_step_kernel<__nv_fp8_e4m3><<<grid, kXferThreads, 0, st>>>(a); break;
    case EUX_DT_BYTES: xfer_rpc_step_kernel<float><<<grid, kXferThreads, 0, st>>>(a); break;  // no handler: bytes only
    default: return EUX_ERR_BAD_ARG;
  }
  return (int)cudaGetLastError();
}

extern "C" int eux_xfer_bulk_launch(const eux_xfer_desc* d, uint32_t* scratch_counter, int max_ctas, void* stream) {
  if (!d || !d->src || !d->dst || d->ndim != 0) return EUX_ERR_BAD_ARG;
  if (d->src_dtype != d->dst_dtype || d->op != EUX_OP_NONE) return EUX_ERR_BAD_ARG;
  if ((((uintptr_t)d->src) | ((uintptr_t)d->dst)) & 15u) return EUX_ERR_BAD_ARG;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return EUX_ERR_BAD_ARG;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(xfer_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBulkSmem);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev] = true;
  }
  const uint64_t bytes = d->n_elems * (uint64_t)dtype_size(d->src_dtype);
  if (max_ctas <= 0) max_ctas = 2 * num_sms();
  uint64_t want = (bytes + kBulkChunk - 1) / kBulkChunk;
  int grid = (int)(want < 1 ? 1 : (want > (uint64_t)max_ctas ? max_ctas : want));
  if (grid > 1 && !scratch_counter) return EUX_ERR_BAD_ARG;
  XferArgs a{*d, scratch_counter};
  xfer_bulk_kernel<<<grid, kBulkThreads, kBulkSmem, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

// One CTA per item, the items in the launch parameters.
struct PullBatchArgs {
  eux_pull_item it[EUX_PULL_BATCH_MAX];
};
// 1024 threads: a 64 KiB message is in flight at once (four 16-byte vectors per thread), so its CTA needs one
// memory round trip for it and not four; the launch is as long as its largest item.
constexpr int kPullBatchThreads = 1024;
__global__ void __launch_bounds__(kPullBatchThreads) xfer_pull_batch_kernel(const __grid_constant__ PullBatchArgs a) {
  const eux_pull_item& d = a.it[blockIdx.x];
  const unsigned char* src = reinterpret_cast<const unsigned char*>(d.src);
  unsigned char* dst = reinterpret_cast<unsigned char*>(d.dst);
  if (((((uintptr_t)src) | ((uintptr_t)dst)) & 15u) == 0) {
    copy_bytes_grid<false>(src, dst, d.nbytes, 0, 1);
  } else {
    for (uint64_t b = threadIdx.x; b < d.nbytes; b += blockDim.x) dst[b] = src[b];
  }
  __syncthreads();
  if (threadIdx.x == 0 && (d.flag || d.flag2)) {
    __threadfence_system();
    if (d.flag) st_release_sys(d.flag, d.flag_value);
    if (d.flag2) st_release_sys(d.flag2, d.flag2_value);
  }
}

extern "C" int eux_xfer_pull_batch_launch(const eux_pull_item* items, int n, void* stream) {
  if (n <= 0) return 0;
  if (!items || n > EUX_PULL_BATCH_MAX) return EUX_ERR_BAD_ARG;
  PullBatchArgs a;
  for (int i = 0; i < n; ++i) {
    if (!items[i].src || !items[i].dst) return EUX_ERR_BAD_ARG;
    a.it[i] = items[i];
  }
  for (int i = n; i < EUX_PULL_BATCH_MAX; ++i) a.it[i] = eux_pull_item{};
  xfer_pull_batch_kernel<<<n, kPullBatchThreads, 0, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

extern "C" int eux_xfer_batch_launch(const eux_xfer_desc* descs_dev, int n, void* stream) {
  if (n <= 0) return 0;
  if (!descs_dev) return EUX_ERR_BAD_ARG;
  xfer_batch_kernel<<<n, 256, 0, (cudaStream_t)stream>>>(descs_dev, n);
  return (int)cudaGetLastError();
}

extern "C" int eux_pingpong_launch(const eux_pingpong_desc* d, int ctas, void* stream) {
  if (!d || !d->local_buf || !d->peer_buf || !d->grid_bar || (d->nbytes & 15u)) return EUX_ERR_BAD_ARG;
  if (d->initiator != 2 && (!d->local_flag || !d->peer_flag)) return EUX_ERR_BAD_ARG;
  const int sms = num_sms();
  if (ctas <= 0 || ctas > sms) ctas = sms;  // every CTA must be resident: they wait on one another
  uint64_t want = (d->nbytes + (uint64_t)kXferThreads * 64 - 1) / ((uint64_t)kXferThreads * 64);
  if ((uint64_t)ctas > want) ctas = (int)(want < 1 ? 1 : want);
  eux_pingpong_desc dd = *d;
  void* args[] = {&dd};
  cudaError_t e = cudaLaunchCooperativeKernel((const void*)pingpong_kernel, dim3(ctas), dim3(kXferThreads), args, 0,
                                              (cudaStream_t)stream);
  return (int)e;
}

extern "C" int eux_ipc_export(void* dev_ptr, unsigned char handle_out[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, dev_ptr);
  if (e == cudaSuccess) memcpy(handle_out, &h, 64);
  return (int)e;
}
extern "C" int eux_ipc_open(const unsigned char handle[64], void** dev_ptr_out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  return (int)cudaIpcOpenMemHandle(dev_ptr_out, h, cudaIpcMemLazyEnablePeerAccess);
}
extern "C" int eux_ipc_close(void* dev_ptr) { return (int)cudaIpcCloseMemHandle(dev_ptr); }
extern "C" int eux_memcpy_peer_async(void* dst, int dst_device, const void* src, int src_device, size_t bytes, void* stream) {
  return (int)cudaMemcpyPeerAsync(dst, dst_device, src, src_device, bytes, (cudaStream_t)stream);
}
extern "C" int eux_enable_peer_access(int this_dev, int peer_dev) {
  int can = 0;
  cudaError_t e = cudaDeviceCanAccessPeer(&can, this_dev, peer_dev);
  if (e != cudaSuccess) return (int)e;
  if (!can) return EUX_ERR_UNSUPPORTED;
  int cur = 0;
  cudaGetDevice(&cur);
  cudaSetDevice(this_dev);
  e = cudaDeviceEnablePeerAccess(peer_dev, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    e = cudaSuccess;
  }
  cudaSetDevice(cur);
  return (int)e;
}
extern "C" int eux_device_malloc(void** p, size_t bytes) { return (int)cudaMalloc(p, bytes); }
extern "C" int eux_device_free(void* p) { return (int)cudaFree(p); }
extern "C" int eux_host_alloc_mapped(void** host_ptr, void** dev_ptr, size_t bytes) {
  cudaError_t e = cudaHostAlloc(host_ptr, bytes, cudaHostAllocMapped | cudaHostAllocPortable);
  if (e != cudaSuccess) return (int)e;
  memset(*host_ptr, 0, bytes);
  return (int)cudaHostGetDevicePointer(dev_ptr, *host_ptr, 0);
}
extern "C" int eux_host_free(void* host_ptr) { return (int)cudaFreeHost(host_ptr); }
extern "C" const char* eux_error_string(int err) {
  switch (err) {
    case EUX_ERR_BAD_ARG: return "eux: bad argument";
    case EUX_ERR_TOO_LARGE: return "eux: size beyond the supported maximum";
    case EUX_ERR_UNSUPPORTED: return "eux: unsupported on this device";
    default: return cudaGetErrorString((cudaError_t)err);
  }
}


// ---------------------------------------------------------------------------
// Loading every kernel of this file up front. With lazy module loading (the default of the driver) the
// first launch of a kernel loads it, and loading may have to wait for kernels that are running on the
// device. A kernel of some other library that spins until a peer does something (a collective's barrier,
// say) while that peer waits for the reply to a call whose handler launches one of these kernels for the
// first time is then a deadlock. Everything that launches on behalf of a peer loads its kernels first.
// ---------------------------------------------------------------------------
namespace {
template <class K>
int preload_one(K kernel) {
  cudaFuncAttributes attr;
  return (int)cudaFuncGetAttributes(&attr, reinterpret_cast<const void*>(kernel));
}
template <typename S>
int preload_typed() {
  int rc = preload_one(xfer_typed_kernel<S, float>);
  if (!rc) rc = preload_one(xfer_typed_kernel<S, __half>);
  if (!rc) rc = preload_one(xfer_typed_kernel<S, __nv_bfloat16>);
  if (!rc) rc = preload_one(xfer_typed_kernel<S, __nv_fp8_e4m3>);
  if (!rc) rc = preload_one(xfer_rpc_step_kernel<S>);
  return rc;
}
}  // namespace

extern "C" int eux_xfer_preload(void) {
  int rc = preload_one(xfer_bytes_kernel<true>);
  if (!rc) rc = preload_one(xfer_bytes_kernel<false>);
  if (!rc) rc = preload_one(xfer_bulk_kernel);
  if (!rc) rc = preload_one(xfer_strided_kernel);
  if (!rc) rc = preload_one(xfer_batch_kernel);
  if (!rc) rc = preload_one(pingpong_kernel);
  if (!rc) rc = preload_one(xfer_pull_batch_kernel);
  if (!rc) rc = preload_typed<float>();
  if (!rc) rc = preload_typed<__half>();
  if (!rc) rc = preload_typed<__nv_bfloat16>();
  if (!rc) rc = preload_typed<__nv_fp8_e4m3>();
  return rc;
}
