// Device-side helpers shared by the data-plane kernels: system-scope
// flag load/store, bounded waits, 16-byte vector access, dtype conversion.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "eux_kernels.h"

namespace eux {

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Spin until *flag >= value. Gives up after timeout_ns (0 = 2 s default) or
// 2^31 polls, whichever comes first; returns false on give-up.
__device__ __forceinline__ bool wait_flag_ge(const uint64_t* flag, uint64_t value, uint64_t timeout_ns) {
  if (ld_acquire_sys(flag) >= value) return true;
  const uint64_t limit = timeout_ns ? timeout_ns : 2000000000ull;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 0; it < 0x7fffffffu; ++it) {
    if (ld_acquire_sys(flag) >= value) return true;
    if ((it & 63u) == 63u) {
      if (globaltimer_ns() - t0 > limit) return false;
      __nanosleep(32);
    }
  }
  return false;
}
__device__ __forceinline__ bool wait_u32_ge_gpu(const uint32_t* flag, uint32_t value, uint64_t timeout_ns) {
  if (ld_acquire_gpu(flag) >= value) return true;
  const uint64_t limit = timeout_ns ? timeout_ns : 2000000000ull;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 0; it < 0x7fffffffu; ++it) {
    if (ld_acquire_gpu(flag) >= value) return true;
    if ((it & 63u) == 63u) {
      if (globaltimer_ns() - t0 > limit) return false;
      __nanosleep(32);
    }
  }
  return false;
}

__device__ __forceinline__ void set_status(uint32_t* status, uint32_t code, uint32_t where) {
  if (status) atomicCAS(status, 0u, code | (where << 8));
}

// 16-byte accesses that bypass L1 (data may have been written by another GPU).
__device__ __forceinline__ uint4 ld_cg_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_u4(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_stream_u4(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

__host__ __device__ __forceinline__ int dtype_size(int dt) {
  switch (dt) {
    case EUX_DT_F32: return 4;
    case EUX_DT_F16: return 2;
    case EUX_DT_BF16: return 2;
    default: return 1;
  }
}

__device__ __forceinline__ float load_as_float(const void* base, uint64_t idx, int dt) {
  switch (dt) {
    case EUX_DT_F32: return reinterpret_cast<const float*>(base)[idx];
    case EUX_DT_F16: return __half2float(reinterpret_cast<const __half*>(base)[idx]);
    case EUX_DT_BF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
    case EUX_DT_F8E4M3: {
      __nv_fp8_e4m3 v;
      v.__x = reinterpret_cast<const uint8_t*>(base)[idx];
      return float(v);
    }
    default: return float(reinterpret_cast<const uint8_t*>(base)[idx]);
  }
}
__device__ __forceinline__ void store_from_float(void* base, uint64_t idx, int dt, float f) {
  switch (dt) {
    case EUX_DT_F32: reinterpret_cast<float*>(base)[idx] = f; break;
    case EUX_DT_F16: reinterpret_cast<__half*>(base)[idx] = __float2half_rn(f); break;
    case EUX_DT_BF16: reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(f); break;
    case EUX_DT_F8E4M3: reinterpret_cast<uint8_t*>(base)[idx] = __nv_fp8_e4m3(f).__x; break;
    default: reinterpret_cast<uint8_t*>(base)[idx] = (uint8_t)f; break;
  }
}
__device__ __forceinline__ float apply_op(float x, int op, float arg) {
  return op == EUX_OP_ADD ? x + arg : (op == EUX_OP_MUL ? x * arg : x);
}

}  // namespace eux
