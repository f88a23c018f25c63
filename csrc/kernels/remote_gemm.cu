// Remote-GEMM RPC kernel: Y[M,N] = X[M,K] * W[K,N] with the activation X living
// in the caller's (peer) memory and the result written straight back into the
// caller's memory. The reference has no GEMM; this is the callee side of an RPC
// whose handler is a matrix product, fused with the transfer of its argument.
//
// One persistent launch, one CTA per SM, three kinds of CTA / warp:
//   * copy CTAs (blockIdx < copy_ctas): stream 128-row panels of X from the
//     caller's memory into a local staging buffer with bulk asynchronous copies
//     through shared memory and publish a per-panel arrival count;
//   * GEMM CTAs: warp 0 = TMA producer (waits for the panel, then loads A and B
//     tiles with plain per-CTA cp.async.bulk.tensor loads, 128B swizzle), warp 1 =
//     tcgen05.mma issuer (accumulators in TMEM, two 256-column buffers),
//     warps 4..7 = epilogue (tcgen05.ld -> bf16 -> 16-byte stores into Y,
//     which may be peer memory).
// W is resident in K-major form Wt[N,K] so both operands are K-major.
//
// Every wait is bounded: when one runs out the CTA raises an abort flag, stops
// issuing work, lets its copies land, frees its TMEM and returns with
// EUX_ST_TIMEOUT in the status word.
#include <cuda.h>

#include <cstdlib>

#include "eux_bulk.cuh"
#include "eux_device.cuh"

namespace eux {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BKB = 128;  // bytes of K per stage row = one 128B swizzle atom
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BKB;   // 16 KiB
constexpr int B_STAGE_BYTES = BN * BKB;   // 32 KiB
constexpr int GEMM_THREADS = 256;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 8;
constexpr size_t GEMM_SMEM = (size_t)STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 2 * 16384 /* output slabs */ + 1024 + 256;

struct GemmParams {
  const unsigned char* x_src;
  unsigned char* x_stage;
  unsigned char* y;
  int M, N, K;
  int elem_bytes;
  uint32_t* panel_flags;
  uint32_t* sched;
  uint64_t* done_flag;
  uint64_t done_value;
  uint64_t timeout_ns;
  uint32_t* status;
  int copy_ctas;
  int head_blocks;  // height of the first tile group in row blocks (0: like the others)
  int copy_warps;   // warps (two per CTA) that copy X beside the GEMM's own warps; 0 when copy CTAs do it
  uint32_t panel_target;  // count at which a panel of X is complete (0: X is local, nothing to wait for)
  int done_always;        // publish the done flag after a failed run too (the status word says which it was)
  // block-scaled fp8 only
  const float* x_scale_src;   // [M, K/128], caller's (may be peer)
  float* x_scale_stage;       // local copy used by the epilogue (== x_scale_src when X is local)
  const float* w_scale;       // [N/128, K/128], local
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// K-major, 128B-swizzled operand tile: rows are 128 B apart, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);
  d |= (uint64_t)(1024u >> 4) << 32;  // stride byte offset
  d |= (uint64_t)1 << 46;             // descriptor version
  d |= (uint64_t)2 << 61;             // SWIZZLE_128B
  return d;
}

template <bool FP8>
__device__ __forceinline__ void umma(uint32_t tmem_c, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if (FP8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_c),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_c),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Tiles in groups of GROUP_M row blocks (row block fastest inside a group) so that one wave of CTAs
// shares few panels of X and few of W in L2. While X is still arriving from the caller (`head` > 0) the
// first groups are shorter, head, head and 2 * head blocks tall: measured on 8192^3 over NVLink, the
// copy delivers a 256-row block every 8 us at first and every 12 us once the tensor cores are busy, a
// wave of tiles takes 53 us, and with full-height groups the second and third waves wait for rows that
// are still on their way.
__device__ __forceinline__ void tile_coords(int tile, int m_blocks, int n_blocks, int head, int& mb, int& nb) {
  int base = 0;
  if (head > 0) {
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      const int h = i < 2 ? head : 2 * head;
      if (h >= m_blocks - base) break;
      if (tile < h * n_blocks) {
        mb = base + tile % h;
        nb = tile / h;
        return;
      }
      tile -= h * n_blocks;
      base += h;
    }
    m_blocks -= base;
  }
  const int per_group = GROUP_M * n_blocks;
  const int g = tile / per_group, r = tile - g * per_group;
  const int rows = min(GROUP_M, m_blocks - g * GROUP_M);
  mb = base + g * GROUP_M + r % rows;
  nb = r / rows;
}

// instruction descriptor: D=f32, A/B = bf16 (or e4m3), both K-major, M=128, N=BN_
template <bool FP8, int BN_>
__device__ __forceinline__ constexpr uint32_t make_idesc() {
  return (1u << 4) | ((FP8 ? 0u : 1u) << 7) | ((FP8 ? 0u : 1u) << 10) | ((uint32_t)(BN_ >> 3) << 17) |
         ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src), "r"(x),
               "r"(y)
               : "memory");
}
__device__ __forceinline__ void epi_bar_sync(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }
// Two fp32 multiply-adds in one instruction: (a0, a1) += (x0, x1) * s
__device__ __forceinline__ void ffma2(float& a0, float& a1, float x0, float x1, float s) {
  asm("{\n\t.reg .b64 va, vx, vs;\n\t"
      "mov.b64 va, {%0, %1};\n\tmov.b64 vx, {%2, %3};\n\tmov.b64 vs, {%4, %4};\n\t"
      "fma.rn.f32x2 va, vx, vs, va;\n\t"
      "mov.b64 {%0, %1}, va;\n\t}"
      : "+f"(a0), "+f"(a1)
      : "f"(x0), "f"(x1), "f"(s));
}

// OR of `flag` over the 128 threads of a named barrier: the epilogue warps leave their loop together
__device__ __forceinline__ bool epi_vote_any(int id, bool flag) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %2, 0;\n\t"
      "bar.red.or.pred q, %1, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(out)
      : "r"(id), "r"((uint32_t)flag)
      : "memory");
  return out != 0;
}
__device__ __forceinline__ void st_shared_u4(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Tiles are handed out by a global counter (so CTAs that first copied X join the GEMM when
// they are done, and no CTA idles at the tail). The producer warp draws the next tile and
// passes its index to the MMA and epilogue warps through a ring in shared memory; the roles
// are never more than four tiles apart, the ring has eight slots.
constexpr int TILE_RING = 8;

// Output staging for the epilogue: slabs of 128 rows x 64 bf16 columns (128 B per row) in the
// 128B-swizzled layout that the tensor map of Y expects; a slab leaves as one TMA store, so Y
// (which may be the caller's memory across NVLink) is written in full 128-byte lines.
constexpr int EPI_SLAB_BYTES = BM * 128;
constexpr int EPI_SLABS = 2;

constexpr int CP_CHUNK = 16384;   // bytes per bulk copy
constexpr int CP_STAGES = 12;     // 192 KiB of shared memory in flight per copy CTA

// Copy CTAs: all of them work on one panel at a time, in order, so the first
// panel is complete after 1/copy_ctas of its transfer time. The bytes move as
// bulk asynchronous copies through a ring of shared-memory chunks: one thread
// issues the loads from the caller's (peer) memory, another one the stores into
// the local staging buffer. A load over NVLink takes microseconds to come back,
// so what matters is the number of bytes in flight: 12 x 16 KiB per CTA, which
// register-held loads of a whole CTA cannot reach.
__device__ bool copy_role_n(const GemmParams& p, const int nthreads, unsigned char* smem_raw_base) {
  __shared__ uint64_t cp_bars[2 * CP_STAGES];
  __shared__ int cp_abort;
  const size_t row_bytes = (size_t)p.K * p.elem_bytes;
  const size_t panel_bytes = (size_t)BM * row_bytes;
  const int panels = p.M / BM;
  if (p.x_scale_src && p.x_scale_stage && p.x_scale_src != p.x_scale_stage) {
    // the row scales travel first: each CTA copies its slice before it reports any panel
    const size_t n = (size_t)p.M * (p.K / 128);
    for (size_t i = (size_t)blockIdx.x * nthreads + threadIdx.x; i < n; i += (size_t)p.copy_ctas * nthreads)
      p.x_scale_stage[i] = __ldcg(p.x_scale_src + i);
    __threadfence();
  }
  unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw_base + 127) & ~(uintptr_t)127);
  const uint32_t ring0 = smem_u32(ring);
  const uint32_t bar0 = smem_u32(cp_bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (CP_STAGES + s); };
  if (threadIdx.x == 0) {
    cp_abort = 0;
    for (int s = 0; s < CP_STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  volatile int* abort = &cp_abort;
  // this CTA's slice of every panel, in 16-byte units
  const size_t panel_vec = panel_bytes / 16;
  const size_t per_cta = (panel_vec + p.copy_ctas - 1) / p.copy_ctas;
  const size_t lo = min(panel_vec, (size_t)blockIdx.x * per_cta) * 16;
  const size_t hi = min(panel_vec, (size_t)blockIdx.x * per_cta + per_cta) * 16;

  if (threadIdx.x == 0) {
    // ---- loads from the caller's memory ----
    uint32_t c = 0;
    for (int pn = 0; pn < panels && !*abort; ++pn) {
      const unsigned char* src = p.x_src + (size_t)pn * panel_bytes;
      for (size_t off = lo; off < hi; off += CP_CHUNK, ++c) {
        const int st = (int)(c % CP_STAGES);
        const uint32_t ph = (c / CP_STAGES) & 1u;
        if (!mbar_wait(empty_bar(st), ph ^ 1u, abort, p.timeout_ns)) break;
        const uint32_t n = (uint32_t)min((size_t)CP_CHUNK, hi - off);
        mbar_expect_tx(full_bar(st), n);
        bulk_g2s(ring0 + (uint32_t)st * CP_CHUNK, src + off, n, full_bar(st));
      }
    }
    if (*abort) {  // loads that were issued still write shared memory: give them time to land
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
  } else if (threadIdx.x == 32) {
    // ---- stores into the local staging buffer, and the per-panel report ----
    uint32_t c = 0, released = 0;
    for (int pn = 0; pn < panels && !*abort; ++pn) {
      unsigned char* dst = p.x_stage + (size_t)pn * panel_bytes;
      for (size_t off = lo; off < hi; off += CP_CHUNK, ++c) {
        const int st = (int)(c % CP_STAGES);
        const uint32_t ph = (c / CP_STAGES) & 1u;
        if (!mbar_wait(full_bar(st), ph, abort, p.timeout_ns)) break;
        const uint32_t n = (uint32_t)min((size_t)CP_CHUNK, hi - off);
        bulk_s2g(dst + off, ring0 + (uint32_t)st * CP_CHUNK, n);
        bulk_commit();
        bulk_wait_read_1();  // every store but the newest has finished reading its chunk
        for (; released < c; ++released) mbar_arrive(empty_bar((int)(released % CP_STAGES)));
      }
      if (*abort) break;
      bulk_wait_all();  // this panel's slice is in the staging buffer
      for (; released < c; ++released) mbar_arrive(empty_bar((int)(released % CP_STAGES)));
      asm volatile("fence.proxy.async;" ::: "memory");
      __threadfence();
      red_release_gpu_add(p.panel_flags + pn, 1u);
    }
    bulk_wait_all();
    if (*abort) {
      if (p.status) set_status(p.status, EUX_ST_TIMEOUT, 9);
      atomicExch(p.sched + 1, 1u);
    }
  }
  __syncthreads();
  return cp_abort == 0;
}

// Two otherwise idle warps of every CTA copy X while the CTA's other warps compute: the transfer is spread
// over all SMs' load/store units (a few dedicated CTAs moving it with bulk copies reach about half the link
// rate), and no CTA is lost to the GEMM. X is cut into units of 8 KiB that the copy warps draw from a counter,
// in address order, so the panels complete in the order in which the tiles need them; every unit counts once
// on its panel, and a panel is complete at its number of units.
__device__ __forceinline__ void ld_v8_b32(const void* ptr, uint32_t (&v)[8]) {
  asm volatile("ld.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "l"(ptr));
}
__device__ __forceinline__ void st_v8_b32(void* ptr, const uint32_t (&v)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(ptr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
               "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}
__device__ __forceinline__ void copy_warp_role(const GemmParams& p, uint32_t warp_id, int lane) {
  constexpr int U = 8;  // 1 KiB pieces per unit of work: 8 KiB in flight per warp
  const int panels = p.M / BM;
  const uint32_t units_per_panel = (uint32_t)(((size_t)BM * p.K * p.elem_bytes) >> 13);
  // The scales of a panel's rows (fp32 per 1x128, or MX chunks: K * 4 bytes per 128 rows in either format,
  // contiguous) travel as extra units in front of the panel's data units. Nothing here depends on how many
  // CTAs of the grid are running: whichever copy warps are resident draw the units in order, so a grid that
  // shares the device with some other kernel (and does not get every SM) still completes every panel.
  const bool scales = p.x_scale_src && p.x_scale_stage && p.x_scale_src != p.x_scale_stage;
  const size_t scale_panel_bytes = scales ? (size_t)p.K * 4 : 0;
  const uint32_t scale_units = (uint32_t)((scale_panel_bytes + 8191) >> 13);
  const uint32_t per_panel = units_per_panel + scale_units;
  const uint32_t total = (uint32_t)panels * per_panel;
  const unsigned char* src = p.x_src + (size_t)lane * 32;
  unsigned char* dst = p.x_stage + (size_t)lane * 32;
  // Units of 8 KiB, in address order, are drawn from a counter: a warp that falls behind (its SM is busy with
  // an epilogue, its loads queue behind the tile loads) holds up one unit, not a share of every panel. A unit
  // is counted on its panel one unit late: the fence that makes its stores visible then runs while the next
  // unit's loads are in flight.
  auto draw = [&]() -> uint32_t {
    uint32_t u = 0;
    if (lane == 0) u = atomicAdd(p.sched + 3, 1u);
    return __shfl_sync(0xffffffffu, u, 0);
  };
  auto count = [&](int panel) {
    __syncwarp();
    if (lane == 0) {
      __threadfence();
      red_release_gpu_add(p.panel_flags + panel, 1u);
    }
  };
  int pending = -1;  // panel of the unit whose stores have been issued but not counted
  uint32_t u = draw();
  while (u < total) {
    const uint32_t panel = u / per_panel, w = u % per_panel;
    if (w < scale_units) {
      // a slice of this panel's scales: few and small, copied and counted at once
      const size_t begin = (size_t)panel * scale_panel_bytes + ((size_t)w << 13);
      const size_t end = min((size_t)panel * scale_panel_bytes + scale_panel_bytes, begin + 8192);
      const unsigned char* ss = reinterpret_cast<const unsigned char*>(p.x_scale_src);
      unsigned char* sd = reinterpret_cast<unsigned char*>(p.x_scale_stage);
      for (size_t i = begin + (size_t)lane * 16; i < end; i += 512)
        *reinterpret_cast<uint4*>(sd + i) = __ldcg(reinterpret_cast<const uint4*>(ss + i));
      const uint32_t next = draw();
      count((int)panel);
      u = next;
      continue;
    }
    uint32_t v[U][8];
    const size_t off = ((size_t)panel * units_per_panel + (w - scale_units)) << 13;
#pragma unroll
    for (int j = 0; j < U; ++j) ld_v8_b32(src + off + ((size_t)j << 10), v[j]);
    const uint32_t next = draw();
    if (pending >= 0) count(pending);
#pragma unroll
    for (int j = 0; j < U; ++j) st_v8_b32(dst + off + ((size_t)j << 10), v[j]);
    pending = (int)panel;
    u = next;
  }
  if (pending >= 0) count(pending);
}

__device__ __forceinline__ void finish_cta(const GemmParams& p, bool ok) {
  __syncthreads();
  if (threadIdx.x != 0) return;
  __threadfence_system();
  const uint32_t old = atomicAdd(p.sched, 1u);
  if (old == gridDim.x - 1) {
    const bool all_ok = ok && p.sched[1] == 0;
    for (int i = 0; i < p.M / BM; ++i) p.panel_flags[i] = 0;
    p.sched[0] = 0;
    p.sched[1] = 0;
    p.sched[2] = 0;  // the tile counter
    p.sched[3] = 0;  // the copy warps' unit counter
    __threadfence_system();
    // done_always: a caller that reads the status word learns of the end of the kernel either way (an RPC
    // handler must answer); otherwise the flag means "Y is complete" and stays silent after a failure
    if ((all_ok || p.done_always) && p.done_flag) st_release_sys(p.done_flag, p.done_value);
  }
}

template <bool FP8>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
remote_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ CUtensorMap map_y, GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  if ((int)blockIdx.x < p.copy_ctas) {
    // first the transfer of X, then this CTA computes tiles like the others
    const bool ok = copy_role_n(p, GEMM_THREADS, smem_raw);
    if (!ok) {
      finish_cta(p, false);
      return;
    }
    asm volatile("fence.proxy.async;" ::: "memory");
    __syncthreads();
  }
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* sA = smem;
  unsigned char* sB = smem + (size_t)STAGES * A_STAGE_BYTES;
  unsigned char* sEpi = smem + (size_t)STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);  // 1024-aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(sEpi + EPI_SLABS * EPI_SLAB_BYTES);
  // bars: [0,S) full, [S,2S) empty, [2S,2S+2) tmem_full, [2S+2,2S+4) tmem_empty, then TILE_RING tile slots
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ int s_tiles[TILE_RING];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 + b); };
  auto tile_bar = [&](int i) { return bar0 + 8u * (2 * STAGES + 4 + i); };

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 4);
    }
    for (int i = 0; i < TILE_RING; ++i) mbar_init(tile_bar(i), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;

  const int m_blocks = p.M / BM, n_blocks = p.N / BN;
  const int total = m_blocks * n_blocks;
  const int k_iters = p.K * p.elem_bytes / BKB;
  const int kelems = BKB / p.elem_bytes;  // elements of K per stage
  volatile int* abort = &s_abort;
  // the next tile as the consumer roles see it: bounded wait on the ring slot, then its content
  auto next_tile = [&](int it) -> int {
    if (!mbar_wait(tile_bar(it & (TILE_RING - 1)), (uint32_t)(it / TILE_RING) & 1u, abort, p.timeout_ns)) return total;
    return *(volatile int*)&s_tiles[it & (TILE_RING - 1)];
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int it = 0;; ++it) {
        const int tile = *abort ? total : (int)atomicAdd(p.sched + 2, 1u);
        s_tiles[it & (TILE_RING - 1)] = tile;
        mbar_arrive(tile_bar(it & (TILE_RING - 1)));
        if (tile >= total) break;
        int mb, nb;
        tile_coords(tile, m_blocks, n_blocks, p.head_blocks, mb, nb);
        if (p.panel_target > 0) {
          if (!wait_u32_ge_gpu(p.panel_flags + mb, p.panel_target, p.timeout_ns)) {
            *abort = 1;
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort, p.timeout_ns)) break;
          mbar_expect_tx(full_bar(s), A_STAGE_BYTES + B_STAGE_BYTES);
          tma_load_2d(smem_u32(sA + (size_t)s * A_STAGE_BYTES), &map_a, full_bar(s), k * kelems, mb * BM);
          tma_load_2d(smem_u32(sB + (size_t)s * B_STAGE_BYTES), &map_b, full_bar(s), k * kelems, nb * BN);
          if (++s == STAGES) s = 0, ph ^= 1u;
        }
      }
      if (*abort) {  // let copies that are still in flight land before the CTA retires
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc<FP8, BN>();
      int s = 0;
      uint32_t ph = 0;
      for (int it = 0;; ++it) {
        if (next_tile(it) >= total) break;
        const int buf = it & 1;
        const uint32_t tph = (uint32_t)(it >> 1) & 1u;
        if (!mbar_wait(tempty_bar(buf), tph ^ 1u, abort, p.timeout_ns)) break;
        tc_fence_after();
        const uint32_t tacc = tmem_base + (uint32_t)buf * BN;
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(full_bar(s), ph, abort, p.timeout_ns)) break;
          tc_fence_after();
          const uint32_t a0 = smem_u32(sA + (size_t)s * A_STAGE_BYTES);
          const uint32_t b0 = smem_u32(sB + (size_t)s * B_STAGE_BYTES);
#pragma unroll
          for (int kk = 0; kk < BKB / 32; ++kk) {
            umma<FP8>(tacc, umma_desc_sw128(a0 + kk * 32), umma_desc_sw128(b0 + kk * 32), idesc, (uint32_t)((k | kk) != 0));
          }
          umma_commit(empty_bar(s));
          if (++s == STAGES) s = 0, ph ^= 1u;
        }
        umma_commit(tfull_bar(buf));
      }
    }
  } else if (warp < 4) {
    // warps 2 and 3: X (and its scales) from the caller's memory into the staging buffer
    if (p.copy_warps > 0) copy_warp_role(p, (uint32_t)blockIdx.x * 2u + (uint32_t)(warp - 2), lane);
  } else {
    // ---------------- epilogue ----------------
    const int lg = warp - 4;  // TMEM lane group of this warp
    const int row_local = lg * 32 + lane;
    const bool elected = warp == 4 && lane == 0;  // issues (and so owns) the TMA stores
    const uint32_t epi0 = smem_u32(sEpi);
    uint32_t slab = 0;
    for (int it = 0;; ++it) {
      // every lane asks: a lane that gives up (limit, abort) reads `total`, and the vote below
      // takes all four warps out together
      const int tile = next_tile(it);
      if (epi_vote_any(1, tile >= total)) break;
      int mb, nb;
      tile_coords(tile, m_blocks, n_blocks, p.head_blocks, mb, nb);
      const int buf = it & 1;
      const uint32_t tph = (uint32_t)(it >> 1) & 1u;
      const bool got = mbar_wait(tfull_bar(buf), tph, abort, p.timeout_ns);
      if (epi_vote_any(1, !got)) break;  // all four warps or none: the slab barriers below need everyone
      tc_fence_after();
      const uint32_t tbase = tmem_base + ((uint32_t)(lg * 32) << 16) + (uint32_t)buf * BN;
#pragma unroll 1
      for (int sl = 0; sl < BN / 64; ++sl, ++slab) {
        const uint32_t sbuf = epi0 + (slab & 1u) * EPI_SLAB_BYTES;
        if (elected) bulk_wait_read_1();  // the store that used this slab two steps ago has read it
        epi_bar_sync(1);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[32];
          tmem_ld32(tbase + sl * 64 + h * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              q[e] = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2 * e]), __uint_as_float(r[8 * j + 2 * e + 1]));
            const int chunk = h * 4 + j;  // 16-byte chunk of this row's 128 bytes
            st_shared_u4(sbuf + (uint32_t)row_local * 128u + (uint32_t)((chunk ^ (row_local & 7)) * 16), o);
          }
        }
        if (sl == BN / 64 - 1) {  // the accumulator is out of TMEM: the next tile may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar(buf));
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        epi_bar_sync(1);
        if (elected) {
          tma_store_2d(&map_y, sbuf, nb * BN + sl * 64, mb * BM);
          bulk_commit();
        }
      }
    }
    if (elected) {  // Y is complete before this CTA reports
      bulk_wait_all();
      asm volatile("fence.proxy.async;" ::: "memory");
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
  const bool ok = s_abort == 0;
  if (!ok && threadIdx.x == 0) {
    set_status(p.status, EUX_ST_TIMEOUT, 20);
    atomicExch(p.sched + 1, 1u);
  }
  finish_cta(p, ok);
}


// ---------------------------------------------------------------------------
// Block-scaled fp8 (e4m3) variant: X carries one fp32 scale per row per 128
// elements of K, W one per 128x128 block. The tensor cores cannot apply fp32
// scales, so every 128-wide K block is multiplied on its own into one of two
// TMEM buffers (accumulate off) and the epilogue warps add it, scaled by
// sx[row, kb] * sw[nb, kb], into fp32 registers while the next block is being
// multiplied. Tile 128 x 128, one stage = one K block (128 B per row).
// ---------------------------------------------------------------------------
constexpr int BN8 = 128;
constexpr int STAGES8 = 6;
constexpr int A8_STAGE_BYTES = BM * BKB;
constexpr int B8_STAGE_BYTES = BN8 * BKB;
constexpr int GEMM8_THREADS = 384;  // warp 0 TMA, warp 1 MMA, warps 4..11 epilogue (two per TMEM lane group)
constexpr int TMEM8_COLS = 512;
constexpr int TBUF8 = 4;  // partial products in flight: four 128-column TMEM buffers
constexpr size_t GEMM8_SMEM = (size_t)STAGES8 * (A8_STAGE_BYTES + B8_STAGE_BYTES) + 2 * 16384 /* output slabs */ + 1024 + 256;

__global__ void __launch_bounds__(GEMM8_THREADS, 1)
remote_gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_y, GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  if ((int)blockIdx.x < p.copy_ctas) {
    // first the transfer of X and its scales, then this CTA computes tiles like the others
    const bool ok = copy_role_n(p, GEMM8_THREADS, smem_raw);
    if (!ok) {
      finish_cta(p, false);
      return;
    }
    asm volatile("fence.proxy.async;" ::: "memory");
    __syncthreads();
  }
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* sA = smem;
  unsigned char* sB = smem + (size_t)STAGES8 * A8_STAGE_BYTES;
  unsigned char* sEpi = smem + (size_t)STAGES8 * (A8_STAGE_BYTES + B8_STAGE_BYTES);  // 1024-aligned, one slab per half
  uint64_t* bars = reinterpret_cast<uint64_t*>(sEpi + EPI_SLABS * EPI_SLAB_BYTES);
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ int s_tiles[TILE_RING];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES8 + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * STAGES8 + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * STAGES8 + TBUF8 + b); };
  auto tile_bar = [&](int i) { return bar0 + 8u * (2 * STAGES8 + 2 * TBUF8 + i); };
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < TILE_RING; ++i) mbar_init(tile_bar(i), 1);
    for (int s = 0; s < STAGES8; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < TBUF8; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 8);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                 "r"((uint32_t)TMEM8_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  const int m_blocks = p.M / BM, n_blocks = p.N / BN8;
  const int total = m_blocks * n_blocks;
  const int k_blocks = p.K / 128;
  volatile int* abort = &s_abort;
  auto next_tile = [&](int it) -> int {
    if (!mbar_wait(tile_bar(it & (TILE_RING - 1)), (uint32_t)(it / TILE_RING) & 1u, abort, p.timeout_ns)) return total;
    return *(volatile int*)&s_tiles[it & (TILE_RING - 1)];
  };

  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int it = 0;; ++it) {
        const int tile = *abort ? total : (int)atomicAdd(p.sched + 2, 1u);
        s_tiles[it & (TILE_RING - 1)] = tile;
        mbar_arrive(tile_bar(it & (TILE_RING - 1)));
        if (tile >= total) break;
        int mb, nb;
        tile_coords(tile, m_blocks, n_blocks, p.head_blocks, mb, nb);
        if (p.panel_target > 0) {
          if (!wait_u32_ge_gpu(p.panel_flags + mb, p.panel_target, p.timeout_ns)) {
            *abort = 1;
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int k = 0; k < k_blocks; ++k) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort, p.timeout_ns)) break;
          mbar_expect_tx(full_bar(s), A8_STAGE_BYTES + B8_STAGE_BYTES);
          tma_load_2d(smem_u32(sA + (size_t)s * A8_STAGE_BYTES), &map_a, full_bar(s), k * 128, mb * BM);
          tma_load_2d(smem_u32(sB + (size_t)s * B8_STAGE_BYTES), &map_b, full_bar(s), k * 128, nb * BN8);
          if (++s == STAGES8) s = 0, ph ^= 1u;
        }
      }
      if (*abort) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc<true, BN8>();
      int s = 0;
      uint32_t ph = 0;
      uint32_t blk = 0;  // running K-block count: selects the TMEM buffer and its phase
      for (int it = 0;; ++it) {
        if (next_tile(it) >= total || *abort) break;
        for (int k = 0; k < k_blocks && !*abort; ++k, ++blk) {
          const int buf = blk & (TBUF8 - 1);
          const uint32_t tph = (blk / TBUF8) & 1u;
          if (!mbar_wait(tempty_bar(buf), tph ^ 1u, abort, p.timeout_ns)) break;
          if (!mbar_wait(full_bar(s), ph, abort, p.timeout_ns)) break;
          tc_fence_after();
          const uint32_t tacc = tmem_base + (uint32_t)buf * BN8;
          const uint32_t a0 = smem_u32(sA + (size_t)s * A8_STAGE_BYTES);
          const uint32_t b0 = smem_u32(sB + (size_t)s * B8_STAGE_BYTES);
#pragma unroll
          for (int kk = 0; kk < BKB / 32; ++kk)
            umma<true>(tacc, umma_desc_sw128(a0 + kk * 32), umma_desc_sw128(b0 + kk * 32), idesc, (uint32_t)(kk != 0));
          umma_commit(empty_bar(s));
          umma_commit(tfull_bar(buf));
          if (++s == STAGES8) s = 0, ph ^= 1u;
        }
      }
    }
  } else if (warp < 4) {
    // warps 2 and 3: X (and its scales) from the caller's memory into the staging buffer
    if (p.copy_warps > 0) copy_warp_role(p, (uint32_t)blockIdx.x * 2u + (uint32_t)(warp - 2), lane);
  } else {
    const int lg = (warp - 4) & 3;    // TMEM lane group
    const int half = (warp - 4) >> 2;  // which 64 columns of the tile
    const int row_local = lg * 32 + lane;
    const bool elected = lg == 0 && lane == 0;  // one per half: issues (and owns) that half's TMA stores
    const uint32_t sbuf = smem_u32(sEpi) + (uint32_t)half * EPI_SLAB_BYTES;
    uint32_t blk = 0;
    const int kscales = p.K / 128;
    for (int it = 0;; ++it) {
      const int tile = next_tile(it);
      if (epi_vote_any(1 + half, tile >= total)) break;  // the four warps of a half leave together
      int mb, nb;
      tile_coords(tile, m_blocks, n_blocks, p.head_blocks, mb, nb);
      const int row = mb * BM + lg * 32 + lane;
      const float* sx = p.x_scale_stage + (size_t)row * kscales;
      const float* sw = p.w_scale + (size_t)nb * kscales;
      float acc[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) acc[j] = 0.f;
      bool ok = true;
      // When X is pulled from a peer its row scales travel with it: they are known to have landed
      // once the panel is reported, so the warp checks the panel itself before it reads any of them
      // (the loads below run ahead of the MMA, which is what hides their latency).
      if (p.panel_target > 0) {
        int arrived = 1;
        if (lane == 0) arrived = wait_u32_ge_gpu(p.panel_flags + mb, p.panel_target, p.timeout_ns) ? 1 : 0;
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        if (!arrived) {
          *abort = 1;
          ok = false;
        }
      }
      // scales two K-blocks ahead of their use
      float s0 = 0.f, s1 = 0.f;
      if (ok) {
        s0 = __ldcg(sx) * __ldg(sw);
        if (k_blocks > 1) s1 = __ldcg(sx + 1) * __ldg(sw + 1);
      }
      for (int k = 0; ok && k < k_blocks; ++k, ++blk) {
        const int buf = blk & (TBUF8 - 1);
        const uint32_t tph = (blk / TBUF8) & 1u;
        float sx2 = 0.f, sw2 = 0.f;
        if (k + 2 < k_blocks) {
          sx2 = __ldcg(sx + k + 2);
          sw2 = __ldg(sw + k + 2);
        }
        if (!mbar_wait(tfull_bar(buf), tph, abort, p.timeout_ns)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const float scale = s0;
        const uint32_t tbase = tmem_base + ((uint32_t)(lg * 32) << 16) + (uint32_t)buf * BN8 + (uint32_t)half * 64;
        uint32_t r0[32], r1[32];
        tmem_ld32(tbase, r0);
        tmem_ld32(tbase + 32, r1);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(buf));  // the buffer is in registers: the next block may overwrite it
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          ffma2(acc[j], acc[j + 1], __uint_as_float(r0[j]), __uint_as_float(r0[j + 1]), scale);
          ffma2(acc[32 + j], acc[33 + j], __uint_as_float(r1[j]), __uint_as_float(r1[j + 1]), scale);
        }
        s0 = s1;
        s1 = sx2 * sw2;
      }
      if (elected) bulk_wait_read_0();  // the previous tile's store has read this half's slab
      if (epi_vote_any(1 + half, !ok)) break;  // the four warps of a half leave together
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 o;
        __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) q[j] = __floats2bfloat162_rn(acc[c * 8 + 2 * j], acc[c * 8 + 2 * j + 1]);
        st_shared_u4(sbuf + (uint32_t)row_local * 128u + (uint32_t)((c ^ (row_local & 7)) * 16), o);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      epi_bar_sync(1 + half);
      if (elected) {
        tma_store_2d(&map_y, sbuf, nb * BN8 + half * 64, mb * BM);
        bulk_commit();
      }
    }
    if (elected) {  // Y is complete before this CTA reports
      bulk_wait_all();
      asm volatile("fence.proxy.async;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM8_COLS)
                 : "memory");
  }
  const bool ok = s_abort == 0;
  if (!ok && threadIdx.x == 0) {
    set_status(p.status, EUX_ST_TIMEOUT, 21);
    atomicExch(p.sched + 1, 1u);
  }
  finish_cta(p, ok);
}

// ---------------------------------------------------------------------------
// bf16, two CTAs per tile (cta_group::2): a cluster of two CTAs computes a 256 x 256 tile. Each CTA
// loads its 128 rows of A and its 128 of the tile's 256 rows of Wt, the even CTA issues
// tcgen05.mma.cta_group::2 over both CTAs' shared memory, and each CTA ends up with its 128 rows of
// the accumulator in its own TMEM. Per CTA and K-step that is 32 KiB of operands instead of 48 KiB,
// so six stages fit where the one-CTA kernel has four: more bytes in flight against the L2 latency
// and two thirds of the shared-memory reads per flop. M must be a multiple of 256. With a remote X the first
// copy_ctas CTAs (whole pairs) copy it before they join, and the even CTA of each pair draws the pair's
// tiles from the global counter and hands them to its partner through distributed shared memory.
// All loads are per-CTA loads that signal the even CTA's barrier; no load is broadcast.
// ---------------------------------------------------------------------------
constexpr int B2_STAGE_BYTES = (BN / 2) * BKB;  // this CTA's half of the Wt tile: 16 KiB
// The MX variant (e4m3 values, one power-of-two scale per 32 elements along K, applied by the tensor core:
// tcgen05.mma kind::mxf8f6f4.block_scale) runs on the same frame. A K-step is again 128 bytes of every row,
// now 128 elements, and each stage also carries the step's scale factors: 512 bytes for this CTA's 128 rows
// of X and 1024 for the tile's 256 rows of Wt, in the order in which tcgen05.cp puts them into TMEM
// (byte (r % 32) * 16 + (r / 32) * 4 + j for row r and 32-element block j of the step). The scale factors
// take TMEM columns too, so the MX variant has one accumulator buffer where bf16 has two.
constexpr int SF_STAGE_BYTES = 512 + 1024;
template <bool MX> struct PairCfg {
  static constexpr int STAGES = MX ? 5 : 6;
  static constexpr int NBUF = MX ? 1 : 2;  // accumulator buffers of BN columns in TMEM
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B2_STAGE_BYTES + (MX ? SF_STAGE_BYTES : 0);
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 2 * 16384 + 1024 + 256;
};
constexpr uint32_t SF_TMEM_COL = 2 * BN - 16;  // 4 columns of X scales, then 8 of Wt scales (MX has one accumulator: 256..511 are free)

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void st_shared_remote_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// like mbar_wait, but what the arriving CTA of the cluster wrote before its arrive is visible afterwards
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort, uint64_t timeout_ns) {
  auto try_once = [&]() {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
  };
  if (try_once()) return true;
  const uint64_t limit = timeout_ns ? timeout_ns : 2000000000ull;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 0; it < 0x7fffffffu; ++it) {
    if (try_once()) return true;
    if ((it & 255u) == 255u) {
      if (*abort) return false;
      if (globaltimer_ns() - t0 > limit) {
        *abort = 1;
        return false;
      }
    }
  }
  *abort = 1;
  return false;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// per-CTA tile load of a CTA pair: the bytes land in this CTA, the completion is counted on `bar`, a
// shared::cluster address (the even CTA's barrier)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(map), "r"(bar_cluster), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_c, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_c),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on one barrier (shared::cluster address) when the pair's MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster) : "memory");
}

// 128 rows x 4 scale bytes (512 bytes of shared memory, rows of 16 bytes, 8-row groups 128 bytes apart) into
// four TMEM columns of every lane quarter, in both CTAs of the pair
__device__ __forceinline__ void sf_to_tmem_pair(uint32_t tmem_col, uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);
  d |= (uint64_t)(128u >> 4) << 32;  // stride byte offset
  d |= (uint64_t)1 << 46;            // descriptor version; no swizzle
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(d) : "memory");
}
__device__ __forceinline__ void umma_mx_pair(uint32_t tmem_c, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t tmem_sfa,
                                             uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(tmem_c),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}

template <bool MX>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
remote_gemm_2cta_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const __grid_constant__ CUtensorMap map_y, const __grid_constant__ CUtensorMap map_sfa,
                        const __grid_constant__ CUtensorMap map_sfb, GemmParams p) {
  constexpr int STAGES2 = PairCfg<MX>::STAGES;
  constexpr int NBUF = PairCfg<MX>::NBUF;
  extern __shared__ unsigned char smem_raw[];
  bool copy_ok = true;
  if ((int)blockIdx.x < p.copy_ctas) {
    // whole pairs copy X first (copy_ctas is even). A CTA whose copy failed still walks through the
    // rest with its abort flag set: its partner waits for it at the cluster barriers.
    copy_ok = copy_role_n(p, GEMM_THREADS, smem_raw);
    asm volatile("fence.proxy.async;" ::: "memory");
    __syncthreads();
  }
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* sA = smem;
  unsigned char* sB = smem + (size_t)STAGES2 * A_STAGE_BYTES;
  unsigned char* sEpi = smem + (size_t)STAGES2 * (A_STAGE_BYTES + B2_STAGE_BYTES);  // 1024-aligned: the stores are swizzled
  unsigned char* sSF = sEpi + EPI_SLABS * EPI_SLAB_BYTES;                           // MX only
  uint64_t* bars = reinterpret_cast<uint64_t*>(sSF + (MX ? (size_t)STAGES2 * SF_STAGE_BYTES : 0));
  // bars: [0,S) full (used in the even CTA), [S,2S) empty, [2S,2S+2) tmem_full, [2S+2,2S+4) tmem_empty (even CTA),
  // then TILE_RING tile slots
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ int s_tiles[TILE_RING];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const bool leader = rank == 0;
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES2 + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * STAGES2 + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * STAGES2 + 2 + b); };
  auto tile_bar = [&](int i) { return bar0 + 8u * (2 * STAGES2 + 4 + i); };
  if (threadIdx.x == 0) {
    s_abort = copy_ok ? 0 : 1;
    for (int i = 0; i < TILE_RING; ++i) mbar_init(tile_bar(i), 1);
    for (int s = 0; s < STAGES2; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 8);  // four epilogue warps in each CTA of the pair
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {  // one warp of each CTA, together
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the partner's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;

  const int m_blocks = p.M / (2 * BM), n_blocks = p.N / BN;
  const int total = m_blocks * n_blocks;
  const int k_iters = p.K * p.elem_bytes / BKB;
  const int kelems = BKB / p.elem_bytes;
  volatile int* abort = &s_abort;
  // The even CTA draws the pair's next tile from the global counter and puts it into both CTAs'
  // rings (its own, and the partner's through distributed shared memory).
  auto next_tile = [&](int it) -> int {
    if (!mbar_wait_cluster(tile_bar(it & (TILE_RING - 1)), (uint32_t)(it / TILE_RING) & 1u, abort, p.timeout_ns)) return total;
    return *(volatile int*)&s_tiles[it & (TILE_RING - 1)];
  };

  if (warp == 0) {
    // ---------------- loads: both CTAs, completion counted in the even CTA ----------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int it = 0;; ++it) {
        int tile;
        if (leader) {
          tile = *abort ? total : (int)atomicAdd(p.sched + 2, 1u);
          const int slot = it & (TILE_RING - 1);
          s_tiles[slot] = tile;
          mbar_arrive(tile_bar(slot));
          st_shared_remote_u32(map_to_cta(smem_u32(&s_tiles[slot]), 1), (uint32_t)tile);
          mbar_arrive_remote(map_to_cta(tile_bar(slot), 1));
        } else {
          tile = next_tile(it);
        }
        if (tile >= total) break;
        int mb, nb;
        tile_coords(tile, m_blocks, n_blocks, p.head_blocks, mb, nb);
        if (p.panel_target > 0) {  // this CTA's 128 rows of the 256-row block
          if (!wait_u32_ge_gpu(p.panel_flags + 2 * mb + (int)rank, p.panel_target, p.timeout_ns)) {
            *abort = 1;
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort, p.timeout_ns)) break;
          const uint32_t full_leader = map_to_cta(full_bar(s), 0);
          if (leader) mbar_expect_tx(full_bar(s), 2 * PairCfg<MX>::STAGE_BYTES);
          tma_load_2d_pair(smem_u32(sA + (size_t)s * A_STAGE_BYTES), &map_a, full_leader, k * kelems, mb * 2 * BM + (int)rank * BM);
          tma_load_2d_pair(smem_u32(sB + (size_t)s * B2_STAGE_BYTES), &map_b, full_leader, k * kelems, nb * BN + (int)rank * (BN / 2));
          if (MX) {  // this CTA's X scales of the step, and the whole tile's Wt scales (each CTA needs all 256 in its TMEM)
            const uint32_t sf = smem_u32(sSF + (size_t)s * SF_STAGE_BYTES);
            tma_load_2d_pair(sf, &map_sfa, full_leader, 0, (mb * 2 + (int)rank) * k_iters + k);
            tma_load_2d_pair(sf + 512, &map_sfb, full_leader, 0, k * (p.N / 128) + nb * 2);
          }
          if (++s == STAGES2) s = 0, ph ^= 1u;
        }
      }
      if (*abort) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA: the even CTA issues for the pair ----------------
    if (leader && lane == 0) {
      // bf16: D fp32 (bit 4), A and B bf16 (bits 7, 10). MX: A and B e4m3 (zero), scales UE8M0 (bit 23); the
      // 32-element block of the K-step goes into bits 29..30 (X scales) and 4..5 (Wt scales) per instruction.
      constexpr uint32_t idesc = (MX ? (1u << 23) : ((1u << 4) | (1u << 7) | (1u << 10))) | ((uint32_t)(BN >> 3) << 17) |
                                 ((uint32_t)((2 * BM) >> 4) << 24);
      int s = 0;
      uint32_t ph = 0;
      for (int it = 0;; ++it) {
        if (next_tile(it) >= total || *abort) break;
        const int buf = it % NBUF;
        const uint32_t tph = (uint32_t)(it / NBUF) & 1u;
        if (!mbar_wait(tempty_bar(buf), tph ^ 1u, abort, p.timeout_ns)) break;
        tc_fence_after();
        const uint32_t tacc = tmem_base + (uint32_t)buf * BN;
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(full_bar(s), ph, abort, p.timeout_ns)) break;
          tc_fence_after();
          const uint32_t a0 = smem_u32(sA + (size_t)s * A_STAGE_BYTES);
          const uint32_t b0 = smem_u32(sB + (size_t)s * B2_STAGE_BYTES);
          if (MX) {
            // the step's scale factors into TMEM, in both CTAs; the tensor pipe runs them before the MMAs below
            const uint32_t sf = smem_u32(sSF + (size_t)s * SF_STAGE_BYTES);
            const uint32_t tsf = tmem_base + SF_TMEM_COL;
            sf_to_tmem_pair(tsf, sf);
            sf_to_tmem_pair(tsf + 4, sf + 512);
            sf_to_tmem_pair(tsf + 8, sf + 1024);
#pragma unroll
            for (int kk = 0; kk < BKB / 32; ++kk)
              umma_mx_pair(tacc, umma_desc_sw128(a0 + kk * 32), umma_desc_sw128(b0 + kk * 32),
                           idesc | ((uint32_t)kk << 29) | ((uint32_t)kk << 4), tsf, tsf + 4, (uint32_t)((k | kk) != 0));
          } else {
#pragma unroll
            for (int kk = 0; kk < BKB / 32; ++kk)
              umma_pair(tacc, umma_desc_sw128(a0 + kk * 32), umma_desc_sw128(b0 + kk * 32), idesc, (uint32_t)((k | kk) != 0));
          }
          // the stage is free in both CTAs once these MMAs have read it
          umma_commit_pair(empty_bar(s));
          umma_commit_pair(map_to_cta(empty_bar(s), 1));
          if (++s == STAGES2) s = 0, ph ^= 1u;
        }
        umma_commit_pair(tfull_bar(buf));
        umma_commit_pair(map_to_cta(tfull_bar(buf), 1));
      }
    }
  } else if (warp < 4) {
    // ---------------- warps 2 and 3: X from the caller's memory into the staging buffer ----------------
    if (p.copy_warps > 0) copy_warp_role(p, (uint32_t)blockIdx.x * 2u + (uint32_t)(warp - 2), lane);
  } else {
    // ---------------- epilogue: each CTA stores its 128 rows ----------------
    const int lg = warp - 4;
    const int row_local = lg * 32 + lane;
    const bool elected = warp == 4 && lane == 0;
    const uint32_t epi0 = smem_u32(sEpi);
    uint32_t slab = 0;
    for (int it = 0;; ++it) {
      const int tile = next_tile(it);
      if (epi_vote_any(1, tile >= total)) break;
      int mb, nb;
      tile_coords(tile, m_blocks, n_blocks, p.head_blocks, mb, nb);
      const int buf = it % NBUF;
      const uint32_t tph = (uint32_t)(it / NBUF) & 1u;
      const bool got = !*abort && mbar_wait(tfull_bar(buf), tph, abort, p.timeout_ns);
      if (epi_vote_any(1, !got)) break;
      tc_fence_after();
      const uint32_t tbase = tmem_base + ((uint32_t)(lg * 32) << 16) + (uint32_t)buf * BN;
      if (MX) {
        // One accumulator buffer: the next tile's MMAs wait for this epilogue, so the whole row comes out of
        // TMEM first, rounded to bf16 in registers (128 words per thread), and the buffer is handed back
        // before anything is written; the slabs then leave while the tensor pipe works on the next tile.
        uint32_t pk[BN / 2];
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tbase + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            __nv_bfloat162 q = __floats2bfloat162_rn(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1]));
            pk[c * 16 + e] = *reinterpret_cast<uint32_t*>(&q);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(map_to_cta(tempty_bar(buf), 0));
#pragma unroll
        for (int sl = 0; sl < BN / 64; ++sl, ++slab) {
          const uint32_t sbuf = epi0 + (slab & 1u) * EPI_SLAB_BYTES;
          if (elected) bulk_wait_read_1();
          epi_bar_sync(1);
#pragma unroll
          for (int chunk = 0; chunk < 8; ++chunk) {
            const uint4 o = make_uint4(pk[sl * 32 + chunk * 4], pk[sl * 32 + chunk * 4 + 1], pk[sl * 32 + chunk * 4 + 2],
                                       pk[sl * 32 + chunk * 4 + 3]);
            st_shared_u4(sbuf + (uint32_t)row_local * 128u + (uint32_t)((chunk ^ (row_local & 7)) * 16), o);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          epi_bar_sync(1);
          if (elected) {
            tma_store_2d(&map_y, sbuf, nb * BN + sl * 64, mb * 2 * BM + (int)rank * BM);
            bulk_commit();
          }
        }
        continue;
      }
#pragma unroll 1
      for (int sl = 0; sl < BN / 64; ++sl, ++slab) {
        const uint32_t sbuf = epi0 + (slab & 1u) * EPI_SLAB_BYTES;
        if (elected) bulk_wait_read_1();
        epi_bar_sync(1);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[32];
          tmem_ld32(tbase + sl * 64 + h * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              q[e] = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2 * e]), __uint_as_float(r[8 * j + 2 * e + 1]));
            const int chunk = h * 4 + j;
            st_shared_u4(sbuf + (uint32_t)row_local * 128u + (uint32_t)((chunk ^ (row_local & 7)) * 16), o);
          }
        }
        if (sl == BN / 64 - 1) {  // this CTA's half of the accumulator is out of TMEM
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_remote(map_to_cta(tempty_bar(buf), 0));
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        epi_bar_sync(1);
        if (elected) {
          tma_store_2d(&map_y, sbuf, nb * BN + sl * 64, mb * 2 * BM + (int)rank * BM);
          bulk_commit();
        }
      }
    }
    if (elected) {
      bulk_wait_all();
      asm volatile("fence.proxy.async;" ::: "memory");
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still touch its shared memory or TMEM
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
  }
  const bool ok = s_abort == 0;
  if (!ok && threadIdx.x == 0) {
    set_status(p.status, EUX_ST_TIMEOUT, 22);
    atomicExch(p.sched + 1, 1u);
  }
  finish_cta(p, ok);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// rows x cols (cols contiguous), box = box_rows x (128 bytes of columns), 128B swizzle
static int make_map(CUtensorMap* m, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return EUX_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(BKB / elem_bytes), box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : EUX_ERR_BAD_ARG;
}

// scale factors of the MX variant: `chunks` blocks of 512 bytes, `box_chunks` of them per load, no swizzle
static int make_map_sf(CUtensorMap* m, const void* base, uint64_t chunks, uint32_t box_chunks) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return EUX_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {128, chunks};  // 128 words of 4 bytes
  cuuint64_t strides[1] = {512};
  cuuint32_t box[2] = {128, box_chunks};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : EUX_ERR_BAD_ARG;
}

}  // namespace eux

using namespace eux;

extern "C" int eux_gemm_num_sms(void) {
  int dev = 0, n = 0;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  return n;
}

extern "C" int eux_gemm_launch(const eux_gemm_desc* d, void* stream) {
  if (!d || !d->x_stage || !d->w_t || !d->y_dst || !d->sched || !d->panel_flags) return EUX_ERR_BAD_ARG;
  const bool mx = d->fp8 == 2;  // e4m3 with one UE8M0 scale per 32 elements, scaled by the tensor core
  if (mx && (d->M % (2 * BM) || d->N % BN)) return EUX_ERR_BAD_ARG;
  const int bn = mx ? BN : d->fp8 ? BN8 : BN;
  if (d->M <= 0 || d->N <= 0 || d->K <= 0 || d->M % BM || d->N % bn) return EUX_ERR_BAD_ARG;
  const int eb = d->fp8 ? 1 : 2;
  if ((d->K * eb) % BKB) return EUX_ERR_BAD_ARG;
  if (d->fp8 && (d->K % 128 || !d->x_scale || !d->w_scale)) return EUX_ERR_BAD_ARG;
  const bool pull = d->x_src && d->x_src != d->x_stage;
  if (d->fp8 && pull && !d->x_scale_stage) return EUX_ERR_BAD_ARG;
  // Copy CTAs (when the flags do not ask for copy warps) turn into GEMM CTAs once X is here. Measured on
  // two B200s (8192^3): 16 are best for bf16, 48 for fp8; two copy warps in every CTA beat both, by 4 %
  // (bf16 on pairs) and 7 % (fp8).
  int copy_ctas = pull ? (d->copy_ctas > 0 ? d->copy_ctas : (d->fp8 ? 48 : 16)) : 0;
  const int sms = eux_gemm_num_sms();
  if (copy_ctas >= sms) return EUX_ERR_BAD_ARG;
  CUtensorMap ma, mb;
  if (int rc = make_map(&ma, d->x_stage, eb, (uint64_t)d->M, (uint64_t)d->K, BM)) return rc;
  if (int rc = make_map(&mb, d->w_t, eb, (uint64_t)d->N, (uint64_t)d->K, bn)) return rc;
  CUtensorMap my;  // Y[M,N] bf16 in slabs of 128 rows x 64 columns
  if (int rc = make_map(&my, d->y_dst, 2, (uint64_t)d->M, (uint64_t)d->N, BM)) return rc;
  GemmParams p;
  p.x_src = (const unsigned char*)d->x_src;
  p.x_stage = (unsigned char*)d->x_stage;
  p.y = (unsigned char*)d->y_dst;
  p.M = d->M, p.N = d->N, p.K = d->K, p.elem_bytes = eb;
  p.panel_flags = d->panel_flags, p.sched = d->sched;
  p.done_flag = d->done_flag, p.done_value = d->done_value;
  p.timeout_ns = d->wait_timeout_ns, p.status = d->status, p.copy_ctas = copy_ctas;
  p.x_scale_src = d->fp8 ? d->x_scale : nullptr;
  p.x_scale_stage = d->fp8 ? (pull ? d->x_scale_stage : const_cast<float*>(d->x_scale)) : nullptr;
  p.w_scale = d->w_scale;
  // bits 8..15 of the flags: 1 + the height of the first tile group, 0 for the default
  const int head_arg = (int)((d->flags >> 8) & 0xffu) - 1;
  p.copy_warps = 0;
  p.done_always = (d->flags & EUX_GEMM_FLAG_DONE_ALWAYS) ? 1 : 0;
  p.panel_target = (uint32_t)copy_ctas;
  // copy warps: units of 8 KiB per 128-row panel, plus the units that carry the panel's scales (K * 4 bytes)
  auto warp_target = [&](int) {
    return (uint32_t)(((size_t)BM * d->K * eb) >> 13) + (d->fp8 ? (uint32_t)(((size_t)d->K * 4 + 8191) >> 13) : 0u);
  };
  p.head_blocks = !pull ? 0 : head_arg >= 0 ? head_arg : 4;  // of 128 rows: groups of 4, 4, 8, then 8
  static bool attr_set[64][2] = {{false}};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return EUX_ERR_BAD_ARG;
  if (!attr_set[dev][d->fp8 ? 1 : 0]) {
    cudaError_t e = d->fp8 ? cudaFuncSetAttribute(remote_gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM8_SMEM)
                           : cudaFuncSetAttribute(remote_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev][d->fp8 ? 1 : 0] = true;
  }
  // bf16 with M in whole 256-row blocks can run on CTA pairs (bit 0 of the descriptor's flags)
  const bool want_pairs = (d->flags & EUX_GEMM_FLAG_CTA_PAIRS) != 0;
  if (mx || (want_pairs && !d->fp8 && d->M % (2 * BM) == 0)) {
    static bool attr2_set[64][2] = {{false}};
    if (!attr2_set[dev][mx ? 1 : 0]) {
      cudaError_t e = mx ? cudaFuncSetAttribute(remote_gemm_2cta_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                (int)PairCfg<true>::SMEM)
                         : cudaFuncSetAttribute(remote_gemm_2cta_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                (int)PairCfg<false>::SMEM);
      if (e != cudaSuccess) return (int)e;
      attr2_set[dev][mx ? 1 : 0] = true;
    }
    CUtensorMap mb2;  // this CTA's half of a Wt tile: 128 rows
    if (int rc = make_map(&mb2, d->w_t, eb, (uint64_t)d->N, (uint64_t)d->K, BN / 2)) return rc;
    const int tiles2 = (d->M / (2 * BM)) * (d->N / BN);
    int copy_pairs = pull ? (copy_ctas + 1) / 2 : 0;
    if (copy_pairs > sms / 2 - 1) copy_pairs = sms / 2 - 1;
    p.copy_ctas = 2 * copy_pairs;
    p.panel_target = (uint32_t)p.copy_ctas;
    if (pull && head_arg < 0) p.head_blocks = 2;  // of 256 rows: groups of 2, 2, 4, then 8
    if (pull && (d->flags & EUX_GEMM_FLAG_COPY_WARPS)) {  // two warps of every CTA copy, no CTA only copies
      p.copy_ctas = 0;
      p.copy_warps = 2 * 2 * (sms / 2);
      p.panel_target = warp_target(p.copy_warps);
    }
    // every pair computes (the copying ones after their transfer), and they all have to be resident:
    // pairs that copy must not wait for a slot behind pairs that wait for their panels
    const int pairs = pull ? sms / 2 : (tiles2 < sms / 2 ? tiles2 : sms / 2);
    if (mx) {
      CUtensorMap msa, msb;
      if (int rc = make_map_sf(&msa, p.x_scale_stage, (uint64_t)(d->M / 128) * (d->K / 128), 1)) return rc;
      if (int rc = make_map_sf(&msb, d->w_scale, (uint64_t)(d->N / 128) * (d->K / 128), 2)) return rc;
      remote_gemm_2cta_kernel<true><<<2 * pairs, GEMM_THREADS, PairCfg<true>::SMEM, (cudaStream_t)stream>>>(ma, mb2, my, msa, msb, p);
    } else {
      remote_gemm_2cta_kernel<false><<<2 * pairs, GEMM_THREADS, PairCfg<false>::SMEM, (cudaStream_t)stream>>>(ma, mb2, my, ma, ma, p);
    }
    return (int)cudaGetLastError();
  }
  const int tiles = (d->M / BM) * (d->N / bn);
  int grid = copy_ctas + (tiles < sms - copy_ctas ? tiles : sms - copy_ctas);
  if (pull && (d->flags & EUX_GEMM_FLAG_COPY_WARPS)) {  // every SM takes part in the copy, with or without a tile
    grid = sms;
    p.copy_ctas = 0;
    p.copy_warps = 2 * grid;
    p.panel_target = warp_target(p.copy_warps);
  }
  if (d->fp8) remote_gemm_fp8_kernel<<<grid, GEMM8_THREADS, GEMM8_SMEM, (cudaStream_t)stream>>>(ma, mb, my, p);
  else remote_gemm_kernel<false><<<grid, GEMM_THREADS, GEMM_SMEM, (cudaStream_t)stream>>>(ma, mb, my, p);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------
// eux_gemm_bf16_noalloc: the GEMM for callers that cannot allocate (see eux_no_alloc.h).
// The scratch the kernel needs lives in this static device array. In host code the
// name `g_noalloc_gemm_scratch` is only a stand-in: the address a kernel can use is
// obtained per device with cudaGetSymbolAddress below.
// ---------------------------------------------------------------------------
#include <atomic>

#include "eux_no_alloc.h"

static __device__ __align__(256) uint32_t g_noalloc_gemm_scratch[EUX_NOALLOC_GEMM_SCRATCH_BYTES / 4];

extern "C" int eux_gemm_bf16_noalloc(const void* x, const void* w_t, void* y, int M, int N, int K, uint32_t* status,
                                     uint64_t wait_timeout_ns, void* stream) {
  if (!x || !w_t || !y || M <= 0 || N <= 0 || K <= 0) return EUX_ERR_BAD_ARG;
  if (M > EUX_NOALLOC_GEMM_MAX_M) return EUX_ERR_TOO_LARGE;  // one counter per 128 rows is all the static array holds
  // The shapes the kernels take, checked here so that a call that is going to be refused has put
  // nothing on the stream: the clear below touches the array that every call shares.
  if (M % 128 || N % 256 || K % 64) return EUX_ERR_BAD_ARG;
  // Set-up, once per device, with that device current: the device address of the static array.
  // Host threads may race to be first; they would all store the same address, atomically.
  static std::atomic<uint32_t*> scratch_addr[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return EUX_ERR_BAD_ARG;
  uint32_t* scratch = scratch_addr[dev].load(std::memory_order_acquire);
  if (!scratch) {
    uint32_t* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_gemm_scratch);
    if (e != cudaSuccess) return (int)e;
    scratch_addr[dev].store(ptr, std::memory_order_release);
    scratch = ptr;
  }
  // The array keeps whatever the previous call (or an interrupted kernel) left: counters must start at zero.
  const size_t used = ((size_t)M / 128 + 64) * sizeof(uint32_t);
  e = cudaMemsetAsync(scratch, 0, used, (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  eux_gemm_desc d;
  memset(&d, 0, sizeof(d));
  d.x_src = x;
  d.x_stage = const_cast<void*>(x);  // X is local: no staging, no copy CTAs
  d.w_t = w_t;
  d.y_dst = y;
  d.M = M, d.N = N, d.K = K;
  d.fp8 = 0;
  d.sched = scratch;             // first 64 words: completion counters
  d.panel_flags = scratch + 64;  // then one word per 128-row panel
  d.wait_timeout_ns = wait_timeout_ns;
  d.status = status;
  d.copy_ctas = 0;
  d.flags = EUX_GEMM_FLAG_CTA_PAIRS;  // taken when M is a multiple of 256
  return eux_gemm_launch(&d, stream);
}


// Loads every GEMM kernel (see eux_xfer_preload in tensor_xfer.cu for why a first launch must not be the one
// that loads): a service that launches on behalf of a peer calls this when it is set up.
extern "C" int eux_gemm_preload(void) {
  cudaFuncAttributes attr;
  const void* kernels[] = {(const void*)remote_gemm_kernel<false>, (const void*)remote_gemm_fp8_kernel, (const void*)remote_gemm_2cta_kernel<false>,
                           (const void*)remote_gemm_2cta_kernel<true>};
  for (const void* k : kernels) {
    cudaError_t e = cudaFuncGetAttributes(&attr, k);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}
