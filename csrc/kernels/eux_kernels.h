/* C ABI of libeux_kernels.so: the sm_100a data-plane kernels.
 *
 * Every function returns 0 on success or a cudaError_t / EUX_ERR_* value.
 * Pointers named *_peer may point into another GPU's memory that has been
 * mapped into this process (CUDA IPC or peer access); kernels only ever touch
 * such memory with plain loads/stores or per-CTA bulk copies.
 *
 * All device-side waits are bounded: when a wait runs out the kernel writes
 * EUX_ST_TIMEOUT (plus a location code) into the caller's status word and
 * returns normally, so the context stays usable and the host can turn the
 * status into DEADLINE_EXCEEDED.
 */
#ifndef EUX_KERNELS_H_
#define EUX_KERNELS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define EUX_API __attribute__((visibility("default")))
#else
#define EUX_API
#endif

/* element types understood by the pack / cast path */
enum eux_dtype {
  EUX_DT_BYTES = 0, /* opaque bytes: no cast, no arithmetic */
  EUX_DT_F32 = 1,
  EUX_DT_F16 = 2,
  EUX_DT_BF16 = 3,
  EUX_DT_F8E4M3 = 4,
};

/* elementwise handler fused into the receive / echo side */
enum eux_op {
  EUX_OP_NONE = 0,
  EUX_OP_ADD = 1, /* y = x + arg   (the "+1.0" RPC handler)            */
  EUX_OP_MUL = 2, /* y = x * arg   (arg = 0.5: the divide-by-two handler) */
};

/* device status word values (low 8 bits = code, high bits = where) */
enum eux_status {
  EUX_ST_OK = 0,
  EUX_ST_TIMEOUT = 1,
  EUX_ST_BAD_ARG = 2,
  EUX_ST_OVERFLOW = 3,
};

#define EUX_ERR_BAD_ARG 100001
#define EUX_ERR_TOO_LARGE 100002
#define EUX_ERR_UNSUPPORTED 100003

#define EUX_MAX_DIMS 8

/* One transfer: read `n_elems` elements of `src_dtype` from `src` (dense, or
 * strided when ndim > 0, strides in elements), apply `op`, cast to
 * `dst_dtype`, write densely to `dst`, then release-store `flag_value` to
 * `flag` at system scope. Optional acquire-wait on `wait_flag >= wait_value`
 * before the first read (receive side of a push from a peer). */
typedef struct eux_xfer_desc {
  const void* src;
  void* dst;
  uint64_t n_elems;
  int32_t src_dtype;
  int32_t dst_dtype;
  int32_t op;
  float op_arg;
  int32_t ndim; /* 0: src is dense */
  int32_t reserved0;
  int64_t shape[EUX_MAX_DIMS];
  int64_t stride[EUX_MAX_DIMS];
  uint64_t* flag; /* may be peer memory or mapped pinned host memory; may be NULL */
  uint64_t flag_value;
  const uint64_t* wait_flag; /* local device memory; may be NULL */
  uint64_t wait_value;
  uint64_t wait_timeout_ns;
  uint32_t* status; /* local device (or mapped host) word; may be NULL */
  uint64_t* flag2;  /* a second word published together with `flag` (the sender's own completion word when
                       `flag` belongs to the receiver); may be NULL */
  uint64_t flag2_value;
} eux_xfer_desc;

/* scratch: one zero-initialised uint32 counter per in-flight transfer, used to
 * find the last CTA (which publishes the flag). The kernel leaves it at zero. */
EUX_API int eux_xfer_launch(const eux_xfer_desc* d, uint32_t* scratch_counter, int max_ctas, void* stream);

/* Batch of independent small transfers in one launch: CTA i handles descs[i]
 * (device-resident array of n descriptors). No scratch needed: one CTA each. */
/* Same contract as eux_xfer_launch for a dense same-type copy of 16-byte aligned buffers, moved by the
 * bulk-copy engine (TMA) through shared memory instead of by register loads and stores. */
EUX_API int eux_xfer_bulk_launch(const eux_xfer_desc* desc, uint32_t* scratch_counter, int max_ctas, void* stream);
/* One echo step of a tensor RPC in one launch: `req` (push to the partner + flag), then `resp` (wait for the
   partner's request, handler, push back + flag), then `done` (wait for the response flag; nothing is copied).
   Dense, 16-byte aligned, one dtype; scratch3: three zeroed words, left zero. */
EUX_API int eux_xfer_rpc_step_launch(const eux_xfer_desc* req, const eux_xfer_desc* resp, const eux_xfer_desc* done,
                                     uint32_t* scratch3, int max_ctas, void* stream);
EUX_API int eux_xfer_batch_launch(const eux_xfer_desc* descs_dev, int n, void* stream);

/* Many small dense copies in ONE launch with the descriptors in the launch parameters (nothing is read
 * from host or device memory to find the work): CTA i copies items[i] and then release-stores
 * items[i].flag_value to items[i].flag at system scope, so the host learns of every copy on its own.
 * The transport uses it to pull the payloads of all the small messages that arrived in one pass of its
 * loop (sources are peers' memory), and in the other direction to push small device payloads into the
 * receive ring of a peer (destinations and `flag` are the peer's, `flag2` is the sender's own completion
 * word). n <= EUX_PULL_BATCH_MAX; buffers of any alignment. */
#define EUX_PULL_BATCH_MAX 48
typedef struct eux_pull_item {
  const void* src;
  void* dst;
  uint64_t nbytes;
  uint64_t* flag; /* mapped pinned host memory or device memory; may be NULL */
  uint64_t flag_value;
  uint64_t* flag2; /* a second word published with the first (sender-side completion of a push); may be NULL */
  uint64_t flag2_value;
} eux_pull_item;
EUX_API int eux_xfer_pull_batch_launch(const eux_pull_item* items, int n, void* stream);

/* Device-driven ping-pong between two GPUs (or loopback on one): see
 * tensor_xfer.cu. ts_out receives iters+1 globaltimer stamps (ns). */
typedef struct eux_pingpong_desc {
  void* local_buf;       /* this side's send+recv buffer (nbytes) */
  void* peer_buf;        /* the other side's buffer, peer-mapped */
  uint64_t nbytes;       /* multiple of 16 */
  uint64_t* local_flag;  /* written by the other side */
  uint64_t* peer_flag;   /* the other side's local_flag, peer-mapped */
  uint32_t* grid_bar;    /* scratch: 2 zeroed uint32 for the in-kernel grid barrier */
  uint64_t* ts_out;      /* iters+1 stamps, may be NULL */
  uint32_t* status;
  int32_t iters;
  int32_t initiator;     /* 1: send first; 0: echo */
  uint64_t base_seq;     /* flags count up from base_seq+1 */
  uint64_t wait_timeout_ns;
} eux_pingpong_desc;
EUX_API int eux_pingpong_launch(const eux_pingpong_desc* d, int ctas, void* stream);

/* ---- memory export for peer mapping (used by the memory resource) ---- */
EUX_API int eux_ipc_export(void* dev_ptr, unsigned char handle_out[64]);
EUX_API int eux_ipc_open(const unsigned char handle[64], void** dev_ptr_out);
EUX_API int eux_ipc_close(void* dev_ptr);
EUX_API int eux_enable_peer_access(int this_dev, int peer_dev);
EUX_API int eux_device_malloc(void** p, size_t bytes);
EUX_API int eux_device_free(void* p);
EUX_API int eux_host_alloc_mapped(void** host_ptr, void** dev_ptr, size_t bytes);
EUX_API int eux_host_free(void* host_ptr);
EUX_API const char* eux_error_string(int err);
/* Load the kernels of a family on the current device now, so that no later launch has to (a first launch that
 * loads can deadlock against a running kernel that waits for a peer: see tensor_xfer.cu). */
EUX_API int eux_xfer_preload(void);
EUX_API int eux_moe_preload(void);
EUX_API int eux_gemm_preload(void);
/* cudaMemcpyPeerAsync, for the copy-engine baseline of the benchmarks (not used by the data plane) */
EUX_API int eux_memcpy_peer_async(void* dst, int dst_device, const void* src, int src_device, size_t bytes, void* stream);

/* ---- MoE dispatch / combine (moe_dispatch.cu) ---- */
typedef struct eux_moe_desc {
  int32_t rank, world;        /* this rank / number of ranks */
  int32_t n_tokens;           /* tokens on this rank */
  int32_t hidden;             /* elements per token (multiple of 128) */
  int32_t topk;
  int32_t n_experts;          /* global; experts_per_rank = n_experts / world */
  int32_t fp8;                /* 0: bf16 rows; 1: e4m3 rows + hidden/128 fp32 scales */
  int32_t capacity;           /* rows per (src,dst) region of a receive arena */
  const void* x;              /* [n_tokens, hidden] bf16 */
  const int32_t* topk_idx;    /* [n_tokens, topk] global expert id */
  const float* topk_w;        /* [n_tokens, topk] gate weights */
  void* const* arena_peer;    /* device array [world]: base of every rank's receive arena */
  uint64_t* const* meta_peer; /* device array [world]: row headers, 16 B each */
  uint64_t* const* flag_peer; /* device array [world]: [world] arrival flags + [world] counts */
  int32_t* slot_of;           /* [n_tokens, topk] scratch+output: slot inside (src,dst) region */
  int32_t* counters;          /* scratch [world + n_experts + 8] zero on entry, zero on exit */
  void* out;                  /* combine output [n_tokens, hidden] bf16 */
  uint64_t seq;               /* flag value of this dispatch/combine exchange (monotonic) */
  uint64_t wait_timeout_ns;
  uint32_t* status;
} eux_moe_desc;
EUX_API size_t eux_moe_row_bytes(int hidden, int fp8);
EUX_API int eux_moe_dispatch_launch(const eux_moe_desc* d, int ctas, void* stream);
EUX_API int eux_moe_expert_ready_launch(const eux_moe_desc* d, void* stream);
EUX_API int eux_moe_combine_launch(const eux_moe_desc* d, int ctas, void* stream);

/* ---- remote GEMM (remote_gemm.cu): Y[M,N] = X[M,K] * W[K,N] ---- */
typedef struct eux_gemm_desc {
  const void* x_src;   /* caller's X (may be peer memory), row-major [M,K] */
  void* x_stage;       /* local staging copy of X, [M,K]; == x_src when X is already local */
  const void* w_t;     /* resident weight, stored [N,K] (K-major), local */
  void* y_dst;         /* result [M,N] bf16 (may be peer memory) */
  const float* x_scale; /* fp8: [M, K/128] (may be peer) */
  float* x_scale_stage; /* fp8: local staging of x_scale */
  const float* w_scale; /* fp8: [N/128, K/128] local */
  int32_t M, N, K;
  int32_t fp8;
  uint32_t* panel_flags; /* scratch [M/128] zero on entry; kernel re-zeroes */
  uint32_t* sched;       /* scratch [4] zero on entry; kernel re-zeroes */
  uint64_t* done_flag;   /* release-stored when Y is complete (may be peer) */
  uint64_t done_value;
  uint64_t wait_timeout_ns;
  uint32_t* status;
  int32_t copy_ctas;     /* CTAs that stream X from the peer; 0 when x_stage == x_src */
  int32_t flags;         /* EUX_GEMM_FLAG_* */
} eux_gemm_desc;
/* bf16 with M % 256 == 0: tiles of 256 x 256 computed by pairs of CTAs (cta_group::2) */
#define EUX_GEMM_FLAG_CTA_PAIRS 1
/* With a remote X: two spare warps of every CTA copy X (and its scales) beside the GEMM's warps, instead of
   copy_ctas CTAs that copy first and compute afterwards. */
#define EUX_GEMM_FLAG_COPY_WARPS 2
/* Store done_value to done_flag when the kernel ends, whether or not it succeeded (the status word tells):
   for callers that must learn of the end either way. Without it the flag means "Y is complete". */
#define EUX_GEMM_FLAG_DONE_ALWAYS 4
/* With a remote X the first group of tiles is only a few row blocks tall, so that the first wave of
   CTAs waits for the first panels only. EUX_GEMM_FLAG_HEAD(n) overrides that height (0: no short group). */
#define EUX_GEMM_FLAG_HEAD(n) ((((n) + 1) & 0xff) << 8)
EUX_API int eux_gemm_launch(const eux_gemm_desc* d, void* stream);
EUX_API int eux_gemm_num_sms(void);

#ifdef __cplusplus
}
#endif
#endif /* EUX_KERNELS_H_ */
