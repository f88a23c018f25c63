/* Plain-C data model shared by every layer of the runtime: memory kinds, a
 * (pointer, length) buffer, an active message with one contiguous payload, an
 * active message with a scatter-gather payload, and a completion-queue entry.
 * Field names and enumerator order follow the reference's
 * ucx_context/ucx_context_def.h:27-158 so that code written against either
 * compiles against both. Nothing here depends on a transport library. */
#ifndef EUX_UCX_CONTEXT_DEF_H_
#define EUX_UCX_CONTEXT_DEF_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum ucx_memory_type {
  HOST,         /* ordinary system memory */
  CUDA,         /* cudaMalloc / cuMem device memory */
  CUDA_MANAGED, /* cudaMallocManaged memory */
  ROCM,
  ROCM_MANAGED,
  RDMA,
  ZE_HOST,
  ZE_DEVICE,
  ZE_MANAGED,
  LAST,
  UNKNOWN = LAST
} ucx_memory_type_t;

/* Same layout as a scatter-gather element {void*, size_t}: an array of these
 * can be handed to the transport as its iov list without conversion. */
typedef struct ucx_buffer {
  void* data;
  size_t size;
} ucx_buffer_t;

typedef ucx_buffer_t ucx_header_t;

typedef struct ucx_am_data {
  ucx_buffer_t header;           /* always host memory */
  ucx_buffer_t buffer;           /* payload, memory kind given by buffer_type */
  ucx_memory_type_t buffer_type;
  void* mem_h;                   /* registration handle of the payload, may be NULL */
} ucx_am_data_t;

typedef struct ucx_am_iovec {
  ucx_buffer_t header;
  ucx_buffer_t* buffer_vec;
  size_t buffer_count;
  ucx_memory_type_t buffer_type;
  void* mem_h;
} ucx_am_iovec_t;

typedef struct ucx_am_cqe {
  size_t user_data; /* submitter's cookie (a pointer to its completion state) */
  int res;          /* status of the finished operation */
  int flags;
} ucx_am_cqe_t;

#ifdef __cplusplus
}
#endif
#endif /* EUX_UCX_CONTEXT_DEF_H_ */
