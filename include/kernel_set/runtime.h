/*
 * Device, stream and memory helpers for bindings that have no GPU library of
 * their own, plus library introspection and the thread-local error string.
 *
 * Replaces include/kernel_set/runtime.h:20-80 of the reference project
 * (implemented there in kernels/src/common/runtime.cu:26-181). Same 17
 * symbols, same argument order, same status behaviour.
 */
#ifndef KERNEL_SET_RUNTIME_H_
#define KERNEL_SET_RUNTIME_H_

#include "kernel_set/types.h"

KS_BEGIN_EXTERN_C

/* -- introspection (reference runtime.h:20-35) --------------------------- */
KS_API const char* ks_version(void);                      /* "0.2.1+b200"   */
KS_API const char* ks_status_string(ks_status_t status);  /* never NULL     */
KS_API int ks_dtype_size_bits(ks_dtype_t dtype);          /* I4 -> 4, unknown -> 0 */
KS_API const char* ks_dtype_name(ks_dtype_t dtype);       /* "bf16", "f8e4m3", ... */
KS_API const char* ks_backend_name(void);                 /* always "cuda"  */

/* -- device queries (reference runtime.h:39-58) -------------------------- */
typedef struct ks_device_properties_t {
  char name[256];
  int compute_major;
  int compute_minor;
  int multiprocessor_count;
  int max_threads_per_block;
  int max_shared_memory_per_block; /* bytes, the non-opt-in limit */
  int warp_size;
  size_t total_global_memory;      /* bytes */
  int supports_bf16;
  int supports_fp8;
  int supports_tf32;
} ks_device_properties_t;

KS_API ks_status_t ks_device_count(int* out_count);
KS_API ks_status_t ks_set_device(int device);
KS_API ks_status_t ks_get_device(int* out_device);
KS_API ks_status_t ks_get_device_properties(int device,
                                            ks_device_properties_t* out_props);

/* Message recorded by the last failing ks_* call on the calling thread.
 * Stays valid until that thread's next ks_* call. Never NULL. */
KS_API const char* ks_last_error_string(void);

/* -- streams (reference runtime.h:62-64) --------------------------------- */
KS_API ks_status_t ks_stream_create(ks_stream_t* out_stream);
KS_API ks_status_t ks_stream_destroy(ks_stream_t stream);
KS_API ks_status_t ks_stream_synchronize(ks_stream_t stream);

/* -- device memory (reference runtime.h:68-80) --------------------------- */
KS_API ks_status_t ks_malloc_device(void** out_ptr, size_t bytes);
KS_API ks_status_t ks_free_device(void* ptr);

typedef enum ks_memcpy_kind_t {
  KS_MEMCPY_HOST_TO_DEVICE = 0,
  KS_MEMCPY_DEVICE_TO_HOST = 1,
  KS_MEMCPY_DEVICE_TO_DEVICE = 2
} ks_memcpy_kind_t;

/* Both are stream-ordered and return before the copy/fill has finished. */
KS_API ks_status_t ks_memcpy(void* dst, const void* src, size_t bytes,
                             ks_memcpy_kind_t kind, ks_stream_t stream);
KS_API ks_status_t ks_memset_device(void* dst, int value, size_t bytes,
                                    ks_stream_t stream);

KS_END_EXTERN_C

#endif /* KERNEL_SET_RUNTIME_H_ */
