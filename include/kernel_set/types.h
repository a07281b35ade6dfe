/*
 * Scalar types, status codes and dtype ids shared by every entry point.
 *
 * Replaces include/kernel_set/types.h:21-68 of the reference project. The
 * numeric values are part of the binary contract: every language binding of
 * the reference hard-codes them, so they must not move.
 *
 * Plain C, no CUDA headers: device buffers travel as void*, a stream as an
 * opaque pointer that is a cudaStream_t underneath (NULL = default stream).
 */
#ifndef KERNEL_SET_TYPES_H_
#define KERNEL_SET_TYPES_H_

#include <stddef.h>
#include <stdint.h>

#include "kernel_set/export.h"

KS_BEGIN_EXTERN_C

typedef void* ks_stream_t;

/* Return code of every ks_* function (reference types.h:24-34). */
typedef enum ks_status_t {
  KS_SUCCESS = 0,
  KS_ERROR_INVALID_ARGUMENT = 1,  /* NULL where a buffer is required, dims <= 0 */
  KS_ERROR_UNSUPPORTED_DTYPE = 2, /* dtype id outside what the op accepts       */
  KS_ERROR_UNSUPPORTED_SHAPE = 3, /* divisibility / range rule of the op broken */
  KS_ERROR_CUDA = 4,              /* the CUDA runtime reported an error         */
  KS_ERROR_NOT_IMPLEMENTED = 5,   /* declared feature without an implementation */
  KS_ERROR_OUT_OF_MEMORY = 6,     /* a device allocation failed                 */
  KS_ERROR_ARCH_UNSUPPORTED = 7,  /* current device is not compute capability 10.x */
  KS_ERROR_INTERNAL = 8           /* a kernel reported a broken invariant       */
} ks_status_t;

/* Element types (reference types.h:37-49). */
typedef enum ks_dtype_t {
  KS_DTYPE_F32 = 0,
  KS_DTYPE_F16 = 1,
  KS_DTYPE_BF16 = 2,
  KS_DTYPE_F8E4M3 = 3, /* OCP e4m3fn: no infinities, max finite 448 */
  KS_DTYPE_F8E5M2 = 4, /* OCP e5m2: max finite 57344                */
  KS_DTYPE_F64 = 5,
  KS_DTYPE_I64 = 6,
  KS_DTYPE_I32 = 7,
  KS_DTYPE_I8 = 8,
  KS_DTYPE_U8 = 9,
  KS_DTYPE_I4 = 10     /* two 4-bit codes per byte */
} ks_dtype_t;

/* Kept so that code written against the reference headers still compiles
 * (reference types.h:52-66); no entry point of this library takes them. */
typedef enum ks_activation_t {
  KS_ACT_NONE = 0,
  KS_ACT_RELU = 1,
  KS_ACT_GELU = 2,
  KS_ACT_GELU_TANH = 3,
  KS_ACT_SILU = 4
} ks_activation_t;

typedef enum ks_quant_mode_t {
  KS_QUANT_PER_TENSOR = 0,
  KS_QUANT_PER_TOKEN = 1,
  KS_QUANT_PER_CHANNEL = 2,
  KS_QUANT_GROUPWISE = 3
} ks_quant_mode_t;

KS_END_EXTERN_C

#endif /* KERNEL_SET_TYPES_H_ */
