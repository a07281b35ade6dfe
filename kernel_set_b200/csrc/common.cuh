// Shared host/device plumbing for every translation unit of the library:
// the thread-local error string behind ks_last_error_string(), the status
// helpers every entry point uses, and fp32 <-> storage-type conversion.
//
// Plays the role of kernels/src/common/{dispatch,dtype,platform}.cuh of the
// reference project (status macros dispatch.cuh:32-50; conversions
// dtype.cuh:43-52), written for one backend (CUDA, sm_100a) only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "kernel_set/types.h"

namespace ksb {

// ---- error plumbing --------------------------------------------------------
void set_last_error(const std::string& msg);
const char* last_error_cstr();

// Records `where: <cuda message>` and maps any CUDA error to KS_ERROR_CUDA.
ks_status_t cuda_status(cudaError_t e, const char* where);

// Returns KS_SUCCESS when the current device is compute capability 10.x,
// KS_ERROR_ARCH_UNSUPPORTED (with a message) otherwise. Cached per device.
ks_status_t require_sm100(const char* where);

// Number of SMs of the current device (cached per device).
int sm_count();

// A kernel that gives up on a bounded wait writes a non-zero code into a
// host-mapped word; the next entry point on that device reports it here.
ks_status_t poll_kernel_fault(const char* where);
// Device-visible address of that word for the current device (NULL on failure).
unsigned int* kernel_fault_word();
// The same address if an earlier call already set the word up, else NULL.
// Never allocates (the set-up in kernel_fault_word() pins a host page).
unsigned int* kernel_fault_word_if_ready();

inline cudaStream_t as_stream(ks_stream_t s) {
  return static_cast<cudaStream_t>(s);
}

#define KSB_FAIL(status, msg)          \
  do {                                 \
    ::ksb::set_last_error(msg);        \
    return (status);                   \
  } while (0)

#define KSB_REQUIRE_PTR(p)                                              \
  do {                                                                  \
    if ((p) == nullptr)                                                 \
      KSB_FAIL(KS_ERROR_INVALID_ARGUMENT, "null arg: " #p);             \
  } while (0)

#define KSB_CHECK_LAUNCH(where)                                         \
  do {                                                                  \
    ks_status_t st_ = ::ksb::cuda_status(cudaGetLastError(), (where));  \
    if (st_ != KS_SUCCESS) return st_;                                  \
  } while (0)

// ---- storage type <-> fp32 -------------------------------------------------
// Every conversion to a narrower type is round-to-nearest-even; conversions
// to fp8 saturate to the largest finite value (cvt.rn.satfinite).
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_fp8_e4m3>(__nv_fp8_e4m3 v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float to_f32<__nv_fp8_e5m2>(__nv_fp8_e5m2 v) { return static_cast<float>(v); }

template <> __device__ __forceinline__ float to_f32<int8_t>(int8_t v) { return static_cast<float>(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __nv_fp8_e4m3 from_f32<__nv_fp8_e4m3>(float v) { return __nv_fp8_e4m3(v); }
template <> __device__ __forceinline__ __nv_fp8_e5m2 from_f32<__nv_fp8_e5m2>(float v) { return __nv_fp8_e5m2(v); }

inline bool is_fp8(ks_dtype_t d) { return d == KS_DTYPE_F8E4M3 || d == KS_DTYPE_F8E5M2; }
inline bool is_float3(ks_dtype_t d) { return d == KS_DTYPE_F32 || d == KS_DTYPE_F16 || d == KS_DTYPE_BF16; }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace ksb
