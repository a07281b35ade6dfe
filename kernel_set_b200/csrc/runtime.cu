// Implementation of the runtime ABI (device / stream / memory helpers,
// introspection) and of the error plumbing shared by all entry points.
//
// Counterpart of kernels/src/common/runtime.cu:26-181 of the reference
// project: same 17 symbols and status behaviour (a failing CUDA call maps to
// KS_ERROR_CUDA with "<function>: <cuda message>", a failed device allocation
// to KS_ERROR_OUT_OF_MEMORY).
#include <mutex>

#include "common.cuh"
#include "kernel_set/runtime.h"
#include "sm100_host.cuh"

namespace ksb {

namespace {
thread_local std::string tls_error;

constexpr int kMaxDevices = 64;
struct DeviceInfo {
  bool known = false;
  int major = 0, minor = 0, sms = 0;
  unsigned int* fault_host = nullptr;  // host-mapped word written by kernels
  unsigned int* fault_dev = nullptr;
  bool fault_tried = false;
};
DeviceInfo g_dev[kMaxDevices];
std::mutex g_dev_mutex;

DeviceInfo* current_device_info() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  DeviceInfo& d = g_dev[dev];
  if (!d.known) {
    if (cudaDeviceGetAttribute(&d.major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return nullptr;
    cudaDeviceGetAttribute(&d.minor, cudaDevAttrComputeCapabilityMinor, dev);
    cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
    d.known = true;
  }
  return &d;
}
}  // namespace

void set_last_error(const std::string& msg) { tls_error = msg; }
const char* last_error_cstr() { return tls_error.c_str(); }

ks_status_t cuda_status(cudaError_t e, const char* where) {
  if (e == cudaSuccess) return KS_SUCCESS;
  set_last_error(std::string(where) + ": " + cudaGetErrorString(e));
  return KS_ERROR_CUDA;
}

ks_status_t require_sm100(const char* where) {
  DeviceInfo* d = current_device_info();
  if (d == nullptr) {
    cudaGetLastError();
    KSB_FAIL(KS_ERROR_CUDA, std::string(where) + ": no usable CUDA device");
  }
  if (d->major != 10)
    KSB_FAIL(KS_ERROR_ARCH_UNSUPPORTED,
             std::string(where) + ": this library is built for sm_100a only (device is sm_" +
                 std::to_string(d->major) + std::to_string(d->minor) + ")");
  return KS_SUCCESS;
}

int sm_count() {
  DeviceInfo* d = current_device_info();
  return (d != nullptr && d->sms > 0) ? d->sms : 148;
}

unsigned int* kernel_fault_word() {
  DeviceInfo* d = current_device_info();
  if (d == nullptr) return nullptr;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (!d->fault_tried) {
    d->fault_tried = true;
    void* h = nullptr;
    if (cudaHostAlloc(&h, 64, cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess) {
      *static_cast<volatile unsigned int*>(h) = 0u;
      void* dp = nullptr;
      if (cudaHostGetDevicePointer(&dp, h, 0) == cudaSuccess) {
        d->fault_host = static_cast<unsigned int*>(h);
        d->fault_dev = static_cast<unsigned int*>(dp);
      } else {
        cudaFreeHost(h);
      }
    }
    cudaGetLastError();
  }
  return d->fault_dev;
}

unsigned int* kernel_fault_word_if_ready() {
  DeviceInfo* d = current_device_info();
  if (d == nullptr) return nullptr;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  return d->fault_dev;
}

ks_status_t poll_kernel_fault(const char* where) {
  DeviceInfo* d = current_device_info();
  if (d == nullptr || d->fault_host == nullptr) return KS_SUCCESS;
  const unsigned int code = *static_cast<volatile unsigned int*>(d->fault_host);
  if (code == 0u) return KS_SUCCESS;
  *static_cast<volatile unsigned int*>(d->fault_host) = 0u;
  // a kernel that stopped half-way may have left split-K arrival counters non-zero
  sm100::stream_scratch_mark_dirty(1);
  char buf[160];
  snprintf(buf, sizeof(buf),
           "%s: an earlier kernel on this device gave up on a bounded wait (code 0x%08x)",
           where, code);
  KSB_FAIL(KS_ERROR_INTERNAL, buf);
}

}  // namespace ksb

using ksb::as_stream;
using ksb::cuda_status;

extern "C" {

const char* ks_version(void) { return "0.2.1+b200"; }
const char* ks_backend_name(void) { return "cuda"; }
const char* ks_last_error_string(void) { return ksb::last_error_cstr(); }

const char* ks_status_string(ks_status_t status) {
  static const char* const names[] = {
      "KS_SUCCESS",           "KS_ERROR_INVALID_ARGUMENT", "KS_ERROR_UNSUPPORTED_DTYPE",
      "KS_ERROR_UNSUPPORTED_SHAPE", "KS_ERROR_CUDA",       "KS_ERROR_NOT_IMPLEMENTED",
      "KS_ERROR_OUT_OF_MEMORY", "KS_ERROR_ARCH_UNSUPPORTED", "KS_ERROR_INTERNAL"};
  const int s = static_cast<int>(status);
  return (s >= 0 && s <= 8) ? names[s] : "KS_ERROR_UNKNOWN";
}

int ks_dtype_size_bits(ks_dtype_t dtype) {
  static const int bits[] = {32, 16, 16, 8, 8, 64, 64, 32, 8, 8, 4};
  const int d = static_cast<int>(dtype);
  return (d >= 0 && d <= 10) ? bits[d] : 0;
}

const char* ks_dtype_name(ks_dtype_t dtype) {
  static const char* const names[] = {"f32", "f16", "bf16", "f8e4m3", "f8e5m2", "f64",
                                      "i64", "i32", "i8",   "u8",     "i4"};
  const int d = static_cast<int>(dtype);
  return (d >= 0 && d <= 10) ? names[d] : "unknown";
}

ks_status_t ks_device_count(int* out_count) {
  KSB_REQUIRE_PTR(out_count);
  return cuda_status(cudaGetDeviceCount(out_count), "ks_device_count");
}

ks_status_t ks_set_device(int device) {
  return cuda_status(cudaSetDevice(device), "ks_set_device");
}

ks_status_t ks_get_device(int* out_device) {
  KSB_REQUIRE_PTR(out_device);
  return cuda_status(cudaGetDevice(out_device), "ks_get_device");
}

ks_status_t ks_get_device_properties(int device, ks_device_properties_t* out_props) {
  KSB_REQUIRE_PTR(out_props);
  cudaDeviceProp p;
  ks_status_t st = cuda_status(cudaGetDeviceProperties(&p, device), "ks_get_device_properties");
  if (st != KS_SUCCESS) return st;
  size_t i = 0;
  for (; i + 1 < sizeof(out_props->name) && p.name[i] != '\0'; ++i) out_props->name[i] = p.name[i];
  out_props->name[i] = '\0';
  out_props->compute_major = p.major;
  out_props->compute_minor = p.minor;
  out_props->multiprocessor_count = p.multiProcessorCount;
  out_props->max_threads_per_block = p.maxThreadsPerBlock;
  out_props->max_shared_memory_per_block = static_cast<int>(p.sharedMemPerBlock);
  out_props->warp_size = p.warpSize;
  out_props->total_global_memory = p.totalGlobalMem;
  const int cc = p.major * 10 + p.minor;
  out_props->supports_bf16 = cc >= 80;
  out_props->supports_tf32 = cc >= 80;
  out_props->supports_fp8 = cc >= 89;
  return KS_SUCCESS;
}

ks_status_t ks_stream_create(ks_stream_t* out_stream) {
  KSB_REQUIRE_PTR(out_stream);
  cudaStream_t s = nullptr;
  ks_status_t st = cuda_status(cudaStreamCreate(&s), "ks_stream_create");
  if (st == KS_SUCCESS) *out_stream = static_cast<ks_stream_t>(s);
  return st;
}

ks_status_t ks_stream_destroy(ks_stream_t stream) {
  // library-owned workspace of this stream goes with it (a later stream may reuse the handle value)
  ksb::sm100::stream_scratch_release(as_stream(stream));
  return cuda_status(cudaStreamDestroy(as_stream(stream)), "ks_stream_destroy");
}

ks_status_t ks_stream_synchronize(ks_stream_t stream) {
  ks_status_t st = cuda_status(cudaStreamSynchronize(as_stream(stream)), "ks_stream_synchronize");
  if (st != KS_SUCCESS) return st;
  return ksb::poll_kernel_fault("ks_stream_synchronize");
}

ks_status_t ks_malloc_device(void** out_ptr, size_t bytes) {
  KSB_REQUIRE_PTR(out_ptr);
  cudaError_t e = cudaMalloc(out_ptr, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    KSB_FAIL(KS_ERROR_OUT_OF_MEMORY, std::string("ks_malloc_device: ") + cudaGetErrorString(e));
  }
  return KS_SUCCESS;
}

ks_status_t ks_free_device(void* ptr) {
  return cuda_status(cudaFree(ptr), "ks_free_device");
}

ks_status_t ks_memcpy(void* dst, const void* src, size_t bytes, ks_memcpy_kind_t kind,
                      ks_stream_t stream) {
  KSB_REQUIRE_PTR(dst);
  KSB_REQUIRE_PTR(src);
  cudaMemcpyKind k = cudaMemcpyDeviceToDevice;
  if (kind == KS_MEMCPY_HOST_TO_DEVICE) k = cudaMemcpyHostToDevice;
  if (kind == KS_MEMCPY_DEVICE_TO_HOST) k = cudaMemcpyDeviceToHost;
  return cuda_status(cudaMemcpyAsync(dst, src, bytes, k, as_stream(stream)), "ks_memcpy");
}

ks_status_t ks_memset_device(void* dst, int value, size_t bytes, ks_stream_t stream) {
  KSB_REQUIRE_PTR(dst);
  return cuda_status(cudaMemsetAsync(dst, value, bytes, as_stream(stream)), "ks_memset_device");
}

}  // extern "C"
