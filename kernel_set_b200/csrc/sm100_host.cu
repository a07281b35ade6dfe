#include "sm100_host.cuh"

#include <cstdlib>

#include <map>
#include <mutex>
#include <utility>

namespace ksb {
namespace sm100 {
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    cudaGetLastError();
  });
  return fn;
}

struct Scratch {
  void* ptr = nullptr;
  size_t bytes = 0;
  bool dirty = false;
};
std::mutex g_scratch_mutex;
std::map<std::pair<std::pair<int, cudaStream_t>, int>, Scratch> g_scratch;

}  // namespace

bool tma_available() { return encode_fn() != nullptr; }

bool tma_encode(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
                const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr || rank < 2 || rank > 3) return false;
  cuuint64_t gdim[3];
  cuuint64_t gstr[2];
  cuuint32_t bdim[3];
  cuuint32_t estr[3] = {1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
  }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  return fn(map, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstr, bdim, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

void* stream_scratch(cudaStream_t stream, size_t bytes, int kind) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  Scratch& s = g_scratch[std::make_pair(std::make_pair(dev, stream), kind)];
  if (s.bytes >= bytes && s.ptr != nullptr) return s.ptr;
  const size_t floor_bytes = kind == 0 ? (size_t(1) << 20) : (size_t(64) << 10);
  size_t want = bytes < floor_bytes ? floor_bytes : bytes;
  want = (want + 0xFFFF) & ~size_t(0xFFFF);
  void* fresh = nullptr;
  if (cudaMallocAsync(&fresh, want, stream) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  if (cudaMemsetAsync(fresh, 0, want, stream) != cudaSuccess) {
    cudaGetLastError();
    cudaFreeAsync(fresh, stream);
    return nullptr;
  }
  if (s.ptr != nullptr) cudaFreeAsync(s.ptr, stream);
  s.ptr = fresh;
  s.bytes = want;
  return fresh;
}

size_t stream_scratch_bytes(cudaStream_t stream, int kind) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  auto it = g_scratch.find(std::make_pair(std::make_pair(dev, stream), kind));
  return it == g_scratch.end() ? 0 : it->second.bytes;
}

void stream_scratch_mark_dirty(int kind) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  for (auto& kv : g_scratch)
    if (kv.first.first.first == dev && kv.first.second == kind) kv.second.dirty = true;
}

bool stream_scratch_take_dirty(cudaStream_t stream, int kind) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  auto it = g_scratch.find(std::make_pair(std::make_pair(dev, stream), kind));
  if (it == g_scratch.end() || !it->second.dirty) return false;
  it->second.dirty = false;
  return true;
}

void stream_scratch_release(cudaStream_t stream) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  for (auto it = g_scratch.begin(); it != g_scratch.end();) {
    if (it->first.first.first == dev && it->first.first.second == stream) {
      if (it->second.ptr != nullptr) cudaFreeAsync(it->second.ptr, stream);
      it = g_scratch.erase(it);
    } else {
      ++it;
    }
  }
  cudaGetLastError();
}

bool programmatic_launch_enabled() {
  static const bool enabled = std::getenv("KS_B200_NO_PDL") == nullptr;
  return enabled;
}

}  // namespace sm100
}  // namespace ksb
