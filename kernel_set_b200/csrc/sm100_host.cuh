// Host-side helpers shared by the sm_100a kernels: TMA tensor-map encoding
// through the driver entry point (no link-time dependency on libcuda) and a
// per-(device, stream) scratch allocation for kernels that need workspace.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ksb {
namespace sm100 {

// True when cuTensorMapEncodeTiled could be resolved.
bool tma_available();

// Encodes a tiled tensor map of rank 2 or 3 (dimension 0 innermost).
// strides_bytes has rank-1 entries (strides of dimensions 1..rank-1, multiples
// of 16 bytes); base must be 16-byte aligned; box[0] * element size must be a
// multiple of 16 bytes and, with a swizzle, at most the swizzle span.
bool tma_encode(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
                const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle);

// Library-owned scratch memory for the current device, the given stream and the given
// purpose (`kind`: buffers of different kinds never share memory), at least `bytes` large
// and zero-filled when (re)allocated. The pointer stays valid until a later call asks for
// more of the same kind on the same (device, stream); growth is stream-ordered
// (cudaMallocAsync / cudaFreeAsync), so work already queued on the stream keeps its buffer.
// Returns NULL when the allocation fails.
void* stream_scratch(cudaStream_t stream, size_t bytes, int kind = 0);
// Size of that buffer (0 when none exists).
size_t stream_scratch_bytes(cudaStream_t stream, int kind);
// Marks every buffer of `kind` on the current device as possibly modified by a kernel
// that stopped half-way; stream_scratch_take_dirty() reports and clears the mark of one
// (device, stream) buffer, whose owner then restores the buffer's invariant.
void stream_scratch_mark_dirty(int kind);
bool stream_scratch_take_dirty(cudaStream_t stream, int kind);
// Frees (stream-ordered) every buffer of the current device that belongs to `stream`;
// called when the stream is destroyed, so that a recycled handle starts clean.
void stream_scratch_release(cudaStream_t stream);

// Launches `kernel` with programmatic stream serialization: it may begin while the kernel
// before it on the stream is still running, once every CTA of that kernel has executed
// griddepcontrol.launch_dependents or exited (a kernel that never executes it is simply
// waited for, as in an ordinary launch). The launched kernel must order its own accesses
// with griddepcontrol.wait (grid_dependency_wait() in sm100_ptx.cuh).
// False when the environment variable KS_B200_NO_PDL is set (read once): launch_programmatic
// then launches the ordinary way.
bool programmatic_launch_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_programmatic(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem,
                                       cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = programmatic_launch_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace sm100
}  // namespace ksb
