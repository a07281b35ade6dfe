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

}  // namespace sm100
}  // namespace ksb
