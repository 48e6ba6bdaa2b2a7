// Library-owned device scratch (split-K partial sums, padded / transposed operand copies, column
// partial sums, arg-max planes).  One buffer per (device, stream, tag): kernels that run concurrently
// on different streams never share one.  A buffer grows on demand; the one it replaces is parked, not
// freed (cudaFree synchronises the whole device in the middle of a step), until tsb_scratch_trim() is
// called from a quiet point.  Every byte obtained here is counted, so a trainer that caps its
// activation pool can report what lives outside the cap (tsb_scratch_bytes).
//
// Role in the reference: the cuDNN workspaces its accounting allocator hands out and charges to the
// budget (src/ops/CudnnConv2d.cu:184-198, src/cuda_common/reuse_gpu_memory_manager.cc:24-65).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace tsb_scratch {

enum Tag {
  CONV_SPLITK = 0, CONV_FILTER_T = 1, CONV_UPSAMPLE = 2,
  GEMM_SPLITK = 10, GEMM_PAD_A = 11, GEMM_PAD_B = 12,
  NORM_PARTIALS = 20, POOL_ARGMAX = 30, LOSS_ROWS = 31, COLSUM_PARTIALS = 40,
};

// At least `bytes` (and at least `floor_bytes` when a new buffer has to be obtained); nullptr when the
// device is out of memory.  The pointer stays valid until the next larger request with the same key.
void* get(cudaStream_t stream, int tag, size_t bytes, size_t floor_bytes = 0);

}  // namespace tsb_scratch

extern "C" {
// Bytes of device memory the library currently holds as scratch on all devices (parked buffers included).
long long tsb_scratch_bytes();
// Frees the parked buffers.  Call only when no kernel of this library is in flight; returns bytes freed.
long long tsb_scratch_trim();
}
