// Packing many small tensors into one contiguous bucket (and back) with one launch.
//
// Data-parallel gradient averaging reduces buckets, not parameters: the gradients of a bucket are
// gathered into one slice of the symmetric working buffer, all-reduced in place, and scattered
// back.  Doing the gather with one copy kernel per parameter costs a launch (a few microseconds)
// per parameter on each side of the collective; here a whole batch of (tensor, offset, size)
// triples travels in the kernel's parameter space and one grid moves all of them.  The scatter can
// apply a scale (the 1/W of an average) and convert on the fly, so no separate scaling kernel runs.
// The reference has no bucketing (it ships collectives only).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../common/util.h"
#include "../engine/cuda_driver.h"
#include "gemm_host.h"

namespace pccl {
namespace gemm {

namespace {

__global__ void __launch_bounds__(256) bucket_pack_kernel(const PackBatch batch, uint8_t* bucket, int unpack) {
  const PackEntry e = batch.entry[blockIdx.y];
  uint8_t* tensor = static_cast<uint8_t*>(e.tensor);
  uint8_t* slot = bucket + e.bucket_offset;
  const uint8_t* src = unpack ? slot : tensor;
  uint8_t* dst = unpack ? tensor : slot;
  const uint64_t tid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const uint64_t nthreads = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
  if (aligned) {
    const uint64_t vecs = e.bytes / 16;
    for (uint64_t i = tid; i < vecs; i += nthreads)
      reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    for (uint64_t b = vecs * 16 + tid; b < e.bytes; b += nthreads) dst[b] = src[b];
  } else {
    // Offsets inside a bucket follow the element counts, so odd-sized tensors shift their
    // successors off the 16-byte grid: those move in 2-byte units (every supported dtype is
    // at least that wide, and offsets are multiples of the element size).
    if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | e.bytes) & 1u) == 0) {
      const uint64_t halves = e.bytes / 2;
      for (uint64_t i = tid; i < halves; i += nthreads)
        reinterpret_cast<uint16_t*>(dst)[i] = reinterpret_cast<const uint16_t*>(src)[i];
    } else {
      for (uint64_t b = tid; b < e.bytes; b += nthreads) dst[b] = src[b];
    }
  }
}

}  // namespace

void bucket_pack(const PackEntry* entries, int count, void* bucket, bool unpack, cudaStream_t stream) {
  for (int first = 0; first < count; first += kPackBatch) {
    PackBatch batch{};
    const int n = count - first < kPackBatch ? count - first : kPackBatch;
    uint64_t largest = 0;
    for (int i = 0; i < n; ++i) {
      batch.entry[i] = entries[first + i];
      if (batch.entry[i].bytes > largest) largest = batch.entry[i].bytes;
    }
    // grid.y = tensors of the batch, grid.x = enough CTAs for the largest of them (4 KB per CTA and pass).
    unsigned gx = static_cast<unsigned>((largest + 256 * 16 * 4 - 1) / (256 * 16 * 4));
    if (gx < 1) gx = 1;
    if (gx > 64) gx = 64;
    bucket_pack_kernel<<<dim3(gx, static_cast<unsigned>(n)), 256, 0, stream>>>(batch, static_cast<uint8_t*>(bucket),
                                                                              unpack ? 1 : 0);
    PCCL_CUDA(cudaGetLastError());
  }
}

}  // namespace gemm
}  // namespace pccl
