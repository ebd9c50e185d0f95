// Host-side entry points of the tcgen05 GEMM family (no torch dependency).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace pccl {
namespace gemm {

// Lazily allocated device word that kernels of this family write on a timeout
// (0 = ok).  read_error() synchronises the device.
uint32_t* error_word();
uint32_t read_error();
void clear_error();

struct MatrixDesc {
  const void* ptr;       // bf16, row-major
  int rows, cols;        // cols is the contiguous (K) dimension
  int64_t ld;            // elements between rows (multiple of 8)
};

// C[M,N] (bf16, row-major, leading dimension ldc) = A[M,K] * B[N,K]^T.
// `ctas` = 0 uses one CTA per SM.  Throws pccl::Error on invalid arguments.
void gemm_bf16_nt(const MatrixDesc& a, const MatrixDesc& b, void* c, int64_t ldc, cudaStream_t stream,
                  int ctas = 0, uint64_t timeout_ms = 2000);

}  // namespace gemm
}  // namespace pccl
