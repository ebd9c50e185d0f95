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

// Every rank's symmetric heap base as mapped into this process, plus rank / world.
struct PeerBases {
  uint8_t* base[8];
  int rank, world;
};

// Fused tensor-parallel GEMM -> reduce-scatter.  x[M, K_local], w[N, K_local] local bf16;
// out[M / world, N] local bf16.  recv_off / flags_off are symmetric-heap offsets of
// recv[2][world][M / world][N] bf16 and flags[world][M / world / 128] u32 (zeroed once, before
// the first call, on every rank); block_counter is a local zero-initialised u32[M / 128].
// epoch = 1, 2, 3, ... must advance by one per call on every rank.
void gemm_reduce_scatter(const PeerBases& peers, const MatrixDesc& x, const MatrixDesc& w, uint64_t recv_off,
                         uint64_t flags_off, uint32_t* block_counter, void* out, int64_t ldo, uint32_t epoch,
                         cudaStream_t stream, int ctas = 0, uint64_t timeout_ms = 2000);

// Fused all-gather -> GEMM.  The gathered activations live at heap offset gathered_off on every
// rank ([M, K] bf16, M = world * rows_per_rank); each rank has written its own row shard there
// before the call.  w[N_local, K] local bf16, out[M, N_local] local bf16.  flags_off: symmetric
// u32[2 * world]; ready: local zero-initialised u32[M / 128].
void all_gather_gemm(const PeerBases& peers, uint64_t gathered_off, int M, int K, const MatrixDesc& w,
                     uint64_t flags_off, uint32_t* ready, void* out, int64_t ldc, uint32_t epoch,
                     cudaStream_t stream, int copy_ctas = 20, int ctas = 0, uint64_t timeout_ms = 2000);

// Fused all-reduce + residual add + RMSNorm.  x, y and the residual h are [tokens][hidden] bf16
// at the given symmetric-heap offsets on every rank; flags_off: symmetric u32[2 * world] (zeroed
// once); cta_counter: local zero-initialised u32; mc_base: multicast alias of the heap or null.
void ar_residual_rmsnorm(const PeerBases& peers, uint8_t* mc_base, uint64_t x_off, uint64_t y_off, uint64_t res_off,
                         uint64_t flags_off, const void* gamma, uint32_t* cta_counter, int tokens, int hidden,
                         float eps, uint32_t epoch, cudaStream_t stream, int ctas = 0, uint64_t timeout_ms = 2000);

}  // namespace gemm
}  // namespace pccl
