// Host-side entry points of the tcgen05 GEMM family (no torch dependency).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <vector>

namespace pccl {
namespace gemm {

// Lazily allocated device word that kernels of this family write on a timeout
// (0 = ok).  read_error() synchronises the device.
uint32_t* error_word();
uint32_t read_error();
void clear_error();

// Timeline of the GEMM family's kernels (off by default): while enabled every CTA of a launch
// stamps %globaltimer at its milestones (see Problem::trace); gemm_trace_read returns the stamps
// of the most recent launch, 8 per CTA for up to 256 CTAs (synchronises).
void gemm_trace_enable(bool on);
std::vector<uint64_t> gemm_trace_read();

struct MatrixDesc {
  const void* ptr;       // bf16, row-major
  int rows, cols;        // cols is the contiguous (K) dimension
  int64_t ld;            // elements between rows (multiple of 8)
};

// C[M,N] (bf16, row-major, leading dimension ldc) = A[M,K] * B[N,K]^T.
// `ctas` = 0 uses one CTA per SM.  sms_per_tile: 2 = pairs of SMs work on 256 x 256 tiles with
// tcgen05.mma.cta_group::2, 1 = one SM per 128 x 256 tile, 0 = PCCL_GEMM_SMS_PER_TILE (default 2).
// Throws pccl::Error on invalid arguments.
void gemm_bf16_nt(const MatrixDesc& a, const MatrixDesc& b, void* c, int64_t ldc, cudaStream_t stream,
                  int ctas = 0, uint64_t timeout_ms = 2000, int sms_per_tile = 0);

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
// swiglu: w stacks gate and up rows interleaved in groups of 16 and out is [M, N_local / 2] =
// silu(gate) * up, computed in the epilogue.
void all_gather_gemm(const PeerBases& peers, uint64_t gathered_off, int M, int K, const MatrixDesc& w,
                     uint64_t flags_off, uint32_t* ready, void* out, int64_t ldc, uint32_t epoch,
                     cudaStream_t stream, int copy_ctas = 0, int ctas = 0, uint64_t timeout_ms = 2000,
                     bool swiglu = false);

// Fused all-reduce + residual add + RMSNorm.  x, y and the residual h are [tokens][hidden] bf16
// at the given symmetric-heap offsets on every rank; flags_off: symmetric u32[2 * world] (zeroed
// once); cta_counter: local zero-initialised u32; mc_base: multicast alias of the heap or null.
void ar_residual_rmsnorm(const PeerBases& peers, uint8_t* mc_base, uint64_t x_off, uint64_t y_off, uint64_t res_off,
                         uint64_t flags_off, const void* gamma, uint32_t* cta_counter, int tokens, int hidden,
                         float eps, uint32_t epoch, cudaStream_t stream, int ctas = 0, uint64_t timeout_ms = 2000);

// Small-message all-reduce (sum) with flag-carrying packets; in / out are ordinary device tensors
// (out may alias in).  buf_off: symmetric uint4 [2][world][capacity_bytes / 8], zeroed once before
// the first call on every rank.  dtype: 0 f32, 1 f16, 2 bf16.  epoch = 1, 2, 3, ... per call.
// error: device word this call aborts on and reports to (null = the family's shared word).
void allreduce_ll(const PeerBases& peers, uint64_t buf_off, uint64_t capacity_bytes, const void* in, void* out,
                  uint64_t bytes, int dtype, uint32_t epoch, cudaStream_t stream, uint64_t timeout_ms = 2000,
                  uint32_t* error = nullptr);

// The same packet protocol for the other collectives (sum where one is taken).  `bytes` is ONE RANK'S PART:
//   mode 1 reduce-scatter  in [world * bytes], out [bytes] = the sum of every rank's part `rank`
//   mode 2 all-gather      in [bytes],         out [world * bytes]
//   mode 3 all-to-all      in [world * bytes] (part p goes to rank p), out [world * bytes] (part s came from s)
//   mode 0 all-reduce      in, out [bytes] (allreduce_ll)
// All modes share buf_off and the call counter `epoch`: consecutive calls of any mode alternate the parity.
void collective_ll(int mode, const PeerBases& peers, uint64_t buf_off, uint64_t capacity_bytes, const void* in,
                   void* out, uint64_t bytes, int dtype, uint32_t epoch, cudaStream_t stream,
                   uint64_t timeout_ms = 2000, uint32_t* error = nullptr);

// Fused push collectives for small and medium messages; in / out are ordinary device tensors.
//   kPushAllReduce      sum; push reduce-scatter, reduce, push all-gather; out may alias in
//   kPushReduceScatter  sum; in [bytes], out [bytes / world] = this rank's slice
//   kPushAllGather      in [bytes / world], out [bytes]
//   kPushAllToAll       in [bytes] (part p goes to rank p), out [bytes] (part s came from rank s)
// `bytes` is the full message.  area_off: symmetric bytes [2][2][world][ceil(capacity / 16 / world) * 16];
// flags_off: symmetric u32[2 * world], zeroed once; counters: local zero-initialised u32[2].
// `ctas` must be the same for every call that shares the counters.
enum PushMode : int { kPushAllReduce = 0, kPushReduceScatter = 1, kPushAllGather = 2, kPushAllToAll = 3 };
// A reduce-scatter may alias its output with slice `rank` of its input (the in-place convention) and
// with nothing else of it: other ranks' slices are still being read while the output is written.
// error: device word this call aborts on and reports to (null = the family's shared word).
void collective_push(PushMode mode, const PeerBases& peers, uint64_t area_off, uint64_t capacity_bytes,
                     uint64_t flags_off, uint32_t* counters, const void* in, void* out, uint64_t bytes, int dtype,
                     uint32_t epoch, cudaStream_t stream, int ctas, uint64_t timeout_ms = 2000,
                     uint32_t* error = nullptr);

// Large-message all-reduce (sum) through the switch, in place on `bytes` at symmetric offset data_off
// (16-byte aligned; bytes a multiple of 16 * world).  mc_base: multicast alias of the heap (required).
// flags_off: symmetric u32[2 * world], zeroed once; cta_counter: local zero-initialised u32; `ctas` must be
// the same for every call that shares them.  dtype: 0 f32, 1 f16, 2 bf16.  epoch = 1, 2, 3, ... per call.
void allreduce_nvls(const PeerBases& peers, uint8_t* mc_base, uint64_t data_off, uint64_t bytes, int dtype,
                    uint64_t flags_off, uint32_t* cta_counter, uint32_t epoch, cudaStream_t stream, int ctas,
                    uint64_t timeout_ms = 2000, uint32_t* error = nullptr);

// ---- gradient buckets ------------------------------------------------------------------------------
// Gather `count` tensors into one bucket (or scatter them back, unpack = true) with one launch per
// kPackBatch tensors: the table travels in the kernel's parameters, no host-to-device copy.
struct PackEntry {
  void* tensor;             // device address of the tensor's first byte (contiguous)
  uint64_t bucket_offset;   // bytes from the bucket's start
  uint64_t bytes;
};
constexpr int kPackBatch = 128;
struct PackBatch { PackEntry entry[kPackBatch]; };
void bucket_pack(const PackEntry* entries, int count, void* bucket, bool unpack, cudaStream_t stream);

// ---- expert-parallel MoE feed-forward (top-2 routing) ------------------------------------------------
// Symmetric-heap offsets (identical on every rank) of the buffers the three kernels share.
// regions = (experts / world) * world, region = local_expert * world + source rank.
struct MoeBuffers {
  uint64_t recv_off;      // bf16 [regions][cap][hidden]: dispatched token rows
  uint64_t meta_off;      // uint2 [regions][cap]: {token * 2 + k, gate}
  uint64_t counts_off;    // u32 [regions]: rows filled (rewritten by every call)
  uint64_t ready_off;     // u32 [world]: dispatch flags, zeroed once
  uint64_t done_off;      // u32 [world]: expert-finished flags, zeroed once
  uint64_t comb_off;      // bf16 [tokens][2][hidden]: expert outputs back at the tokens' home rank
  int cap;                // rows per region, a multiple of 128 (>= tokens per rank: nothing is dropped)
};

// Router (+ dispatch).  x[tokens, hidden], wg[experts, hidden] local bf16.  scratch: local
// u32[experts + 1], cleared by this call on `stream`.  Optional outputs (null to skip):
// topk_idx / topk_gate / topk_slot [tokens, 2], expert_counts [experts].  With dispatch the
// rows, metadata and counts land in the expert ranks' buffers and the ready flag is posted.
// experts * hidden * 2 bytes of router weight must fit in shared memory (200 KB).
void moe_route_dispatch(const PeerBases& peers, const MoeBuffers& buf, const void* x, const void* wg, int tokens,
                        int hidden, int experts, uint32_t* scratch, int32_t* topk_idx, float* topk_gate,
                        int32_t* topk_slot, uint32_t* expert_counts, bool dispatch, uint32_t epoch,
                        cudaStream_t stream);

// Expert GEMM 1 with the SwiGLU epilogue: h[regions * cap, ffn] = silu(X W1^T) * (X W3^T) over the
// filled rows.  w13: local bf16 [local_experts * 2 * ffn, hidden], gate and up rows interleaved in
// groups of 16 per expert.  Waits (bounded) for every source rank's dispatch flag of this epoch.
void moe_expert_up(const PeerBases& peers, const MoeBuffers& buf, int hidden, int ffn, int local_experts,
                   const void* w13, void* h, uint32_t epoch, cudaStream_t stream, int ctas = 0,
                   uint64_t timeout_ms = 2000);

// Expert GEMM 2 + gate-weighted return + combine: out[tokens, hidden] = sum of the two expert
// outputs of each local token.  w2: local bf16 [local_experts * hidden, ffn].  cta_counter: local
// zero-initialised u32; `ctas` must not change between calls of one layer.
void moe_expert_down(const PeerBases& peers, const MoeBuffers& buf, int tokens, int hidden, int ffn,
                     int local_experts, const void* h, const void* w2, void* out, uint32_t* cta_counter,
                     uint32_t epoch, cudaStream_t stream, int ctas = 0, uint64_t timeout_ms = 2000);

}  // namespace gemm
}  // namespace pccl
