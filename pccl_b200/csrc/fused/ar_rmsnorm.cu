// All-reduce + residual add + RMSNorm in one kernel (tensor-parallel block epilogue).
//
//   h = residual + sum_r x_r          (x_r: this layer's partial output on rank r, bf16)
//   y = h * rsqrt(mean(h^2) + eps) * gamma
// Every rank ends with the full y and the updated residual h.
//
// x lives in symmetric memory.  Tokens are split over the ranks ("two-shot": a rank reduces
// its T/W tokens and delivers y and h for them to every rank) unless T is too small to split,
// in which case every rank reduces every token itself ("one-shot", nothing to deliver).
// Only h crosses the fabric: a rank delivers the h rows of its tokens to every rank and, once all
// ranks have delivered, every rank normalises the rows it received itself (one local read of h,
// one local write of y), which halves the NVLink bytes against delivering y as well.
// With NVLS the reduction is one multimem.ld_reduce per 16 bytes (the switch sums the ranks'
// copies, fp32 accumulation) and the delivery one multimem.st; without it the kernel pulls the
// peers' rows with 16-byte loads and pushes h with plain peer stores.
// Synchronisation: call-counting flags in symmetric memory ("my x is in place", "I have
// delivered / finished reading"), bounded waits, error word on timeout.
// The unfused baseline is NCCL all-reduce + torch add + RMSNorm; the reference has no such op.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../common/launch.h"
#include "../common/util.h"
#include "../engine/cuda_driver.h"
#include "../ptx/multimem.cuh"
#include "../ptx/sync.cuh"
#include "gemm_host.h"

namespace pccl {
namespace gemm {

namespace {

constexpr int kThreadsNorm = 256;
// Resident CTAs per SM.  A CTA alternates a load phase and a store phase around a block barrier, and a thread
// has only two or three 16-byte loads in flight, so DRAM and NVLink stay busy only when several CTAs overlap
// on an SM: two per SM reached 30 % of DRAM throughput in a profile; four leave 64 registers per thread,
// enough to keep two 16-byte groups of a row in flight.
constexpr int kNormCtasPerSm = 4;

struct NormParams {
  PeerBases peers;
  uint8_t* mc_base;          // multicast alias of the heap (null without NVLS)
  uint64_t x_off, y_off, res_off, flags_off;   // symmetric offsets: x, y, h [T][H] bf16; flags u32[2*world]
  const __nv_bfloat16* gamma;
  uint32_t* cta_counter;     // local, monotonic
  uint32_t* error;
  int tokens, hidden;
  int one_shot;
  float eps;
  uint32_t epoch;
  uint64_t timeout_ns;
};

__device__ __forceinline__ bool wait_ge(const uint32_t* flag, uint32_t want, uint64_t deadline,
                                        const volatile uint32_t* abort_flag) {
  uint32_t spins = 0;
  while (static_cast<int32_t>(ptx::ld_acquire_sys(flag) - want) < 0) {
    if ((++spins & 63u) == 0u) {
      if (*abort_flag || ptx::globaltimer() > deadline) return false;
      __nanosleep(64);
    }
  }
  return true;
}

__device__ __forceinline__ void unpack8(uint4 v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// h = residual + sum over ranks of x for one token row: h (rounded to bf16, as every rank will read
// it) goes to h_row and to every rank's residual buffer; returns this thread's share of sum(h^2).
// kW: 0 = in-switch reduction (one multimem.ld_reduce per 16 bytes), else the number of peer loads
// issued per 16 bytes (slots past the world re-read the own row and are not added).  kB 16-byte
// groups are in flight per thread: every load is issued, unconditionally and from a clamped
// address, before the first use, since a conditionally assigned register or a store between two
// loads makes each load wait for the one before.
template <int kW, int kB>
__device__ __forceinline__ float sum_row(const NormParams& p, uint64_t row, int vecs, float* h_row) {
  constexpr int kLoads = kW > 0 ? kW : 1;
  const int me = p.peers.rank, world = p.peers.world;
  uint8_t* self = p.peers.base[me];
  float ss = 0.f;
  for (int v0 = threadIdx.x; v0 < vecs; v0 += kB * kThreadsNorm) {
    uint4 res[kB], x[kB][kLoads];
    int v[kB];
#pragma unroll
    for (int b = 0; b < kB; ++b) v[b] = v0 + b * kThreadsNorm < vecs ? v0 + b * kThreadsNorm : v0;
#pragma unroll
    for (int b = 0; b < kB; ++b) res[b] = ptx::ld_local_v4(self + p.res_off + row + v[b] * 16);
#pragma unroll
    for (int b = 0; b < kB; ++b) {
      if constexpr (kW == 0) {
        x[b][0] = ptx::mm_ld_reduce_add_bf16(p.mc_base + p.x_off + row + v[b] * 16);
      } else {
#pragma unroll
        for (int r = 0; r < kW; ++r)
          x[b][r] = ptx::ld_peer_v4(p.peers.base[r < world ? r : me] + p.x_off + row + v[b] * 16);
      }
    }
#pragma unroll
    for (int b = 0; b < kB; ++b) {
      if (b > 0 && v0 + b * kThreadsNorm >= vecs) break;
      float acc[8], f[8];
      unpack8(res[b], acc);
#pragma unroll
      for (int r = 0; r < kLoads; ++r) {
        if (kW > 0 && r >= world) break;
        unpack8(x[b][r], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
      const uint4 hp = pack8(acc);
      unpack8(hp, acc);
#pragma unroll
      for (int i = 0; i < 8; ++i) { h_row[v[b] * 8 + i] = acc[i]; ss += acc[i] * acc[i]; }
      const uint64_t at = p.res_off + row + v[b] * 16;
      if (p.one_shot) {
        ptx::st_v4(self + at, hp);
      } else if (kW == 0) {
        ptx::mm_st_v4(p.mc_base + at, hp);
      } else {
        for (int i = 0; i < world; ++i) ptx::st_v4(p.peers.base[(me + i) % world] + at, hp);
      }
    }
  }
  return ss;
}

__global__ void __launch_bounds__(kThreadsNorm, kNormCtasPerSm) ar_residual_rmsnorm_kernel(const NormParams p) {
  extern __shared__ float h_row[];            // hidden fp32 values of the current token
  __shared__ float warp_sums[kThreadsNorm / 32];
  __shared__ uint32_t s_ok;
  const int me = p.peers.rank, world = p.peers.world;
  const volatile uint32_t* abort_flag = p.error;
  const uint64_t deadline = ptx::globaltimer() + p.timeout_ns;
  uint32_t* my_flags = reinterpret_cast<uint32_t*>(p.peers.base[me] + p.flags_off);

  // 1. "my x is in place" -> every peer; then wait for every peer's.
  if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < world && static_cast<int>(threadIdx.x) != me) {
    ptx::fence_sys();
    ptx::red_release_sys_add(reinterpret_cast<uint32_t*>(p.peers.base[threadIdx.x] + p.flags_off) + me, 1u);
  }
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < world && static_cast<int>(threadIdx.x) != me) {
    if (!wait_ge(my_flags + threadIdx.x, p.epoch, deadline, abort_flag)) { s_ok = 0; atomicCAS(p.error, 0u, 0x601u); }
  }
  __syncthreads();
  if (!s_ok) return;

  // 2. tokens of this rank
  const int per_rank = p.one_shot ? p.tokens : p.tokens / world;
  const int first = p.one_shot ? 0 : me * per_rank;
  const int vecs = p.hidden / 8;
  const uint64_t row_bytes = static_cast<uint64_t>(p.hidden) * 2;
  const bool use_mc = p.mc_base != nullptr;
  uint8_t* self = p.peers.base[me];

  // Sum of squares of the row now in h_row -> the row's scale; y = h * scale * gamma, stored locally.
  auto row_scale = [&](float ss) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < kThreadsNorm / 32; ++w) total += warp_sums[w];
    return rsqrtf(total / static_cast<float>(p.hidden) + p.eps);
  };

  // 2a. own tokens: h = residual + sum of the ranks' x; h goes to every rank, y stays here.
  for (int t = first + blockIdx.x; t < first + per_rank; t += gridDim.x) {
    const uint64_t row = static_cast<uint64_t>(t) * row_bytes;
    float ss;
    if (use_mc) ss = sum_row<0, 2>(p, row, vecs, h_row);
    else if (world <= 2) ss = sum_row<2, 2>(p, row, vecs, h_row);
    else if (world <= 4) ss = sum_row<4, 1>(p, row, vecs, h_row);
    else ss = sum_row<8, 1>(p, row, vecs, h_row);
    const float scale = row_scale(ss);
    for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
      float g[8], yv[8];
      unpack8(*reinterpret_cast<const uint4*>(p.gamma + v * 8), g);
#pragma unroll
      for (int i = 0; i < 8; ++i) yv[i] = h_row[v * 8 + i] * scale * g[i];
      ptx::st_v4(self + p.y_off + row + v * 16, pack8(yv));
    }
    __syncthreads();
  }

  // 3. "delivered / done reading" -> every peer, once all CTAs of this rank are through; every CTA
  //    then waits for every peer's: the other ranks' h rows are in this rank's memory after that.
  __syncthreads();
  if (threadIdx.x == 0) {
    // GPU scope suffices here: the CTA that completes the count fences at system scope before it posts,
    // and that fence is cumulative over every arrival it counted (a system fence per CTA is slow while
    // other SMs stream stores over NVLink).
    ptx::fence_gpu();
    const uint32_t done = atomicAdd(p.cta_counter, 1u) + 1u;
    s_ok = done == p.epoch * gridDim.x ? 2u : 1u;
  }
  __syncthreads();
  if (s_ok == 2u && static_cast<int>(threadIdx.x) < world && static_cast<int>(threadIdx.x) != me) {
    ptx::fence_sys();
    ptx::red_release_sys_add(reinterpret_cast<uint32_t*>(p.peers.base[threadIdx.x] + p.flags_off) + world + me, 1u);
  }
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < world && static_cast<int>(threadIdx.x) != me) {
    if (!wait_ge(my_flags + world + threadIdx.x, p.epoch, deadline, abort_flag)) { s_ok = 0; atomicCAS(p.error, 0u, 0x602u); }
  }
  __syncthreads();
  if (!s_ok || p.one_shot) return;

  // 2b. the other ranks' tokens: their h rows arrived above; the norm is local work (one read of h,
  //     one write of y), so y never crosses NVLink.
  const int others = p.tokens - per_rank;
  for (int i = blockIdx.x; i < others; i += gridDim.x) {
    const int t = i < first ? i : i + per_rank;
    const uint64_t row = static_cast<uint64_t>(t) * row_bytes;
    float ss = 0.f;
    for (int v0 = threadIdx.x; v0 < vecs; v0 += 2 * kThreadsNorm) {
      const int v1 = v0 + kThreadsNorm < vecs ? v0 + kThreadsNorm : v0;
      const uint4 raw0 = ptx::ld_peer_v4(self + p.res_off + row + v0 * 16);
      const uint4 raw1 = ptx::ld_peer_v4(self + p.res_off + row + v1 * 16);
      float acc[8];
      unpack8(raw0, acc);
#pragma unroll
      for (int k = 0; k < 8; ++k) { h_row[v0 * 8 + k] = acc[k]; ss += acc[k] * acc[k]; }
      if (v1 != v0) {
        unpack8(raw1, acc);
#pragma unroll
        for (int k = 0; k < 8; ++k) { h_row[v1 * 8 + k] = acc[k]; ss += acc[k] * acc[k]; }
      }
    }
    const float scale = row_scale(ss);
    for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
      float g[8], yv[8];
      unpack8(*reinterpret_cast<const uint4*>(p.gamma + v * 8), g);
#pragma unroll
      for (int k = 0; k < 8; ++k) yv[k] = h_row[v * 8 + k] * scale * g[k];
      ptx::st_v4(self + p.y_off + row + v * 16, pack8(yv));
    }
    __syncthreads();
  }
}

}  // namespace

void ar_residual_rmsnorm(const PeerBases& peers, uint8_t* mc_base, uint64_t x_off, uint64_t y_off, uint64_t res_off,
                         uint64_t flags_off, const void* gamma, uint32_t* cta_counter, int tokens, int hidden,
                         float eps, uint32_t epoch, cudaStream_t stream, int ctas, uint64_t timeout_ms) {
  PCCL_CHECK(hidden % 8 == 0 && hidden <= 16384, "AR+RMSNorm: hidden must be a multiple of 8, at most 16384");
  PCCL_CHECK(epoch >= 1, "AR+RMSNorm: epoch counts calls from 1");
  NormParams p{};
  p.peers = peers;
  p.mc_base = mc_base;
  p.x_off = x_off; p.y_off = y_off; p.res_off = res_off; p.flags_off = flags_off;
  p.gamma = static_cast<const __nv_bfloat16*>(gamma);
  p.cta_counter = cta_counter;
  p.error = error_word();
  p.tokens = tokens; p.hidden = hidden;
  // Splitting tokens pays once every rank has at least a few of them.
  p.one_shot = (peers.world == 1 || tokens % peers.world != 0 || tokens / peers.world < 4) ? 1 : 0;
  p.eps = eps;
  p.epoch = epoch;
  p.timeout_ns = timeout_ms * 1000000ull;
  const int mine = p.one_shot ? tokens : tokens / peers.world;
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = ctas > 0 ? ctas : (mine < kNormCtasPerSm * sms ? mine : kNormCtasPerSm * sms);
  if (grid < 1) grid = 1;
  // The grid size is part of the completion count: it must not change between calls of one
  // operator instance (the Python wrapper fixes tokens per instance).
  const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
  if (smem > 48 * 1024)
    PCCL_CUDA(cudaFuncSetAttribute(ar_residual_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(smem)));
  launch_coresident(ar_residual_rmsnorm_kernel, static_cast<uint32_t>(grid), kThreadsNorm, smem, stream, p, true);
  PCCL_CUDA(cudaGetLastError());
}

}  // namespace gemm
}  // namespace pccl
