// Large-message all-reduce through the switch, in place on a tensor in symmetric memory.
//
// One kernel, no plan: every rank owns 1 / world of the message; for each 16 bytes of its part a
// thread issues one multimem.ld_reduce (the NVSwitch reads that address in every rank's copy and
// returns the sum, fp32 accumulation) and one multimem.st (the switch writes the sum to every
// rank's copy).  A rank therefore sends and receives about (1 + 1 / world) x the message, against
// 2 (world - 1) / world for any algorithm built on peer loads and stores.
// Synchronisation is two flag rounds for the whole grid: "my input is in place" before the first
// load, "I have delivered my part" after the last store; the kernel ends only when every peer has
// delivered, so the result is complete when the kernel is.  Flags count calls and are never reset.
// The plan interpreter runs the same data loop per channel (kStepMmAllreduce) with one barrier
// pair per chain; this kernel is for the sizes where those fixed costs show (tens to hundreds of MB).
// Sum only, f32 / f16 / bf16.  All waits are bounded; on a timeout the error word is set.
// The reference's large-message kernels are its fused ring / RHD step kernels
// (csrc/plugins/cuda/cuda_executor.cu:963-1057); its NVLS kernel is opt-in and two-pass.
#include <cuda_runtime.h>

#include "../common/launch.h"
#include "../common/util.h"
#include "../ptx/multimem.cuh"
#include "../ptx/sync.cuh"
#include "gemm_host.h"

namespace pccl {
namespace gemm {

namespace {

constexpr int kNvlsThreads = 512;
constexpr int kNvlsUnroll = 4;          // 16-byte groups in flight per thread

struct NvlsParams {
  PeerBases peers;
  uint8_t* mc_base;          // multicast alias of the heap
  uint64_t data_off;         // symmetric offset of the tensor
  uint64_t vecs;             // 16-byte vectors in the whole message (a multiple of world)
  uint64_t flags_off;        // symmetric u32[2 * world]: [0, world) "in place", [world, 2 world) "delivered"
  uint32_t* cta_counter;     // local, monotonic
  uint32_t* error;
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

template <int DT>
__device__ __forceinline__ uint4 switch_sum(const void* mc) {
  if (DT == 0) return ptx::mm_ld_reduce_add_f32(mc);
  if (DT == 1) return ptx::mm_ld_reduce_add_f16(mc);
  return ptx::mm_ld_reduce_add_bf16(mc);
}

template <int DT>
__global__ void __launch_bounds__(kNvlsThreads) allreduce_nvls_kernel(const NvlsParams p) {
  __shared__ uint32_t s_ok;
  const int me = p.peers.rank, world = p.peers.world;
  const volatile uint32_t* abort_flag = p.error;
  const uint64_t deadline = ptx::globaltimer() + p.timeout_ns;
  uint32_t* my_flags = reinterpret_cast<uint32_t*>(p.peers.base[me] + p.flags_off);

  // 1. "my input is in place" -> every peer (CTA 0); every CTA waits for every peer's.
  if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < world && static_cast<int>(threadIdx.x) != me)
    ptx::red_release_sys_add(reinterpret_cast<uint32_t*>(p.peers.base[threadIdx.x] + p.flags_off) + me, 1u);
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < world && static_cast<int>(threadIdx.x) != me) {
    if (!wait_ge(my_flags + threadIdx.x, p.epoch, deadline, abort_flag)) { s_ok = 0; atomicCAS(p.error, 0u, 0x901u); }
  }
  __syncthreads();
  if (!s_ok) return;

  // 2. this rank's part: sum in the switch, deliver to everyone.  Full rounds issue all their loads,
  //    unconditionally, before the first store; what is left goes one vector per thread.  (No lane
  //    re-reads a clamped address to stay unconditional here: a redundant multimem load is a
  //    redundant reduction in the switch.)
  const uint64_t per = p.vecs / world, first = per * me;
  uint8_t* mc = p.mc_base + p.data_off + first * 16;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kNvlsThreads;
  uint64_t v0 = static_cast<uint64_t>(blockIdx.x) * kNvlsThreads + threadIdx.x;
  for (; v0 + (kNvlsUnroll - 1) * stride < per; v0 += stride * kNvlsUnroll) {
    uint4 x[kNvlsUnroll];
#pragma unroll
    for (int u = 0; u < kNvlsUnroll; ++u) x[u] = switch_sum<DT>(mc + (v0 + u * stride) * 16);
#pragma unroll
    for (int u = 0; u < kNvlsUnroll; ++u) ptx::mm_st_v4(mc + (v0 + u * stride) * 16, x[u]);
  }
  for (; v0 < per; v0 += stride) ptx::mm_st_v4(mc + v0 * 16, switch_sum<DT>(mc + v0 * 16));

  // 3. "delivered" -> every peer once all CTAs of this rank are through (the CTA that completes the
  //    count fences at system scope: cumulative over the arrivals it counted); that CTA then waits
  //    for every peer's, so the whole result is here when the kernel ends.
  __syncthreads();
  if (threadIdx.x == 0) {
    ptx::fence_gpu();
    s_ok = atomicAdd(p.cta_counter, 1u) + 1u == p.epoch * gridDim.x ? 2u : 1u;
  }
  __syncthreads();
  if (s_ok != 2u) return;
  if (static_cast<int>(threadIdx.x) < world && static_cast<int>(threadIdx.x) != me) {
    ptx::fence_sys();
    ptx::red_release_sys_add(reinterpret_cast<uint32_t*>(p.peers.base[threadIdx.x] + p.flags_off) + world + me, 1u);
    if (!wait_ge(my_flags + world + threadIdx.x, p.epoch, deadline, abort_flag)) atomicCAS(p.error, 0u, 0x902u);
  }
}

}  // namespace

void allreduce_nvls(const PeerBases& peers, uint8_t* mc_base, uint64_t data_off, uint64_t bytes, int dtype,
                    uint64_t flags_off, uint32_t* cta_counter, uint32_t epoch, cudaStream_t stream, int ctas,
                    uint64_t timeout_ms, uint32_t* error) {
  PCCL_CHECK(mc_base != nullptr, "in-switch all-reduce: the engine has no multicast mapping");
  PCCL_CHECK(bytes % (16ull * peers.world) == 0 && data_off % 16 == 0,
             "in-switch all-reduce: the message must split into 16-byte vectors per rank");
  PCCL_CHECK(epoch >= 1 && ctas > 0, "in-switch all-reduce: epoch counts calls from 1 and the grid is fixed per instance");
  PCCL_CHECK(dtype >= 0 && dtype <= 2, "in-switch all-reduce: f32, f16 or bf16");
  NvlsParams p{};
  p.peers = peers;
  p.mc_base = mc_base;
  p.data_off = data_off;
  p.vecs = bytes / 16;
  p.flags_off = flags_off;
  p.cta_counter = cta_counter;
  p.error = error ? error : error_word();
  p.epoch = epoch;
  p.timeout_ns = timeout_ms * 1000000ull;
  // The grid is part of the completion count and every CTA waits on the peers: fixed per instance, co-resident.
  switch (dtype) {
    case 0: launch_coresident(allreduce_nvls_kernel<0>, static_cast<uint32_t>(ctas), kNvlsThreads, 0, stream, p, true); break;
    case 1: launch_coresident(allreduce_nvls_kernel<1>, static_cast<uint32_t>(ctas), kNvlsThreads, 0, stream, p, true); break;
    default: launch_coresident(allreduce_nvls_kernel<2>, static_cast<uint32_t>(ctas), kNvlsThreads, 0, stream, p, true); break;
  }
}

}  // namespace gemm
}  // namespace pccl
