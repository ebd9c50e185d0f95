// The router + dispatch kernel itself (see moe_dispatch.cu for the operator around it).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../ptx/sync.cuh"

namespace pccl {
namespace gemm {

constexpr int kMoeRouteMaxExperts = 64;
constexpr int kMoeRouteWarps = 8;

struct MoeRouteParams {
  uint8_t* base[8];           // every rank's symmetric heap as mapped here (dispatch only)
  int rank, world;
  const __nv_bfloat16* x;     // [tokens][hidden]
  const __nv_bfloat16* wg;    // [experts][hidden]
  uint64_t recv_off, meta_off, counts_off, ready_off;
  uint32_t* scratch;          // [experts] slot counters, [experts] = finished CTAs; zero at launch
  int32_t* topk_idx;          // optional [tokens][2]
  float* topk_gate;           // optional [tokens][2]
  int32_t* topk_slot;         // optional [tokens][2]: row claimed in the expert's region
  uint32_t* expert_counts;    // optional [experts]: tokens routed to each expert by this rank
  int tokens, hidden, experts, local_experts, cap;
  int dispatch;
  uint32_t epoch;
};

template <int kE>
__global__ void __launch_bounds__(kMoeRouteWarps * 32) moe_route_kernel(const MoeRouteParams p) {
  extern __shared__ uint4 wg_s[];                  // [kE][hidden / 8]
  __shared__ uint32_t is_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int vecs = p.hidden / 8;
  for (int i = threadIdx.x; i < kE * vecs; i += blockDim.x)
    wg_s[i] = reinterpret_cast<const uint4*>(p.wg)[i];
  __syncthreads();

  for (int t = blockIdx.x * kMoeRouteWarps + warp; t < p.tokens; t += gridDim.x * kMoeRouteWarps) {
    const uint4* row = reinterpret_cast<const uint4*>(p.x + static_cast<int64_t>(t) * p.hidden);
    float logit[kE];
#pragma unroll
    for (int e = 0; e < kE; ++e) logit[e] = 0.f;
    for (int v = lane; v < vecs; v += 32) {
      const uint4 xv = row[v];
      const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
      float xf[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        xf[2 * j] = __uint_as_float(xw[j] << 16);
        xf[2 * j + 1] = __uint_as_float(xw[j] & 0xffff0000u);
      }
#pragma unroll
      for (int e = 0; e < kE; ++e) {
        const uint4 wv = wg_s[e * vecs + v];
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          logit[e] = fmaf(xf[2 * j], __uint_as_float(ww[j] << 16), logit[e]);
          logit[e] = fmaf(xf[2 * j + 1], __uint_as_float(ww[j] & 0xffff0000u), logit[e]);
        }
      }
    }
#pragma unroll
    for (int e = 0; e < kE; ++e)
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) logit[e] += __shfl_xor_sync(0xffffffffu, logit[e], o);

    // Top-2 of the softmax = top-2 of the logits; renormalised gates need only those two.
    // The selection is total: a non-finite logit (a NaN or Inf activation makes the whole row
    // non-finite) counts as the lowest value, and the two picks start as experts 0 and 1, so both
    // are always valid, distinct expert numbers whatever the input holds.
#pragma unroll
    for (int e = 0; e < kE; ++e)
      if (!(fabsf(logit[e]) <= 3.0e38f)) logit[e] = -3.0e38f;
    int e1 = 0, e2 = 1;
    float l1 = logit[0], l2 = logit[1];
    if (l2 > l1) { e1 = 1; e2 = 0; l1 = logit[1]; l2 = logit[0]; }
#pragma unroll
    for (int e = 2; e < kE; ++e) {
      if (logit[e] > l1) { l2 = l1; e2 = e1; l1 = logit[e]; e1 = e; }
      else if (logit[e] > l2) { l2 = logit[e]; e2 = e; }
    }
    const float g2 = 1.f / (1.f + __expf(l1 - l2));          // p2 / (p1 + p2)
    const float g1 = 1.f - g2;
    const int choice[2] = {e1, e2};
    const float gate[2] = {g1, g2};
    int slot[2] = {0, 0};
    if (lane == 0) {
      slot[0] = static_cast<int>(atomicAdd(p.scratch + e1, 1u));
      slot[1] = static_cast<int>(atomicAdd(p.scratch + e2, 1u));
      for (int k = 0; k < 2; ++k) {
        if (p.topk_idx) p.topk_idx[2 * t + k] = choice[k];
        if (p.topk_gate) p.topk_gate[2 * t + k] = gate[k];
        if (p.topk_slot) p.topk_slot[2 * t + k] = slot[k];
      }
    }
    if (p.dispatch) {
      slot[0] = __shfl_sync(0xffffffffu, slot[0], 0);
      slot[1] = __shfl_sync(0xffffffffu, slot[1], 0);
      uint8_t* dst[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int dest = choice[k] / p.local_experts;
        const int region = (choice[k] % p.local_experts) * p.world + p.rank;
        const uint64_t row_index = static_cast<uint64_t>(region) * p.cap + slot[k];
        dst[k] = slot[k] < p.cap ? p.base[dest] + p.recv_off + row_index * p.hidden * 2 : nullptr;
        if (lane == 0 && dst[k]) {
          uint2 m;
          m.x = static_cast<uint32_t>(2 * t + k);
          m.y = __float_as_uint(gate[k]);
          *reinterpret_cast<uint2*>(p.base[dest] + p.meta_off + row_index * sizeof(uint2)) = m;
        }
      }
      // Four row vectors per lane are loaded before the first store (the row was just read for the
      // logits, so these hit in cache); loads are unconditional, the tail re-reads the last vector.
      for (int v0 = lane; v0 < vecs; v0 += 128) {
        uint4 xv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) xv[u] = row[min(v0 + 32 * u, vecs - 1)];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int v = v0 + 32 * u;
          if (v < vecs) {
            if (dst[0]) ptx::st_v4(dst[0] + v * 16, xv[u]);
            if (dst[1]) ptx::st_v4(dst[1] + v * 16, xv[u]);
          }
        }
      }
    }
  }

  // The last CTA publishes: counts per expert locally, and (dispatching) the row count of each
  // region at its expert rank followed by this rank's flag there.
  __syncthreads();
  if (threadIdx.x == 0) {
    // GPU scope suffices here: the CTA that completes the count fences at system scope before it posts,
    // and that fence is cumulative over every arrival it counted (a system fence per CTA is slow while
    // other SMs stream stores over NVLink).
    ptx::fence_gpu();
    is_last = atomicAdd(p.scratch + kE, 1u) + 1u == gridDim.x ? 1u : 0u;
  }
  __syncthreads();
  if (!is_last) return;
  ptx::fence_sys();
  if (static_cast<int>(threadIdx.x) < kE) {
    const int e = threadIdx.x;
    const uint32_t n = atomicAdd(p.scratch + e, 0u);
    if (p.expert_counts) p.expert_counts[e] = n;
    if (p.dispatch) {
      const int dest = e / p.local_experts;
      const int region = (e % p.local_experts) * p.world + p.rank;
      ptx::st_relaxed_sys(reinterpret_cast<uint32_t*>(p.base[dest] + p.counts_off) + region,
                              n < static_cast<uint32_t>(p.cap) ? n : static_cast<uint32_t>(p.cap));
    }
  }
  __syncthreads();
  if (p.dispatch && static_cast<int>(threadIdx.x) < p.world) {
    ptx::fence_sys();
    ptx::red_release_sys_add(reinterpret_cast<uint32_t*>(p.base[threadIdx.x] + p.ready_off) + p.rank, 1u);
  }
}

inline cudaError_t launch_moe_route(const MoeRouteParams& p, cudaStream_t stream) {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = (p.tokens + kMoeRouteWarps - 1) / kMoeRouteWarps;
  if (grid > 2 * sms) grid = 2 * sms;
  if (grid < 1) grid = 1;
  const size_t smem = static_cast<size_t>(p.experts) * p.hidden * 2;
  cudaError_t err = cudaSuccess;
#define PCCL_MOE_ROUTE_CASE(E)                                                                              \
  case E:                                                                                                   \
    if (smem > 48 * 1024)                                                                                   \
      err = cudaFuncSetAttribute(moe_route_kernel<E>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                                 static_cast<int>(smem));                                                   \
    if (err == cudaSuccess) moe_route_kernel<E><<<grid, kMoeRouteWarps * 32, smem, stream>>>(p);          \
    break;
  switch (p.experts) {
    PCCL_MOE_ROUTE_CASE(2)
    PCCL_MOE_ROUTE_CASE(4)
    PCCL_MOE_ROUTE_CASE(8)
    PCCL_MOE_ROUTE_CASE(16)
    PCCL_MOE_ROUTE_CASE(32)
    PCCL_MOE_ROUTE_CASE(64)
    default: return cudaErrorInvalidValue;
  }
#undef PCCL_MOE_ROUTE_CASE
  return err != cudaSuccess ? err : cudaGetLastError();
}

}  // namespace gemm
}  // namespace pccl
