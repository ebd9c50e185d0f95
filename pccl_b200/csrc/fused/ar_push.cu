// Medium-size all-reduce (sum) in one kernel: push reduce-scatter, reduce, push all-gather.
//
//   1. every rank pushes slice p of its input into peer p's receive area A (plain NVLink stores:
//      posted writes, no read round trip), then the last CTA to finish posts one flag per peer;
//   2. after the W - 1 flags a rank sums its own slice (fp32, rank order: each slice is reduced
//      by exactly one rank, so every rank ends with identical bits), writes it to its output and
//      pushes it into every peer's area B, then posts the second flag;
//   3. after those flags the rank copies the W - 1 reduced slices from B to its output.
// Input and output are ordinary device tensors (no staging into symmetric memory, output may
// alias input); NVLink carries the optimal 2 (W - 1) / W of the message per direction and there
// are two flag rounds in total.  Areas are double-buffered by call parity and flags count calls
// (a rank can be at most one call ahead of a peer), so nothing is reset between calls.
// Every wait is bounded; a timeout sets the error word and the kernel returns.
// The same kernel serves reduce-scatter (stops after step 2, keeps only its own slice), all-gather
// (step 1 pushes the whole shard to every peer, step 2 is skipped, step 3 copies from A) and
// all-to-all (step 1 as is, step 3 copies from A), selected by `mode`.
// The plan interpreter runs the same algorithm as a chain of steps with a barrier after each;
// this kernel is its fused form for sizes where those barriers dominate.  The reference's
// counterpart is its fused-step kernel (csrc/plugins/cuda/cuda_executor.cu:963-1057).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../common/launch.h"
#include "../common/util.h"
#include "../engine/cuda_driver.h"
#include "../ptx/sync.cuh"
#include "gemm_host.h"

namespace pccl {
namespace gemm {

namespace {

constexpr int kPushThreads = 512;
constexpr int kPushUnroll = 4;

struct PushParams {
  PeerBases peers;
  uint64_t area_off;         // symmetric bytes: [2 parities][A | B][world][slice_cap]
  uint64_t slice_cap;        // bytes per (area, source) slot, multiple of 16
  uint64_t flags_off;        // symmetric u32 [2][world]: phase-1 and phase-2 flags, call counting
  uint32_t* counters;        // local u32[2], monotonic: CTAs through phase 1 / phase 2
  const uint8_t* in;
  uint8_t* out;
  uint64_t vecs;             // 16-byte vectors in the message
  uint64_t per;              // vectors per slice (the last slice may be shorter)
  int dtype;                 // 0 f32, 1 f16, 2 bf16
  int mode;                  // PushMode
  uint32_t epoch;
  uint32_t* error;
  uint64_t timeout_ns;
};

// Copy `len` 16-byte vectors, the whole grid cooperating; loads unconditional, stores predicated.
template <bool kRemoteDst>
__device__ __forceinline__ void grid_copy(const uint4* src, uint4* dst, uint64_t len, uint64_t tid, uint64_t nthreads) {
  for (uint64_t i = tid; i < len; i += nthreads * kPushUnroll) {
    uint4 v[kPushUnroll];
#pragma unroll
    for (int u = 0; u < kPushUnroll; ++u) {
      const uint64_t j = i + u * nthreads;
      v[u] = ptx::ld_local_v4(src + (j < len ? j : len - 1));
    }
#pragma unroll
    for (int u = 0; u < kPushUnroll; ++u) {
      const uint64_t j = i + u * nthreads;
      if (j < len) {
        if (kRemoteDst) ptx::st_v4(dst + j, v[u]); else dst[j] = v[u];
      }
    }
  }
}

__device__ __forceinline__ bool wait_ge(const uint32_t* flag, uint32_t want, uint64_t deadline,
                                        const volatile uint32_t* abort_flag) {
  uint32_t spins = 0;
  while (static_cast<int32_t>(ptx::ld_acquire_sys(flag) - want) < 0) {
    if ((++spins & 63u) == 0u && (*abort_flag || ptx::globaltimer() > deadline)) return false;
  }
  return true;
}

template <int DT>
__device__ __forceinline__ void add_into(float* acc, uint4 v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (DT == 0) {
      acc[j] += __uint_as_float(w[j]);
    } else if (DT == 2) {
      acc[2 * j] += __uint_as_float(w[j] << 16);
      acc[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
    } else {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
      acc[2 * j] += f.x;
      acc[2 * j + 1] += f.y;
    }
  }
}
template <int DT>
__device__ __forceinline__ uint4 pack(const float* acc) {
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (DT == 0) {
      w[j] = __float_as_uint(acc[j]);
    } else if (DT == 2) {
      __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&h);
    } else {
      __half2 h = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&h);
    }
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// All CTAs arrive; the one that completes the count posts `flag_row[me]` at every peer, one thread
// per peer so that the W - 1 release operations travel in parallel.
__device__ __forceinline__ void arrive_and_post(const PushParams& p, int phase) {
  __shared__ uint32_t is_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    // GPU scope suffices here: the CTA that completes the count fences at system scope before it posts,
    // and that fence is cumulative over every arrival it counted (a system fence per CTA is slow while
    // other SMs stream stores over NVLink).
    ptx::fence_gpu();
    const uint32_t seen = atomicAdd(p.counters + phase, 1u) + 1u;
    is_last = seen == p.epoch * gridDim.x ? 1u : 0u;
  }
  __syncthreads();
  const int me = p.peers.rank, peer = static_cast<int>(threadIdx.x);
  if (is_last && peer < p.peers.world && peer != me) {
    ptx::fence_sys();
    uint32_t* flags = reinterpret_cast<uint32_t*>(p.peers.base[peer] + p.flags_off) + phase * p.peers.world;
    ptx::red_release_sys_add(flags + me, 1u);
  }
}

__device__ __forceinline__ bool wait_peers(const PushParams& p, int phase, uint64_t deadline, uint32_t* ok) {
  const int me = p.peers.rank;
  const volatile uint32_t* abort_flag = p.error;
  if (threadIdx.x == 0) *ok = 1;
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < p.peers.world && static_cast<int>(threadIdx.x) != me) {
    const uint32_t* flags = reinterpret_cast<const uint32_t*>(p.peers.base[me] + p.flags_off) + phase * p.peers.world;
    if (!wait_ge(flags + threadIdx.x, p.epoch, deadline, abort_flag)) {
      *ok = 0;
      atomicCAS(p.error, 0u, 0x801u + static_cast<uint32_t>(phase));
    }
  }
  __syncthreads();
  return *ok != 0;
}

// kW: compile-time bound on the world size (2, 4 or 8) so that a thread loads exactly the sources
// there are; kV vectors per thread keep eight 16-byte loads in flight whatever kW is.
template <int DT, int kW>
__global__ void __launch_bounds__(kPushThreads) allreduce_push_kernel(const PushParams p) {
  constexpr int kLanes = DT == 0 ? 4 : 8;
  constexpr int kV = 8 / kW;
  __shared__ uint32_t ok;
  const int me = p.peers.rank, world = p.peers.world;
  const uint64_t parity = p.epoch & 1u;
  const uint64_t area_bytes = static_cast<uint64_t>(world) * p.slice_cap;             // one of A / B
  const uint64_t a_off = p.area_off + parity * 2 * area_bytes, b_off = a_off + area_bytes;
  const uint64_t deadline = ptx::globaltimer() + p.timeout_ns;
  const uint64_t tid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const uint64_t nthreads = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  auto slice_len = [&](int s) -> uint64_t {
    const uint64_t begin = static_cast<uint64_t>(s) * p.per;
    return begin >= p.vecs ? 0 : (p.vecs - begin < p.per ? p.vecs - begin : p.per);
  };
  const uint4* in = reinterpret_cast<const uint4*>(p.in);
  uint4* out = reinterpret_cast<uint4*>(p.out);

  // 1. push slice `peer` of my input (all-gather: my whole shard) into the peer's A[me]
  for (int k = 1; k < world; ++k) {
    const int peer = (me + k) % world;
    const bool whole = p.mode == kPushAllGather;
    const uint64_t len = whole ? slice_len(me) : slice_len(peer);
    const uint4* src = whole ? in : in + static_cast<uint64_t>(peer) * p.per;
    uint4* dst = reinterpret_cast<uint4*>(p.peers.base[peer] + a_off + static_cast<uint64_t>(me) * p.slice_cap);
    grid_copy<true>(src, dst, len, tid, nthreads);
  }
  arrive_and_post(p, 0);
  if (!wait_peers(p, 0, deadline, &ok)) return;

  // 2. reduce my slice in rank order; result to my output and (all-reduce) to every peer's B[me]
  if (p.mode == kPushAllReduce || p.mode == kPushReduceScatter) {
    const bool scatter_only = p.mode == kPushReduceScatter;
    const uint64_t len = slice_len(me);
    const uint64_t base = static_cast<uint64_t>(me) * p.per;
    const uint8_t* a_mine = p.peers.base[me] + a_off;
    for (uint64_t i0 = tid; i0 < len; i0 += nthreads * kV) {
      uint4 raw[kV][kW];
#pragma unroll
      for (int v = 0; v < kV; ++v) {                         // every source of kV vectors in flight before the first add
        const uint64_t j = i0 + v * nthreads;
        const uint64_t i = j < len ? j : len - 1;
#pragma unroll
        for (int s = 0; s < kW; ++s) {
          const int ss = s < world ? s : me;
          // select the address, then load unconditionally (one instruction, no branch around it)
          const uint4* ptr = ss == me ? in + base + i
                                      : reinterpret_cast<const uint4*>(a_mine + static_cast<uint64_t>(ss) * p.slice_cap) + i;
          raw[v][s] = ptx::ld_local_v4(ptr);
        }
      }
#pragma unroll
      for (int v = 0; v < kV; ++v) {
        const uint64_t i = i0 + v * nthreads;
        if (i >= len) continue;
        float acc[kLanes];
#pragma unroll
        for (int l = 0; l < kLanes; ++l) acc[l] = 0.f;
#pragma unroll
        for (int s = 0; s < kW; ++s)
          if (s < world) add_into<DT>(acc, raw[v][s]);
        const uint4 r = pack<DT>(acc);
        if (scatter_only) {
          out[i] = r;                                          // the output is this rank's shard only
          continue;
        }
        out[base + i] = r;
        for (int k = 1; k < world; ++k) {
          const int peer = (me + k) % world;
          ptx::st_v4(reinterpret_cast<uint4*>(p.peers.base[peer] + b_off + static_cast<uint64_t>(me) * p.slice_cap) + i, r);
        }
      }
    }
  }
  // All modes share the counters and flags (they count calls), so the modes with a single flag
  // round still tick the second one; nobody waits for it.
  if (p.mode == kPushReduceScatter) {
    arrive_and_post(p, 1);
    return;
  }
  uint64_t from_off = a_off;                                 // all-gather / all-to-all read what step 1 delivered
  if (p.mode == kPushAllReduce) {
    arrive_and_post(p, 1);
    if (!wait_peers(p, 1, deadline, &ok)) return;
    from_off = b_off;
  } else {
    // my own part goes straight from the input to the output
    const uint4* src = p.mode == kPushAllGather ? in : in + static_cast<uint64_t>(me) * p.per;
    grid_copy<false>(src, out + static_cast<uint64_t>(me) * p.per, slice_len(me), tid, nthreads);
  }

  // 3. gather the other slices into my output
  for (int k = 1; k < world; ++k) {
    const int s = (me + k) % world;
    const uint4* src = reinterpret_cast<const uint4*>(p.peers.base[me] + from_off + static_cast<uint64_t>(s) * p.slice_cap);
    grid_copy<false>(src, out + static_cast<uint64_t>(s) * p.per, slice_len(s), tid, nthreads);
  }
  if (p.mode != kPushAllReduce) arrive_and_post(p, 1);
}

}  // namespace

void collective_push(PushMode mode, const PeerBases& peers, uint64_t area_off, uint64_t capacity_bytes,
                     uint64_t flags_off, uint32_t* counters, const void* in, void* out, uint64_t bytes, int dtype,
                     uint32_t epoch, cudaStream_t stream, int ctas, uint64_t timeout_ms, uint32_t* error) {
  // `bytes` is the size of the full message: the all-reduce tensor, the reduce-scatter input, the
  // all-gather output, either side of the all-to-all.
  PCCL_CHECK(bytes % 16 == 0 && bytes > 0, "push all-reduce: size must be a positive multiple of 16 bytes");
  PCCL_CHECK(mode == kPushAllReduce || bytes % (16ull * peers.world) == 0,
             "push collective: every rank's part must be a multiple of 16 bytes");
  PCCL_CHECK(mode != kPushAllToAll || in != out, "push all-to-all cannot run in place");
  if (mode == kPushReduceScatter) {
    // Step 2 writes the output while other CTAs of this rank may still push input slices to the
    // peers in step 1; only this rank's own slice is never read by step 1.
    const uintptr_t in_lo = reinterpret_cast<uintptr_t>(in), in_hi = in_lo + bytes;
    const uintptr_t shard = bytes / peers.world;
    const uintptr_t out_lo = reinterpret_cast<uintptr_t>(out), out_hi = out_lo + shard;
    const bool overlaps = out_lo < in_hi && in_lo < out_hi;
    PCCL_CHECK(!overlaps || out_lo == in_lo + static_cast<uintptr_t>(peers.rank) * shard,
               "push reduce-scatter: the output may alias the input only at this rank's own slice");
  }
  PCCL_CHECK(bytes <= capacity_bytes, "push all-reduce: " << bytes << " bytes exceed the areas' " << capacity_bytes);
  PCCL_CHECK(reinterpret_cast<uintptr_t>(in) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0,
             "push all-reduce: tensors must be 16-byte aligned");
  PCCL_CHECK(dtype >= 0 && dtype <= 2, "push all-reduce: f32, f16 and bf16 only");
  PCCL_CHECK(epoch != 0 && ctas > 0, "push all-reduce: the call number starts at 1 and the grid is fixed per instance");
  PushParams p{};
  p.peers = peers;
  p.area_off = area_off;
  // Slot size from the capacity, not from this call: the layout must not move between calls.
  const uint64_t cap_vecs = (capacity_bytes / 16 + peers.world - 1) / peers.world;
  p.slice_cap = cap_vecs * 16;
  p.flags_off = flags_off;
  p.counters = counters;
  p.in = static_cast<const uint8_t*>(in);
  p.out = static_cast<uint8_t*>(out);
  p.vecs = bytes / 16;
  p.per = (p.vecs + peers.world - 1) / peers.world;
  p.dtype = dtype;
  p.mode = mode;
  p.epoch = epoch;
  p.error = error ? error : error_word();
  p.timeout_ns = timeout_ms * 1000000ull;
  // The grid is part of the completion count: it is the same for every call of an instance.
  // Every CTA spins on flags that a peer posts when its last CTA arrives: the whole grid must be
  // resident, here and on the peer.
#define PCCL_PUSH_LAUNCH(DT)                                                                                  \
  do {                                                                                                        \
    if (peers.world <= 2) launch_coresident(allreduce_push_kernel<DT, 2>, ctas, kPushThreads, 0, stream, p, true);      \
    else if (peers.world <= 4) launch_coresident(allreduce_push_kernel<DT, 4>, ctas, kPushThreads, 0, stream, p, true); \
    else launch_coresident(allreduce_push_kernel<DT, 8>, ctas, kPushThreads, 0, stream, p, true);                       \
  } while (0)
  switch (dtype) {
    case 0: PCCL_PUSH_LAUNCH(0); break;
    case 1: PCCL_PUSH_LAUNCH(1); break;
    default: PCCL_PUSH_LAUNCH(2); break;
  }
#undef PCCL_PUSH_LAUNCH
}

}  // namespace gemm
}  // namespace pccl
