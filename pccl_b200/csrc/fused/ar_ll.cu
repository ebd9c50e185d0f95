// Small-message all-reduce in one kernel with flag-carrying packets ("low latency" protocol).
//
// Every rank pushes its input to every peer as 16-byte packets {data, flag, data, flag}: 8 bytes
// of payload and the call number twice, each 8-byte half valid on its own, so a receiver needs
// no separate signal: it polls the packet until both flags show this call's number.  There is
// no barrier, no notify / wait round trip and no staging copy: the kernel reads the caller's
// input, writes the caller's output, and costs one NVLink store latency plus the poll.
// Receive buffers are double-buffered by call parity; a rank can be at most one call ahead of a
// peer (finishing call n needs every peer's packets of call n), so parity n is never rewritten
// while a peer still reads it.  Sums are taken in rank order in fp32: every rank gets the same
// bits.  Payload doubles on the wire, so this is for messages up to a few hundred KB.
// All polls are bounded; on a timeout the error word is set and the kernel returns.
// The reference's small-message path is its tree / fused-step kernel (docs/roadmap.md:402-424
// gives 37.5 us for 4 KB on two H100); it has no packet protocol.
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

constexpr int kLLThreads = 256;

struct LLParams {
  PeerBases peers;
  uint64_t buf_off;          // symmetric: uint4 [2][world][capacity_units]
  uint64_t capacity_units;   // 8-byte payload units per (parity, source)
  const uint2* in;           // 8-byte units of the input
  uint2* out;
  uint64_t units;
  int dtype;                 // 0 f32, 1 f16, 2 bf16
  int mode;                  // 0 all-reduce (units = whole message); 1 reduce-scatter, 2 all-gather,
                             // 3 all-to-all (units = one rank's part)
  uint32_t flag;             // call number, never 0
  uint32_t* error;
  uint64_t timeout_ns;
};

__device__ __forceinline__ void st_packet(uint4* p, uint2 d, uint32_t flag) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(d.x), "r"(flag), "r"(d.y), "r"(flag)
               : "memory");
}
__device__ __forceinline__ uint4 ld_packet(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

template <int DT>
__device__ __forceinline__ void accumulate(float* acc, uint2 d) {
  if (DT == 0) {
    acc[0] += __uint_as_float(d.x);
    acc[1] += __uint_as_float(d.y);
  } else if (DT == 2) {
    acc[0] += __uint_as_float(d.x << 16); acc[1] += __uint_as_float(d.x & 0xffff0000u);
    acc[2] += __uint_as_float(d.y << 16); acc[3] += __uint_as_float(d.y & 0xffff0000u);
  } else {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&d.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&d.y));
    acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
  }
}
template <int DT>
__device__ __forceinline__ uint2 finish(const float* acc) {
  uint2 r;
  if (DT == 0) {
    r.x = __float_as_uint(acc[0]);
    r.y = __float_as_uint(acc[1]);
  } else if (DT == 2) {
    __nv_bfloat162 a = __floats2bfloat162_rn(acc[0], acc[1]), b = __floats2bfloat162_rn(acc[2], acc[3]);
    r.x = *reinterpret_cast<uint32_t*>(&a);
    r.y = *reinterpret_cast<uint32_t*>(&b);
  } else {
    __half2 a = __floats2half2_rn(acc[0], acc[1]), b = __floats2half2_rn(acc[2], acc[3]);
    r.x = *reinterpret_cast<uint32_t*>(&a);
    r.y = *reinterpret_cast<uint32_t*>(&b);
  }
  return r;
}

template <int DT>
__global__ void __launch_bounds__(kLLThreads) allreduce_ll_kernel(const LLParams p) {
  const int me = p.peers.rank, world = p.peers.world;
  const uint64_t parity = p.flag & 1u;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  const uint64_t first = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;

  const uint64_t deadline = ptx::globaltimer() + p.timeout_ns;
  const uint4* mine = reinterpret_cast<const uint4*>(p.peers.base[me] + p.buf_off) + parity * world * p.capacity_units;
  // Packet `i` of source `s` in this rank's buffer; null (with the error word set) when it never arrived.
  auto receive = [&](int s, uint64_t i, uint2* d) {
    const uint4* slot = mine + s * p.capacity_units + i;
    uint4 v = ld_packet(slot);
    uint32_t spins = 0;
    while (v.y != p.flag || v.w != p.flag) {
      if ((++spins & 255u) == 0u && (*reinterpret_cast<volatile uint32_t*>(p.error) || ptx::globaltimer() > deadline)) {
        atomicCAS(p.error, 0u, 0x701u);
        return false;
      }
      v = ld_packet(slot);
    }
    *d = make_uint2(v.x, v.z);
    return true;
  };
  auto slot_at = [&](int peer, uint64_t i) {
    return reinterpret_cast<uint4*>(p.peers.base[peer] + p.buf_off) + (parity * world + me) * p.capacity_units + i;
  };

  if (p.mode == 0) {
    // all-reduce.  1. push my units to every peer's slot for this source
    for (uint64_t i = first; i < p.units; i += stride) {
      const uint2 d = p.in[i];
      for (int k = 1; k < world; ++k) st_packet(slot_at((me + k) % world, i), d, p.flag);
    }
    // 2. poll the peers' packets and reduce in rank order
    for (uint64_t i = first; i < p.units; i += stride) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < world; ++s) {
        uint2 d;
        if (s == me) d = p.in[i];
        else if (!receive(s, i, &d)) return;
        accumulate<DT>(acc, d);
      }
      p.out[i] = finish<DT>(acc);
    }
    return;
  }
  // The other three move one part per peer: part `peer` of the input for reduce-scatter and
  // all-to-all, the whole (one-part) input for all-gather.
  for (uint64_t i = first; i < p.units; i += stride) {
    for (int k = 1; k < world; ++k) {
      const int peer = (me + k) % world;
      st_packet(slot_at(peer, i), p.in[p.mode == 2 ? i : peer * p.units + i], p.flag);
    }
  }
  for (uint64_t i = first; i < p.units; i += stride) {
    if (p.mode == 1) {                                   // reduce-scatter: rank-ordered fp32 sum of my part
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < world; ++s) {
        uint2 d;
        if (s == me) d = p.in[me * p.units + i];
        else if (!receive(s, i, &d)) return;
        accumulate<DT>(acc, d);
      }
      p.out[i] = finish<DT>(acc);
    } else {                                             // all-gather / all-to-all: part s of the output came from s
      for (int s = 0; s < world; ++s) {
        uint2 d;
        if (s == me) d = p.in[p.mode == 2 ? i : me * p.units + i];
        else if (!receive(s, i, &d)) return;
        p.out[s * p.units + i] = d;
      }
    }
  }
}

}  // namespace

void allreduce_ll(const PeerBases& peers, uint64_t buf_off, uint64_t capacity_bytes, const void* in, void* out,
                  uint64_t bytes, int dtype, uint32_t epoch, cudaStream_t stream, uint64_t timeout_ms,
                  uint32_t* error) {
  collective_ll(0, peers, buf_off, capacity_bytes, in, out, bytes, dtype, epoch, stream, timeout_ms, error);
}

void collective_ll(int mode, const PeerBases& peers, uint64_t buf_off, uint64_t capacity_bytes, const void* in,
                   void* out, uint64_t bytes, int dtype, uint32_t epoch, cudaStream_t stream, uint64_t timeout_ms,
                   uint32_t* error) {
  PCCL_CHECK(mode >= 0 && mode <= 3, "LL collective: mode 0..3");
  PCCL_CHECK(bytes % 8 == 0 && bytes > 0, "LL all-reduce: size must be a positive multiple of 8 bytes");
  PCCL_CHECK(bytes <= capacity_bytes, "LL all-reduce: " << bytes << " bytes exceed the buffer's " << capacity_bytes);
  PCCL_CHECK(reinterpret_cast<uintptr_t>(in) % 8 == 0 && reinterpret_cast<uintptr_t>(out) % 8 == 0,
             "LL all-reduce: tensors must be 8-byte aligned");
  PCCL_CHECK(dtype >= 0 && dtype <= 2, "LL all-reduce: f32, f16 and bf16 only");
  PCCL_CHECK(epoch != 0, "LL all-reduce: the call number starts at 1");
  LLParams p{};
  p.peers = peers;
  p.buf_off = buf_off;
  p.capacity_units = capacity_bytes / 8;
  p.in = static_cast<const uint2*>(in);
  p.out = static_cast<uint2*>(out);
  p.units = bytes / 8;
  p.dtype = dtype;
  p.mode = mode;
  p.flag = epoch;
  p.error = error ? error : error_word();
  p.timeout_ns = timeout_ms * 1000000ull;
  // One unit per thread up to 128 CTAs, then a grid-stride loop.
  uint64_t grid = (p.units + kLLThreads - 1) / kLLThreads;
  if (grid > 128) grid = 128;
  // Every CTA polls for packets that the same CTA of each peer pushes: all CTAs must be resident.
  // (The grid follows from the message size alone, so it is the same on every rank; 128 CTAs of
  // 256 threads are far below the resident limit.)
  switch (dtype) {
    case 0: launch_coresident(allreduce_ll_kernel<0>, static_cast<uint32_t>(grid), kLLThreads, 0, stream, p, true); break;
    case 1: launch_coresident(allreduce_ll_kernel<1>, static_cast<uint32_t>(grid), kLLThreads, 0, stream, p, true); break;
    default: launch_coresident(allreduce_ll_kernel<2>, static_cast<uint32_t>(grid), kLLThreads, 0, stream, p, true); break;
  }
}

}  // namespace gemm
}  // namespace pccl
