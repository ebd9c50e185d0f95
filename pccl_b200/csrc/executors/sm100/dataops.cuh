// Data movers of the plan interpreter: vectorised peer copy / reduce / put and
// the multimem variants, for every plan dtype and reduce op.
//
// Work is cut into tiles of (threads x unroll) 16-byte vectors; the CTAs of a
// chain take tiles round-robin and a thread issues all of a tile's loads before
// it touches the first result, so several loads per thread are in flight over
// NVLink; a multi-source reduction additionally prefetches source s+1 while it
// folds source s.  Reductions accumulate in fp32 whatever the storage type and
// round once.  Ranges whose operands are not mutually 16-byte aligned, and the
// ragged head/tail of aligned ones, go through an element-wise path, so no
// element is dropped (the reference drops the n % (16/elem) tail:
// kernel/compute.h:25-43).
//
// Source pointers live in shared memory (SrcTable) because they are indexed by
// a run-time source number; everything else stays in registers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cstdint>

#include "../../ptx/multimem.cuh"
#include "../../ptx/sync.cuh"
#include "program.h"

namespace pccl {

// ---- per-dtype codecs: 16 bytes <-> fp32 lanes -------------------------------------------

template <int DT> struct Codec;

template <> struct Codec<kF32> {
  static constexpr int kLanes = 4;
  __device__ static __forceinline__ void unpack(uint4 v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  __device__ static __forceinline__ uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                      __float_as_uint(f[3]));
  }
  __device__ static __forceinline__ float load1(const void* p) {
    return *reinterpret_cast<const volatile float*>(p);
  }
  __device__ static __forceinline__ void store1(void* p, float f) { *reinterpret_cast<float*>(p) = f; }
};

template <> struct Codec<kF16> {
  static constexpr int kLanes = 8;
  __device__ static __forceinline__ void unpack(uint4 v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = p.x; f[2 * i + 1] = p.y;
    }
  }
  __device__ static __forceinline__ uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  __device__ static __forceinline__ float load1(const void* p) {
    unsigned short raw = *reinterpret_cast<const volatile unsigned short*>(p);
    return __half2float(__ushort_as_half(raw));
  }
  __device__ static __forceinline__ void store1(void* p, float f) {
    *reinterpret_cast<__half*>(p) = __float2half_rn(f);
  }
};

template <> struct Codec<kBF16> {
  static constexpr int kLanes = 8;
  __device__ static __forceinline__ void unpack(uint4 v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {   // bf16 -> f32 is a 16-bit shift
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static __forceinline__ uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  __device__ static __forceinline__ float load1(const void* p) {
    unsigned short raw = *reinterpret_cast<const volatile unsigned short*>(p);
    return __uint_as_float(static_cast<uint32_t>(raw) << 16);
  }
  __device__ static __forceinline__ void store1(void* p, float f) {
    *reinterpret_cast<__nv_bfloat16*>(p) = __float2bfloat16_rn(f);
  }
};

template <__nv_fp8_interpretation_t KIND> struct Fp8Codec {
  static constexpr int kLanes = 16;
  __device__ static __forceinline__ void unpack(uint4 v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        __half2_raw r = __nv_cvt_fp8x2_to_halfraw2(
            static_cast<__nv_fp8x2_storage_t>((w[i] >> (16 * h)) & 0xffffu), KIND);
        float2 p = __half22float2(*reinterpret_cast<__half2*>(&r));
        f[4 * i + 2 * h] = p.x; f[4 * i + 2 * h + 1] = p.y;
      }
    }
  }
  __device__ static __forceinline__ uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * i], f[4 * i + 1]), __NV_SATFINITE, KIND);
      uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * i + 2], f[4 * i + 3]), __NV_SATFINITE, KIND);
      w[i] = lo | (hi << 16);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  __device__ static __forceinline__ float load1(const void* p) {
    unsigned char raw = *reinterpret_cast<const volatile unsigned char*>(p);
    __half_raw r = __nv_cvt_fp8_to_halfraw(raw, KIND);
    return __half2float(*reinterpret_cast<__half*>(&r));
  }
  __device__ static __forceinline__ void store1(void* p, float f) {
    *reinterpret_cast<unsigned char*>(p) = __nv_cvt_float_to_fp8(f, __NV_SATFINITE, KIND);
  }
};
template <> struct Codec<kE4M3> : Fp8Codec<__NV_E4M3> {};
template <> struct Codec<kE5M2> : Fp8Codec<__NV_E5M2> {};

__device__ __forceinline__ float fold1(float a, float b, int op) {
  return op == kRedSum ? a + b : (op == kRedMax ? fmaxf(a, b) : fminf(a, b));
}

// ---- operands -------------------------------------------------------------------------------

struct SrcTable {                      // lives in shared memory, filled once per step
  const uint8_t* ptr[kMaxRanks];
  uint32_t remote_mask;                // bit s: source s is peer memory
  int count;
};

struct Span {                          // how a byte range splits into head / vectors / tail
  uint64_t head, nvec, tail_begin;
  bool uniform;                        // all operands share one misalignment mod 16
};

__device__ __forceinline__ Span make_span(const SrcTable& t, const uint8_t* dst, uint64_t bytes) {
  Span sp;
  const uint32_t mis = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(dst)) & 15u;
  sp.uniform = true;
  for (int s = 0; s < t.count; ++s)
    sp.uniform &= (static_cast<uint32_t>(reinterpret_cast<uintptr_t>(t.ptr[s])) & 15u) == mis;
  sp.head = mis ? 16 - mis : 0;
  if (sp.head > bytes) sp.head = bytes;
  sp.nvec = (bytes - sp.head) / 16;
  sp.tail_begin = sp.head + sp.nvec * 16;
  return sp;
}

__device__ __forceinline__ uint4 load_vec(const uint8_t* p, bool remote) {
  return remote ? ptx::ld_peer_v4(p) : ptx::ld_local_v4(p);
}

// ---- copy family (dtype independent) --------------------------------------------------------

__device__ __forceinline__ void bytes_copy(const uint8_t* src, uint8_t* dst, uint64_t begin, uint64_t end,
                                           uint32_t tid, uint32_t nthr) {
  for (uint64_t b = begin + tid; b < end; b += nthr)
    dst[b] = *reinterpret_cast<const volatile uint8_t*>(src + b);
}

// dst[0..bytes) = src[0..bytes).  kToMulticast: dst is a multicast address (multimem.st).
template <bool kToMulticast>
__device__ __noinline__ void copy_range(const SrcTable& t, uint8_t* dst, uint64_t bytes, uint32_t cta,
                                        uint32_t nctas) {
  constexpr int kU = 8;
  const uint8_t* src = t.ptr[0];
  const bool remote = t.remote_mask & 1u;
  const Span sp = make_span(t, dst, bytes);
  const uint32_t tid = threadIdx.x, nthr = blockDim.x;
  if (!sp.uniform) {          // byte-exact everywhere (multicast ranges are always aligned)
    if (!kToMulticast) bytes_copy(src, dst, 0, bytes, cta * nthr + tid, nctas * nthr);
    return;
  }
  if (cta == 0 && !kToMulticast) {
    bytes_copy(src, dst, 0, sp.head, tid, nthr);
    bytes_copy(src, dst, sp.tail_begin, bytes, tid, nthr);
  }
  src += sp.head;
  dst += sp.head;
  for (uint64_t t0 = static_cast<uint64_t>(cta) * nthr * kU; t0 < sp.nvec;
       t0 += static_cast<uint64_t>(nctas) * nthr * kU) {
    uint4 v[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const uint64_t i = t0 + tid + static_cast<uint64_t>(u) * nthr;
      if (i < sp.nvec) v[u] = load_vec(src + i * 16, remote);
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const uint64_t i = t0 + tid + static_cast<uint64_t>(u) * nthr;
      if (i < sp.nvec) {
        if (kToMulticast) ptx::mm_st_v4(dst + i * 16, v[u]); else ptx::st_v4(dst + i * 16, v[u]);
      }
    }
  }
}

// ---- reduce family ----------------------------------------------------------------------------

template <int DT>
__device__ __forceinline__ void scalar_fold(const SrcTable& t, uint8_t* dst, uint64_t begin, uint64_t end,
                                            int op, float scale, uint32_t tid, uint32_t nthr) {
  using C = Codec<DT>;
  constexpr int kE = 16 / C::kLanes;
  for (uint64_t b = begin + static_cast<uint64_t>(tid) * kE; b < end; b += static_cast<uint64_t>(nthr) * kE) {
    float acc = C::load1(t.ptr[0] + b);
    for (int s = 1; s < t.count; ++s) acc = fold1(acc, C::load1(t.ptr[s] + b), op);
    C::store1(dst + b, acc * scale);
  }
}

// dst = scale * fold(op, sources).  One source + scale != 1 is the "avg" epilogue.
template <int DT>
__device__ __noinline__ void reduce_range(const SrcTable& t, uint8_t* dst, uint64_t bytes, int op,
                                          float scale, uint32_t cta, uint32_t nctas) {
  using C = Codec<DT>;
  constexpr int kU = C::kLanes >= 16 ? 2 : 4;
  const Span sp = make_span(t, dst, bytes);
  const uint32_t tid = threadIdx.x, nthr = blockDim.x;
  if (!sp.uniform) {
    scalar_fold<DT>(t, dst, 0, bytes, op, scale, cta * nthr + tid, nctas * nthr);
    return;
  }
  if (cta == 0) {
    scalar_fold<DT>(t, dst, 0, sp.head, op, scale, tid, nthr);
    scalar_fold<DT>(t, dst, sp.tail_begin, bytes, op, scale, tid, nthr);
  }
  const int nsrc = t.count;
  for (uint64_t t0 = static_cast<uint64_t>(cta) * nthr * kU; t0 < sp.nvec;
       t0 += static_cast<uint64_t>(nctas) * nthr * kU) {
    uint64_t off[kU];
    bool live[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const uint64_t i = t0 + tid + static_cast<uint64_t>(u) * nthr;
      live[u] = i < sp.nvec;
      off[u] = sp.head + i * 16;
    }
    float acc[kU][C::kLanes];
    uint4 cur[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u)
      if (live[u]) cur[u] = load_vec(t.ptr[0] + off[u], t.remote_mask & 1u);
#pragma unroll
    for (int u = 0; u < kU; ++u) C::unpack(live[u] ? cur[u] : make_uint4(0, 0, 0, 0), acc[u]);
    if (nsrc > 1) {
#pragma unroll
      for (int u = 0; u < kU; ++u)
        if (live[u]) cur[u] = load_vec(t.ptr[1] + off[u], t.remote_mask >> 1 & 1u);
      for (int s = 1; s < nsrc; ++s) {
        uint4 nxt[kU];
        if (s + 1 < nsrc) {      // prefetch the next source before folding this one
#pragma unroll
          for (int u = 0; u < kU; ++u)
            if (live[u]) nxt[u] = load_vec(t.ptr[s + 1] + off[u], t.remote_mask >> (s + 1) & 1u);
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          float f[C::kLanes];
          C::unpack(live[u] ? cur[u] : make_uint4(0, 0, 0, 0), f);
#pragma unroll
          for (int l = 0; l < C::kLanes; ++l) acc[u][l] = fold1(acc[u][l], f[l], op);
          cur[u] = nxt[u];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kU; ++u)
      if (live[u]) {
        if (scale != 1.0f) {
#pragma unroll
          for (int l = 0; l < C::kLanes; ++l) acc[u][l] *= scale;
        }
        ptx::st_v4(dst + off[u], C::pack(acc[u]));
      }
  }
}

// ---- multimem reduce family ---------------------------------------------------------------------

template <int DT>
__device__ __forceinline__ uint4 mm_load(const uint8_t* mc, int op) {
  if (DT == kF32) return ptx::mm_ld_reduce_add_f32(mc);
  if (DT == kBF16) {
    return op == kRedSum ? ptx::mm_ld_reduce_add_bf16(mc)
                         : (op == kRedMax ? ptx::mm_ld_reduce_max_bf16(mc) : ptx::mm_ld_reduce_min_bf16(mc));
  }
  return op == kRedSum ? ptx::mm_ld_reduce_add_f16(mc)
                       : (op == kRedMax ? ptx::mm_ld_reduce_max_f16(mc) : ptx::mm_ld_reduce_min_f16(mc));
}

// dst = in-switch reduction of mc_src over all ranks.  kToMulticast: the result is
// broadcast straight back (one-pass allreduce of this rank's slice).
// Ranges are 16-byte aligned by construction (the host lowers others to SM steps).
template <int DT, bool kToMulticast>
__device__ __noinline__ void mm_reduce_range(const uint8_t* mc_src, uint8_t* dst, uint64_t bytes, int op,
                                             uint32_t cta, uint32_t nctas) {
  constexpr int kU = 8;
  const uint64_t nvec = bytes / 16;
  const uint32_t tid = threadIdx.x, nthr = blockDim.x;
  for (uint64_t t0 = static_cast<uint64_t>(cta) * nthr * kU; t0 < nvec;
       t0 += static_cast<uint64_t>(nctas) * nthr * kU) {
    uint4 v[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const uint64_t i = t0 + tid + static_cast<uint64_t>(u) * nthr;
      if (i < nvec) v[u] = mm_load<DT>(mc_src + i * 16, op);
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const uint64_t i = t0 + tid + static_cast<uint64_t>(u) * nthr;
      if (i < nvec) {
        if (kToMulticast) ptx::mm_st_v4(dst + i * 16, v[u]); else ptx::st_v4(dst + i * 16, v[u]);
      }
    }
  }
}

}  // namespace pccl
