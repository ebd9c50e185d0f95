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

// Tuning word set by the host (PCCL_MOVER_TUNING): bit 0 = keep two register tiles in flight per
// thread in copy / reduce steps; bit 1 = only one tile in multimem steps.  Off by default: with unconditional loads one tile of 8 vectors per thread already
// saturates NVLink, and the second tile measured a few percent slower.
__constant__ uint32_t g_mover_tuning = 0;

// Local and peer data are both read with weak L2 loads (one instruction, no branch).
__device__ __forceinline__ uint4 load_vec(const uint8_t* p, bool) { return ptx::ld_local_v4(p); }

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
  const uint32_t tid = threadIdx.x;
  constexpr uint32_t nthr = kInterpThreads;     // compile-time: per-vector offsets become immediates
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
  const uint64_t tile = static_cast<uint64_t>(nthr) * kU, stride = static_cast<uint64_t>(nctas) * tile;
  // Loads are unconditional (see ReduceTile::load); lanes past the end re-read the last vector.
  auto load = [&](uint4* v, uint64_t first) {
    if (first + kU * nthr <= sp.nvec) {
      const uint8_t* p = src + (first + tid) * 16;
#pragma unroll
      for (int u = 0; u < kU; ++u) v[u] = load_vec(p + u * nthr * 16, remote);
    } else {
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const uint64_t i = first + tid + u * nthr;
        v[u] = load_vec(src + (i < sp.nvec ? i : sp.nvec - 1) * 16, remote);
      }
    }
  };
  auto store = [&](const uint4* v, uint64_t first) {
    uint8_t* p = dst + (first + tid) * 16;
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      if (first + tid + u * nthr < sp.nvec) {
        if (kToMulticast) ptx::mm_st_v4(p + u * nthr * 16, v[u]); else ptx::st_v4(p + u * nthr * 16, v[u]);
      }
    }
  };
  // Two tiles in flight: the loads of the next tile are issued before this one is stored.
  uint4 a[kU], b[kU];
  uint64_t t0 = static_cast<uint64_t>(cta) * tile;
  if (t0 >= sp.nvec) return;
  if (!(g_mover_tuning & 1u)) {
    for (; t0 < sp.nvec; t0 += stride) { load(a, t0); store(a, t0); }
    return;
  }
  load(a, t0);
  while (true) {
    const uint64_t t1 = t0 + stride;
    if (t1 < sp.nvec) load(b, t1);
    store(a, t0);
    if (t1 >= sp.nvec) break;
    const uint64_t t2 = t1 + stride;
    if (t2 < sp.nvec) load(a, t2);
    store(b, t1);
    if (t2 >= sp.nvec) break;
    t0 = t2;
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

// One tile of a reduce: kN sources x kU vectors per thread.  Tiles are software-pipelined in
// registers: the loads of tile i+1 are issued before tile i is folded and stored, so that a
// thread keeps 2 * kN * kU independent 16-byte loads in flight (peer latency is microseconds).
template <int DT, int kN, int kU>
struct ReduceTile {
  using C = Codec<DT>;
  uint4 raw[kN][kU];

  __device__ __forceinline__ void load(const SrcTable& t, int nsrc, uint64_t first, uint64_t head, uint64_t nvec,
                                       uint32_t tid) {
#pragma unroll
    for (int s = 0; s < kN; ++s) {
      {
        // A slot beyond the source count re-reads source 0 (its value is never folded): every
        // register of the tile is written unconditionally.
        const int ss = s < nsrc ? s : 0;
        const bool remote = (t.remote_mask >> ss) & 1u;
        // Loads are unconditional (a conditionally assigned register makes the compiler wait for
        // each load before issuing the next); lanes past the end re-read the last vector.
        if (first + kU * kInterpThreads <= nvec) {
          const uint8_t* p = t.ptr[ss] + head + (first + tid) * 16;
#pragma unroll
          for (int u = 0; u < kU; ++u) raw[s][u] = load_vec(p + u * kInterpThreads * 16, remote);
        } else {
          const uint8_t* p = t.ptr[ss] + head;
#pragma unroll
          for (int u = 0; u < kU; ++u) {
            const uint64_t i = first + tid + u * kInterpThreads;
            raw[s][u] = load_vec(p + (i < nvec ? i : nvec - 1) * 16, remote);
          }
        }
      }
    }
  }

  __device__ __forceinline__ void fold_store(int nsrc, uint8_t* dst, uint64_t first, uint64_t head, uint64_t nvec,
                                             int op, float scale, uint32_t tid) const {
    uint8_t* out = dst + head + (first + tid) * 16;
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      if (first + tid + u * kInterpThreads >= nvec) continue;
      float acc[C::kLanes];
      C::unpack(raw[0][u], acc);
#pragma unroll
      for (int s = 1; s < kN; ++s) {
        if (s < nsrc) {
          float f[C::kLanes];
          C::unpack(raw[s][u], f);
#pragma unroll
          for (int l = 0; l < C::kLanes; ++l) acc[l] = fold1(acc[l], f[l], op);
        }
      }
      if (scale != 1.0f) {
#pragma unroll
        for (int l = 0; l < C::kLanes; ++l) acc[l] *= scale;
      }
      ptx::st_v4(out + u * kInterpThreads * 16, C::pack(acc));
    }
  }
};

template <int DT, int kN, int kU>
__device__ __forceinline__ void reduce_tiles(const SrcTable& t, uint8_t* dst, const Span& sp, int op, float scale,
                                             uint32_t cta, uint32_t nctas) {
  const uint32_t tid = threadIdx.x;
  constexpr uint32_t nthr = kInterpThreads;     // compile-time: per-vector offsets become immediates
  const int nsrc = t.count;
  const uint64_t tile = static_cast<uint64_t>(nthr) * kU, stride = static_cast<uint64_t>(nctas) * tile;
  ReduceTile<DT, kN, kU> a, b;
  uint64_t t0 = static_cast<uint64_t>(cta) * tile;
  if (t0 >= sp.nvec) return;
  if (!(g_mover_tuning & 1u)) {
    for (; t0 < sp.nvec; t0 += stride) {
      a.load(t, nsrc, t0, sp.head, sp.nvec, tid);
      a.fold_store(nsrc, dst, t0, sp.head, sp.nvec, op, scale, tid);
    }
    return;
  }
  a.load(t, nsrc, t0, sp.head, sp.nvec, tid);
  while (true) {
    const uint64_t t1 = t0 + stride;
    if (t1 < sp.nvec) b.load(t, nsrc, t1, sp.head, sp.nvec, tid);
    a.fold_store(nsrc, dst, t0, sp.head, sp.nvec, op, scale, tid);
    if (t1 >= sp.nvec) break;
    const uint64_t t2 = t1 + stride;
    if (t2 < sp.nvec) a.load(t, nsrc, t2, sp.head, sp.nvec, tid);
    b.fold_store(nsrc, dst, t1, sp.head, sp.nvec, op, scale, tid);
    if (t2 >= sp.nvec) break;
    t0 = t2;
  }
}

// dst = scale * fold(op, sources).  One source + scale != 1 is the "avg" epilogue.
template <int DT>
__device__ __noinline__ void reduce_range(const SrcTable& t, uint8_t* dst, uint64_t bytes, int op,
                                          float scale, uint32_t cta, uint32_t nctas) {
  using C = Codec<DT>;
  constexpr bool kWide = C::kLanes >= 16;           // fp8: 16 accumulators per vector
  const Span sp = make_span(t, dst, bytes);
  const uint32_t tid = threadIdx.x;
  constexpr uint32_t nthr = kInterpThreads;     // compile-time: per-vector offsets become immediates
  if (!sp.uniform) {
    scalar_fold<DT>(t, dst, 0, bytes, op, scale, cta * nthr + tid, nctas * nthr);
    return;
  }
  if (cta == 0) {
    scalar_fold<DT>(t, dst, 0, sp.head, op, scale, tid, nthr);
    scalar_fold<DT>(t, dst, sp.tail_begin, bytes, op, scale, tid, nthr);
  }
  // 8 loads per tile and thread (4 for fp8), two tiles in flight.
  if (t.count <= 1) reduce_tiles<DT, 1, 4>(t, dst, sp, op, scale, cta, nctas);
  else if (t.count == 2) reduce_tiles<DT, 2, kWide ? 2 : 4>(t, dst, sp, op, scale, cta, nctas);
  else if (t.count <= 4) reduce_tiles<DT, 4, kWide ? 1 : 2>(t, dst, sp, op, scale, cta, nctas);
  else reduce_tiles<DT, 8, 1>(t, dst, sp, op, scale, cta, nctas);
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
  const uint32_t tid = threadIdx.x;
  constexpr uint32_t nthr = kInterpThreads;
  const uint64_t tile = static_cast<uint64_t>(nthr) * kU, stride = static_cast<uint64_t>(nctas) * tile;
  auto load = [&](uint4* v, uint64_t first) {
    if (first + kU * nthr <= nvec) {
      const uint8_t* p = mc_src + (first + tid) * 16;
#pragma unroll
      for (int u = 0; u < kU; ++u) v[u] = mm_load<DT>(p + u * nthr * 16, op);
    } else {
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const uint64_t i = first + tid + u * nthr;
        v[u] = mm_load<DT>(mc_src + (i < nvec ? i : nvec - 1) * 16, op);
      }
    }
  };
  auto store = [&](const uint4* v, uint64_t first) {
    uint8_t* p = dst + (first + tid) * 16;
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      if (first + tid + u * nthr < nvec) {
        if (kToMulticast) ptx::mm_st_v4(p + u * nthr * 16, v[u]); else ptx::st_v4(p + u * nthr * 16, v[u]);
      }
    }
  };
  // Two tiles in flight by default (in-switch reductions have a longer round trip than peer
  // loads); bit 1 of the tuning word selects one tile.
  uint4 a[kU], b[kU];
  uint64_t t0 = static_cast<uint64_t>(cta) * tile;
  if (t0 >= nvec) return;
  if (g_mover_tuning & 2u) {
    for (; t0 < nvec; t0 += stride) { load(a, t0); store(a, t0); }
    return;
  }
  load(a, t0);
  while (true) {
    const uint64_t t1 = t0 + stride;
    if (t1 < nvec) load(b, t1);
    store(a, t0);
    if (t1 >= nvec) break;
    const uint64_t t2 = t1 + stride;
    if (t2 < nvec) load(a, t2);
    store(b, t1);
    if (t2 >= nvec) break;
    t0 = t2;
  }
}

}  // namespace pccl
