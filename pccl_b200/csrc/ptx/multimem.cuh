// multimem.* wrappers: loads that the NVSwitch reduces over every rank's copy
// of an address, and stores that it delivers to every rank (NVLS).  Addresses
// are multicast virtual addresses obtained from a CUDA multicast object.
// One call moves 16 bytes.  (The reference wires only the bf16x2 forms:
// csrc/plugins/cuda/kernel/multimem_helpers.h:9-50.)
#pragma once
#include <cstdint>

namespace pccl {
namespace ptx {

enum class MmOp { kAdd, kMin, kMax };

__device__ __forceinline__ uint4 mm_ld_reduce_add_f32(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ uint4 mm_ld_reduce_add_bf16(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ uint4 mm_ld_reduce_add_f16(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
#define PCCL_MM_MINMAX(NAME, OP, TY)                                                        \
  __device__ __forceinline__ uint4 NAME(const void* mc) {                                   \
    uint4 v;                                                                                \
    asm volatile("multimem.ld_reduce.relaxed.sys.global." OP ".v4." TY " {%0,%1,%2,%3}, [%4];" \
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");      \
    return v;                                                                               \
  }
PCCL_MM_MINMAX(mm_ld_reduce_min_bf16, "min", "bf16x2")
PCCL_MM_MINMAX(mm_ld_reduce_max_bf16, "max", "bf16x2")
PCCL_MM_MINMAX(mm_ld_reduce_min_f16, "min", "f16x2")
PCCL_MM_MINMAX(mm_ld_reduce_max_f16, "max", "f16x2")
#undef PCCL_MM_MINMAX

// A multicast store is a bit copy, so one 16-byte form serves every dtype.
__device__ __forceinline__ void mm_st_v4(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// Signal post delivered to every rank's copy of a flag word.
__device__ __forceinline__ void mm_red_add_u32(uint32_t* mc, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

}  // namespace ptx
}  // namespace pccl
