// pccl_moe_route_static(): the MoE router kernel with its scratch counters in a fixed
// device array of this module instead of caller- or library-allocated memory.
// See moe_route_static.h for the contract.
#include "moe_route_static.h"

#include <cuda_runtime.h>

#include <mutex>

#include "moe_route.cuh"

namespace {

static_assert(PCCL_MOE_ROUTE_STATIC_MAX_EXPERTS == pccl::gemm::kMoeRouteMaxExperts, "limits must agree");

// Slot counter per expert plus the finished-CTA count.
static __device__ __align__(256) uint32_t g_route_scratch[PCCL_MOE_ROUTE_STATIC_MAX_EXPERTS + 1];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
uint32_t* g_scratch_address[kMaxDevices] = {};

// Address of the scratch array on the current device; looked up once per device.
uint32_t* scratch_for_current_device() {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_address[device]) {
    uint32_t* ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_route_scratch) != cudaSuccess) return nullptr;
    g_scratch_address[device] = ptr;
  }
  return g_scratch_address[device];
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int pccl_moe_route_static(
    const void* x, const void* wg, int tokens, int hidden, int experts, int32_t* topk_idx, float* topk_gate,
    int32_t* topk_slot, uint32_t* expert_counts, void* stream) {
  if (tokens < 1 || hidden < 8 || hidden % 8 != 0 || experts < 2 || experts > PCCL_MOE_ROUTE_STATIC_MAX_EXPERTS ||
      (experts & (experts - 1)) != 0 || static_cast<long long>(experts) * hidden * 2 > 200 * 1024)
    return PCCL_ROUTE_STATIC_BAD_SHAPE;
  if (!x || !wg || reinterpret_cast<uintptr_t>(x) % 16 != 0 || reinterpret_cast<uintptr_t>(wg) % 16 != 0)
    return PCCL_ROUTE_STATIC_BAD_POINTER;
  uint32_t* scratch = scratch_for_current_device();
  if (!scratch) return PCCL_ROUTE_STATIC_SETUP_FAILED;

  pccl::gemm::MoeRouteParams p{};
  p.rank = 0;
  p.world = 1;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.wg = static_cast<const __nv_bfloat16*>(wg);
  p.scratch = scratch;
  p.topk_idx = topk_idx;
  p.topk_gate = topk_gate;
  p.topk_slot = topk_slot;
  p.expert_counts = expert_counts;
  p.tokens = tokens;
  p.hidden = hidden;
  p.experts = experts;
  p.local_experts = experts;
  p.dispatch = 0;
  p.epoch = 1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // Only the words this shape uses have to start at zero.
  if (cudaMemsetAsync(scratch, 0, (experts + 1) * sizeof(uint32_t), s) != cudaSuccess)
    return PCCL_ROUTE_STATIC_LAUNCH_FAILED;
  if (pccl::gemm::launch_moe_route(p, s) != cudaSuccess) return PCCL_ROUTE_STATIC_LAUNCH_FAILED;
  return PCCL_ROUTE_STATIC_OK;
}

extern "C" __attribute__((visibility("default"))) const char* pccl_moe_route_static_strerror(int code) {
  switch (code) {
    case PCCL_ROUTE_STATIC_OK: return "ok";
    case PCCL_ROUTE_STATIC_BAD_SHAPE:
      return "shape outside the limits: experts a power of two in [2, 64], hidden a multiple of 8, "
             "experts * hidden * 2 bytes at most 200 KB, tokens at least 1";
    case PCCL_ROUTE_STATIC_BAD_POINTER: return "x and wg must be non-null, 16-byte aligned device pointers";
    case PCCL_ROUTE_STATIC_SETUP_FAILED: return "could not obtain the address of the scratch array on this device";
    case PCCL_ROUTE_STATIC_LAUNCH_FAILED: return "clearing the scratch array or launching the kernel failed";
    default: return "unknown code";
  }
}
