/* MoE top-2 router for callers that must not allocate.
 *
 * Some callers cannot let a library allocate device memory on their behalf: a serving loop
 * that has handed all device memory to its own pool, code running inside a region where the
 * allocator is locked, or a host program written in C with no tensor library at hand.  The
 * router needs a few counters of scratch; pccl_moe_route_static() keeps them in a fixed array
 * that is part of the loaded module, so the call performs no device or host allocation and
 * takes plain pointers.
 *
 * This entry point has no counterpart in the reference.
 *
 * Limits and rules:
 *   - at most PCCL_MOE_ROUTE_STATIC_MAX_EXPERTS experts (a power of two, at least 2), hidden a
 *     multiple of 8, experts * hidden * 2 bytes at most 200 KB; anything else is refused with
 *     PCCL_ROUTE_STATIC_BAD_SHAPE and nothing is launched;
 *   - the first call on a device looks up the scratch array's address (once per device, with
 *     that device current) and therefore should come before any stream capture;
 *   - all calls on one device share the one scratch array.  Each call clears it on `stream`
 *     before its kernel, so calls on the same stream are safe back to back; calls that may
 *     overlap (different streams, different host threads without ordering) race on it.
 *
 * x [tokens][hidden] and wg [experts][hidden] are bf16 device pointers; topk_idx, topk_slot
 * (int32 [tokens][2]), topk_gate (float [tokens][2]) and expert_counts (uint32 [experts]) are
 * device pointers, each optional (null to skip).  `stream` is a cudaStream_t.
 * Returns 0 on success, otherwise one of the codes below; pccl_moe_route_static_strerror()
 * names them.
 */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PCCL_MOE_ROUTE_STATIC_MAX_EXPERTS 64

enum {
  PCCL_ROUTE_STATIC_OK = 0,
  PCCL_ROUTE_STATIC_BAD_SHAPE = 1,     /* experts / hidden / tokens outside the limits above */
  PCCL_ROUTE_STATIC_BAD_POINTER = 2,   /* x or wg null or not 16-byte aligned */
  PCCL_ROUTE_STATIC_SETUP_FAILED = 3,  /* the scratch array's address could not be obtained */
  PCCL_ROUTE_STATIC_LAUNCH_FAILED = 4  /* clearing the scratch or launching the kernel failed */
};

int pccl_moe_route_static(const void* x, const void* wg, int tokens, int hidden, int experts, int32_t* topk_idx,
                          float* topk_gate, int32_t* topk_slot, uint32_t* expert_counts, void* stream);

const char* pccl_moe_route_static_strerror(int code);

#ifdef __cplusplus
}
#endif
