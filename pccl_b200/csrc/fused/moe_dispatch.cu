// MoE router + dispatch in one kernel.
//
// One warp per token: router logits x . Wg^T (Wg staged in shared memory), softmax over the
// experts, top-2 with the two gates renormalised to sum to one.  For each of the two choices
// the warp claims a slot in the destination region (an atomic counter per expert) and pushes
// the token's row straight into the expert rank's receive buffer over NVLink, with a
// {token * 2 + k, gate} record beside it.  The last CTA to finish writes the per-region row
// counts at every expert rank and posts this rank's dispatch flag there.
//
// Scratch: E + 1 u32 words (slot counters per expert, finished-CTA count) that must be zero
// at launch.  With `dispatch == 0` the kernel only routes (indices, gates, slots, counts), which
// is also how the single-GPU tests check the router on its own.
// The reference has no MoE operator (nearest: the alltoall template, pccl/dsl/algorithms/ring.py).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../common/util.h"
#include "../engine/cuda_driver.h"
#include "../ptx/sync.cuh"
#include "gemm_host.h"
#include "moe_route.cuh"

namespace pccl {
namespace gemm {

void moe_route_dispatch(const PeerBases& peers, const MoeBuffers& buf, const void* x, const void* wg, int tokens,
                        int hidden, int experts, uint32_t* scratch, int32_t* topk_idx, float* topk_gate,
                        int32_t* topk_slot, uint32_t* expert_counts, bool dispatch, uint32_t epoch,
                        cudaStream_t stream) {
  PCCL_CHECK(hidden % 8 == 0, "MoE router: hidden must be a multiple of 8");
  PCCL_CHECK(static_cast<size_t>(experts) * hidden * 2 <= 200 * 1024,
             "MoE router: experts x hidden x 2 bytes of router weight must fit in 200 KB of shared memory");
  PCCL_CHECK(experts >= 2 && experts <= kMoeRouteMaxExperts && (experts & (experts - 1)) == 0,
             "MoE router: experts must be a power of two in [2, " << kMoeRouteMaxExperts << "]");
  PCCL_CHECK(experts % peers.world == 0, "MoE router: experts must divide over the ranks");
  MoeRouteParams p{};
  for (int r = 0; r < peers.world; ++r) p.base[r] = peers.base[r];
  p.rank = peers.rank;
  p.world = peers.world;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.wg = static_cast<const __nv_bfloat16*>(wg);
  p.recv_off = buf.recv_off; p.meta_off = buf.meta_off; p.counts_off = buf.counts_off; p.ready_off = buf.ready_off;
  p.scratch = scratch;
  p.topk_idx = topk_idx; p.topk_gate = topk_gate; p.topk_slot = topk_slot; p.expert_counts = expert_counts;
  p.tokens = tokens; p.hidden = hidden; p.experts = experts;
  p.local_experts = experts / peers.world;
  p.cap = buf.cap;
  p.dispatch = dispatch ? 1 : 0;
  p.epoch = epoch;
  PCCL_CUDA(cudaMemsetAsync(scratch, 0, (experts + 1) * sizeof(uint32_t), stream));
  PCCL_CUDA(launch_moe_route(p, stream));
}

}  // namespace gemm
}  // namespace pccl
