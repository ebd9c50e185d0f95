// The two-SM form of the persistent bf16 GEMM: one tcgen05.mma.cta_group::2 instruction drives the
// tensor cores of a pair of SMs on a 256 x 256 tile.
//
// The kernel runs as clusters of two CTAs.  CTA r of a pair owns rows [128 r, 128 r + 128) of the
// tile: it loads its own 128 x 64 block of A and its own *half* of the B block (128 of the 256
// weight rows) per pipeline stage, keeps its half of the accumulator (128 lanes x 256 columns) in
// its own tensor memory and stores its own rows.  The instruction, issued by one thread of the
// even CTA, reads A and B from both CTAs' shared memory, so every byte of B is loaded and held
// once per pair instead of once per SM: a stage costs 32 KB per CTA instead of 48 KB, which buys
// six pipeline stages instead of four, and the shared-memory traffic per flop drops by a quarter.
//
// Hand-off between the CTAs (never a multicast load):
//   * each CTA issues its own plain TMA loads, in the cta_group::2 form whose completion bytes are
//     counted on the *even* CTA's "full" barrier (the odd CTA passes that barrier's address with
//     the pair bit cleared), after registering its expected bytes there with a remote
//     mbarrier.arrive.expect_tx;
//   * tcgen05.commit with a two-CTA mask arrives on the "stage free" and "accumulator ready"
//     barriers of both CTAs at once;
//   * the odd CTA's epilogue warps release an accumulator with a remote mbarrier.arrive on the
//     even CTA's barrier;
//   * cluster-wide barriers bracket the kernel (barrier initialisation, and no CTA exits while its
//     partner may still read its shared memory or signal its barriers).
// Roles, policies, bounded waits and error reporting are those of umma_gemm_kernel.  Policies see
// 128-row blocks as before: the pair processes blocks (2 i, 2 i + 1) of one n-tile together.
// Split tail: tiles are handed out one per pair and round, so a tile count that is not a multiple of
// the pair count leaves most pairs idle in the last round (8192 x 1792: 224 tiles on 74 pairs, two
// tiles in round four).  When the launcher finds at most half the pairs busy in that round it cuts
// each of those tiles along K into slices, one per idle pair; every slice writes its fp32 partial
// accumulator to a workspace, counts itself in, waits (bounded) for the other slices of its tile,
// and the warps of all slices then share the sum and the store of the tile.
// The tile width is a launch parameter (Problem::bn, a multiple of 32 up to 256): the launcher
// picks the width whose tile count divides best over the SM pairs, because with whole 256-column
// tiles a shape like 8192 x 1792 leaves 3.03 rounds of work to be done in 4.
#pragma once
#include "umma_gemm.cuh"

namespace pccl {
namespace gemm {

constexpr int kStages2 = 6;
constexpr uint32_t kBytesA2 = kBM * kBK * 2;                     // this CTA's 128 x 64 block of A
constexpr uint32_t kBytesB2 = (kBN / 2) * kBK * 2;               // this CTA's half of the 256 x 64 block of B
constexpr uint32_t kStageBytes2 = kBytesA2 + kBytesB2;           // 32 KB
constexpr uint32_t kSmemBytes2 = kStages2 * kStageBytes2 + 4 * kEpiWarpBytes + 1024;
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;                      // clears the bit that tells the pair's CTAs apart

namespace ptx2 {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory object in the even CTA of the pair.
__device__ __forceinline__ uint32_t leader_addr(const void* p) { return ptx::smem_u32(p) & kPeerMask; }

__device__ __forceinline__ void mbar_expect_tx_leader(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(leader_addr(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(leader_addr(bar)) : "memory");
}
// Plain (non-multicast) tile load into this CTA's shared memory; completion bytes go to the even
// CTA's barrier.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(ptx::smem_u32(smem_dst)), "l"(map), "r"(leader_addr(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_out, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_u32(smem_out)),
               "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem of both CTAs] (+)= A * B^T with M = 256 over the pair.  One thread of the even CTA issues.
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on `bar` (same offset) in both CTAs once all MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(ptx::smem_u32(bar)), "h"(mask) : "memory");
}

}  // namespace ptx2

// One unit of a pair's work: a whole tile, or (in the split tail) k-blocks [kb_begin, kb_end) of one.
struct WorkItem {
  int tile, kb_begin, kb_end, slice;
  bool partial;
};
__device__ __forceinline__ WorkItem decode_item(const Problem& g, int item, int k_blocks) {
  WorkItem w;
  if (item < g.tail_first) {
    w.tile = item; w.kb_begin = 0; w.kb_end = k_blocks; w.slice = 0; w.partial = false;
  } else {
    const int j = item - g.tail_first;
    w.tile = g.tail_first + j / g.tail_slices;
    w.slice = j % g.tail_slices;
    w.kb_begin = w.slice * g.tail_kb;
    w.kb_end = min(k_blocks, w.kb_begin + g.tail_kb);
    w.partial = true;
  }
  return w;
}

struct Pipe2 {
  uint64_t full[kStages2];      // used in the even CTA: 2 arrivals (one per CTA's producer) + 64 KB
  uint64_t empty[kStages2];     // one per CTA, released by the pair-wide commit
  uint64_t acc_full[2];         // one per CTA, released by the pair-wide commit
  uint64_t acc_empty[2];        // used in the even CTA: 8 arrivals (4 epilogue warps of each CTA)
  uint32_t tmem_base;
  uint32_t stored_count;
};

// The 128-row block that CTA `half` of a pair owns in `tile`: its index, whether it exists (the
// second block of the last pair of an odd count does not; the CTA then loads its partner's block so
// that the MMA has defined operands, and stores nothing), the n-tile and the pair index.
struct HalfBlock {
  int mb, nb, mb2;
  bool present;
};
template <class Policy>
__device__ __forceinline__ HalfBlock half_block(const typename Policy::Params& p, const Problem& g, int tile, int half) {
  HalfBlock hb;
  if constexpr (Policy::kRaggedPairs) {
    Policy::ragged_pair(p, g, tile, half, &hb.mb, &hb.present, &hb.nb);
    hb.mb2 = 0;
  } else {
    Policy::pair_coords(p, g, tile, &hb.mb2, &hb.nb);
    hb.mb = 2 * hb.mb2 + half;
    hb.present = hb.mb < g.tiles_m;
  }
  return hb;
}

// Epilogue of one K-slice of a split tile (one epilogue warp: TMEM lanes [32 quarter, +32) of this
// CTA's half).  Both directions are coalesced: the partial accumulator goes through the warp's
// staging buffer so that a store instruction writes whole 128-byte lines of the workspace, and in
// the sum a load instruction reads 512 contiguous bytes of one row.  Returns false when a wait ran out.
template <class Policy>
__device__ __forceinline__ bool split_tail_epilogue(const typename Policy::Params& p, const Problem& g,
                                                    const WorkItem& work, int mb2, int nb, int half, int quarter,
                                                    int lane, uint32_t tmem_acc, uint64_t* acc_empty, uint8_t* stage_buf,
                                                    uint64_t deadline, const volatile uint32_t* abort_flag) {
  static_assert(Policy::kOutPer32 == 32, "the split tail sums plain accumulators");
  const int t = work.tile - g.tail_first;                       // tail tile number
  const int slices = g.tail_slices;
  float* tile_ws = g.tail_ws + static_cast<size_t>(t) * slices * 2 * kBM * kBN;
  // 1. this warp's 32 rows of the partial accumulator -> workspace (fp32, row-major, 256 floats per row)
  float* rows = tile_ws + (static_cast<size_t>(work.slice * 2 + half) * kBM + quarter * 32) * kBN;
  const uint32_t taddr = tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
  for (int c = 0; c < g.bn; c += 32) {
    uint32_t v[32];
    ptx::tmem_ld_32x32b_x32(taddr + c, v);
    ptx::tmem_ld_wait();
    // lane = row: 8 chunks of 16 bytes, chunk index XOR-swizzled by the row against bank conflicts
#pragma unroll
    for (int i = 0; i < 8; ++i)
      *reinterpret_cast<uint4*>(stage_buf + lane * 128 + ((i ^ (lane & 7)) * 16)) =
          make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    __syncwarp();
    // 8 lanes write one row's 128 bytes, 4 rows per instruction
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int r = it * 4 + lane / 8, j = lane % 8;
      const uint4 val = *reinterpret_cast<const uint4*>(stage_buf + r * 128 + ((j ^ (r & 7)) * 16));
      *reinterpret_cast<uint4*>(rows + static_cast<size_t>(r) * kBN + c + 4 * j) = val;
    }
    __syncwarp();
  }
  ptx::tc_fence_before_sync();
  __syncwarp();
  uint32_t* arrived = g.tail_counters + t;
  uint32_t* finished = g.tail_counters + kTailMaxTiles + t;
  const uint32_t everyone = 8u * static_cast<uint32_t>(slices);  // 4 warps x 2 CTAs x slices
  uint32_t ok = 1;
  if (lane == 0) {
    ptx2::mbar_arrive_leader(acc_empty);                         // the accumulator is free again
    ptx::fence_gpu();
    ptx::red_release_gpu_add(arrived, 1u);
    // 2. wait until every slice of this tile is in the workspace
    uint32_t spins = 0;
    while (ptx::ld_acquire_gpu(arrived) < everyone) {
      if ((++spins & 63u) == 0u && (*abort_flag || ptx::globaltimer() > deadline)) { ok = 0; break; }
      __nanosleep(40);
    }
  }
  ok = __shfl_sync(0xffffffffu, ok, 0);
  if (!ok) return false;
  // 3. sum the slices.  Unit = 128 consecutive floats of one of the tile's 256 rows (a lane owns 4 of
  //    them); the warps of all slices take units round-robin.
  const int segments = g.bn / 128;
  const int units = 2 * kBM * segments;
  const int wid = (work.slice * 2 + half) * 4 + quarter, warps = static_cast<int>(everyone);
  //    Eight units are in flight at a time so that the loop pays one L2 round trip per slice, not per unit.
  constexpr int kBatch = 8;
  const size_t slice_pitch = static_cast<size_t>(2) * kBM * kBN;
  for (int u0 = wid; u0 < units; u0 += kBatch * warps) {
    float acc[kBatch][4];
    size_t at[kBatch];
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      const int u = min(u0 + b * warps, units - 1);               // clamped: extra lanes re-read a valid unit
      at[b] = static_cast<size_t>(u / segments) * kBN + (u % segments) * 128 + lane * 4;
      acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0.f;
    }
#pragma unroll 1
    for (int s = 0; s < slices; ++s) {
      uint4 raw[kBatch];
#pragma unroll
      for (int b = 0; b < kBatch; ++b) raw[b] = ptx::ld_local_v4(tile_ws + s * slice_pitch + at[b]);
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        acc[b][0] += __uint_as_float(raw[b].x); acc[b][1] += __uint_as_float(raw[b].y);
        acc[b][2] += __uint_as_float(raw[b].z); acc[b][3] += __uint_as_float(raw[b].w);
      }
    }
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      const int u = u0 + b * warps;
      if (u >= units) break;
      const int row256 = u / segments, seg = u % segments;
      const int mb = 2 * mb2 + row256 / kBM, r = row256 % kBM;
      const int col = nb * g.bn + seg * 128 + lane * 4;
      if (mb >= g.tiles_m || mb * kBM + r >= g.M || col >= g.N) continue;
      uint8_t* dst = Policy::tile_base(p, g, mb) + static_cast<int64_t>(r) * Policy::row_pitch(p, g);
      __nv_bfloat162 lo = __floats2bfloat162_rn(acc[b][0], acc[b][1]), hi = __floats2bfloat162_rn(acc[b][2], acc[b][3]);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&lo);
      packed.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(dst + static_cast<int64_t>(col) * 2) = packed;   // N % 8 == 0: 4 columns never straddle N
    }
  }
  // 4. the last warp to finish puts the tile's counters back to zero for the next launch
  __syncwarp();
  if (lane == 0) {
    if (atomicAdd(finished, 1u) + 1u == everyone) {
      atomicExch(arrived, 0u);
      atomicExch(finished, 0u);
    }
  }
  return true;
}

template <class Policy>
__global__ void __launch_bounds__(kMaxThreads, 1)
umma_gemm2_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                  const Problem g, const typename Policy::Params p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ Pipe2 pipe;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const volatile uint32_t* abort_flag = g.error;
  const uint64_t deadline = ptx::globaltimer() + g.timeout_ns;
  const int half = static_cast<int>(ptx2::cluster_ctarank());      // 0 = even CTA (issues the MMAs)

  // Auxiliary CTAs (an even number: whole clusters) take no part in the GEMM pipeline or its
  // cluster barriers.
  const int aux = Policy::aux_ctas(p);
  if (static_cast<int>(blockIdx.x) < aux) {
    Policy::aux_main(p, g, blockIdx.x, aux, deadline, abort_flag, smem);
    return;
  }
  const int pair = (blockIdx.x - aux) >> 1, num_pairs = (gridDim.x - aux) >> 1;
  if (threadIdx.x == 0) trace_stamp(g, 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages2; ++s) { ptx::mbar_init(&pipe.full[s], 2); ptx::mbar_init(&pipe.empty[s], 1); }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&pipe.acc_full[a], 1);
      ptx::mbar_init(&pipe.acc_empty[a], 8);
    }
    pipe.stored_count = 0;
    ptx::mbar_init_fence();
    ptx::tma_prefetch_desc(&tma_a);
    ptx::tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    ptx2::tmem_alloc_pair(&pipe.tmem_base, kTmemCols);
    ptx2::tmem_relinquish_pair();
  }
  ptx::tc_fence_before_sync();
  ptx2::cluster_sync();                      // both CTAs' barriers exist before anyone signals the partner
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = pipe.tmem_base;

  // The pair walks the policy's order of 256-row blocks: block pair i = 128-row blocks 2i, 2i+1.
  const int tiles_m = Policy::prepare(p, g, deadline, abort_flag);
  const int k_blocks = (g.K + kBK - 1) / kBK;
  const bool split = Policy::kSplitTail && g.tail_first < (g.tiles_m + 1) / 2 * g.tiles_n;
  int num_tiles = 0;
  if (tiles_m >= 0) {
    if constexpr (Policy::kRaggedPairs) num_tiles = Policy::pair_tiles(p, g);
    else num_tiles = split ? g.num_items : (g.tiles_m + 1) / 2 * g.tiles_n;
  }
  bool failed = false;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      for (int item = pair; item < num_tiles && !failed; item += num_pairs) {
        const WorkItem work = split ? decode_item(g, item, k_blocks) : WorkItem{item, 0, k_blocks, 0, false};
        const HalfBlock hb = half_block<Policy>(p, g, work.tile, half);
        const int mb = hb.mb, nb = hb.nb;
        if (!Policy::before_load(p, g, mb, deadline, abort_flag)) { raise_error(g, kErrPolicyWait, 0); failed = true; break; }
        for (int kb = work.kb_begin; kb < work.kb_end; ++kb) {
          if (!ptx::mbar_wait(&pipe.empty[stage], phase ^ 1u, deadline, abort_flag)) {
            raise_error(g, kErrProducerWait, 0); failed = true; break;
          }
          uint8_t* a_dst = smem + stage * kStageBytes2;
          uint8_t* b_dst = a_dst + kBytesA2;
          ptx2::mbar_expect_tx_leader(&pipe.full[stage], kBytesA2 + static_cast<uint32_t>(g.bn / 2) * kBK * 2);
          ptx2::tma_load_2d_pair(a_dst, &tma_a, &pipe.full[stage], kb * kBK, mb * kBM);
          ptx2::tma_load_2d_pair(b_dst, &tma_b, &pipe.full[stage], kb * kBK,
                                 Policy::b_row(p, g, mb, nb) + half * (g.bn / 2));
          if (++stage == kStages2) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (even CTA only)
    if (lane == 0 && half == 0) {
      const uint32_t idesc = ptx::umma_idesc_f32(2 * kBM, static_cast<uint32_t>(g.bn), true);
      uint32_t stage = 0, phase = 0;
      uint32_t local_tile = 0;
      for (int item = pair; item < num_tiles && !failed; item += num_pairs, ++local_tile) {
        const WorkItem work = split ? decode_item(g, item, k_blocks) : WorkItem{item, 0, k_blocks, 0, false};
        const uint32_t acc = local_tile & 1u, acc_phase = (local_tile >> 1) & 1u;
        if (!ptx::mbar_wait(&pipe.acc_empty[acc], acc_phase ^ 1u, deadline, abort_flag)) {
          raise_error(g, kErrMmaWait, 1); failed = true; break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * kBN;
        for (int kb = work.kb_begin; kb < work.kb_end; ++kb) {
          if (!ptx::mbar_wait(&pipe.full[stage], phase, deadline, abort_flag)) {
            raise_error(g, kErrMmaWait, 1); failed = true; break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t a_addr = ptx::smem_u32(smem + stage * kStageBytes2);
          const uint32_t b_addr = a_addr + kBytesA2;
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            const uint64_t da = ptx::umma_desc_k_sw128(a_addr + k * kUmmaK * 2);
            const uint64_t db = ptx::umma_desc_k_sw128(b_addr + k * kUmmaK * 2);
            ptx2::umma_f16_pair(tmem_d, da, db, idesc, (kb != work.kb_begin || k != 0) ? 1u : 0u);
          }
          ptx2::umma_commit_pair(&pipe.empty[stage]);       // frees the stage in both CTAs
          if (++stage == kStages2) { stage = 0; phase ^= 1u; }
        }
        if (!failed) ptx2::umma_commit_pair(&pipe.acc_full[acc]);   // accumulator halves complete in both CTAs
      }
      trace_stamp(g, 1);
    }
  } else if (warp == 6) {
    // ---------------------------------------------------------------- signal warp
    if (Policy::kSignalsTiles && lane == 0) {
      uint32_t local_tile = 0;
      for (int tile = pair; tile < num_tiles; tile += num_pairs, ++local_tile) {
        const uint32_t want = 4u * (local_tile + 1u);
        const volatile uint32_t* count = &pipe.stored_count;
        uint32_t spins = 0;
        bool ok = true;
        while (static_cast<int32_t>(*count - want) < 0) {
          if ((++spins & 255u) == 0u && (*abort_flag || ptx::globaltimer() > deadline)) { ok = false; break; }
        }
        if (!ok) break;
        __threadfence_block();
        const HalfBlock hb = half_block<Policy>(p, g, tile, half);
        if (hb.present) Policy::tile_done(p, g, hb.mb, hb.nb);
      }
    }
  } else if (warp >= 7) {
    // ---------------------------------------------------------------- reducer warps (policies that have them)
    if constexpr (Policy::kReducerWarps > 0)
      Policy::reducer_main(p, g, static_cast<int>(blockIdx.x) - aux, static_cast<int>(gridDim.x) - aux, warp - 7, lane,
                           deadline, abort_flag);
    if (warp == 7 && lane == 0) trace_stamp(g, 3);
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5, both CTAs)
    const int quarter = warp & 3;
    uint32_t local_tile = 0;
    for (int item = pair; item < num_tiles; item += num_pairs, ++local_tile) {
      const WorkItem work = split ? decode_item(g, item, k_blocks) : WorkItem{item, 0, k_blocks, 0, false};
      const uint32_t acc = local_tile & 1u, acc_phase = (local_tile >> 1) & 1u;
      const HalfBlock hb = half_block<Policy>(p, g, work.tile, half);
      const int mb = hb.mb, nb = hb.nb, mb2 = hb.mb2;
      uint32_t ok = 1;
      if (lane == 0) ok = ptx::mbar_wait(&pipe.acc_full[acc], acc_phase, deadline, abort_flag) ? 1u : 0u;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) { if (lane == 0) raise_error(g, kErrEpilogueWait, 2); break; }
      ptx::tc_fence_after_sync();
      constexpr int kOut = Policy::kOutPer32;
      if constexpr (Policy::kSplitTail) {
        if (work.partial) {
          if (!split_tail_epilogue<Policy>(p, g, work, mb2, nb, half, quarter, lane, tmem_base + acc * kBN,
                                           &pipe.acc_empty[acc],
                                           smem + kStages2 * kStageBytes2 + (warp - 2) * kEpiWarpBytes, deadline,
                                           abort_flag)) {
            if (lane == 0) raise_error(g, kErrEpilogueWait, 9);
            break;
          }
          continue;
        }
      }
      constexpr int kRowBytes = kEpiCols / 32 * kOut * 2;
      constexpr int kChunks = kRowBytes / 16;
      constexpr int kRowsPerSt = 32 / kChunks;
      RowInfo info;
      const bool block_ok = hb.present;                  // an odd number of row blocks leaves the last pair half empty
      if constexpr (Policy::kRowScatter) {
        info = Policy::row_info(p, g, block_ok ? mb : 0, quarter * 32 + lane);
        if (!block_ok) info.valid = 0;
      } else {
        info.dst = Policy::tile_base(p, g, block_ok ? mb : 0) +
                   static_cast<int64_t>(quarter * 32 + lane) * Policy::row_pitch(p, g);
        info.scale = 1.f;
        info.valid = block_ok && mb * kBM + quarter * 32 + lane < g.M ? 1u : 0u;
      }
      const int out_cols = g.N * kOut / 32;
      const uint32_t taddr = tmem_base + acc * kBN + (static_cast<uint32_t>(quarter * 32) << 16);
      uint8_t* stage_buf = smem + kStages2 * kStageBytes2 + (warp - 2) * kEpiWarpBytes;
#pragma unroll 1
      for (int c0 = 0; c0 < g.bn; c0 += kEpiCols) {
#pragma unroll
        for (int q = 0; q < kEpiCols / 32; ++q) {
          if (c0 + q * 32 >= g.bn) break;                  // narrower tiles end inside a pass
          uint32_t v[32];
          ptx::tmem_ld_32x32b_x32(taddr + c0 + q * 32, v);
          ptx::tmem_ld_wait();
          float o[kOut];
          Policy::transform(reinterpret_cast<const float*>(v), info.scale, o);
#pragma unroll
          for (int i = 0; i < kOut / 8; ++i) {
            const int chunk = (q * (kOut / 8) + i) ^ (lane & (kChunks - 1));
            *reinterpret_cast<uint4*>(stage_buf + lane * kRowBytes + chunk * 16) = pack8_bf16(o + 8 * i);
          }
        }
        __syncwarp();
        const int col_first = (nb * g.bn + c0) / 32 * kOut;
        const int pass_cols = min(kEpiCols, g.bn - c0) / 32 * kOut;      // output columns this pass holds
#pragma unroll 4
        for (int it = 0; it < 32 / kRowsPerSt; ++it) {
          const int r = it * kRowsPerSt + lane / kChunks, j = lane % kChunks;
          const uint64_t dst_bits = __shfl_sync(0xffffffffu, reinterpret_cast<uint64_t>(info.dst), r);
          const uint32_t row_ok = __shfl_sync(0xffffffffu, info.valid, r);
          const int col = col_first + j * 8;
          const uint4 val = *reinterpret_cast<const uint4*>(stage_buf + r * kRowBytes + ((j ^ (r & (kChunks - 1))) * 16));
          if (row_ok && j * 8 < pass_cols && col < out_cols)
            ptx::st_v4(reinterpret_cast<uint8_t*>(dst_bits) + static_cast<int64_t>(col) * 2, val);
        }
        __syncwarp();
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        ptx2::mbar_arrive_leader(&pipe.acc_empty[acc]);      // the even CTA's barrier collects both CTAs' warps
        if (Policy::kSignalsTiles) {
          __threadfence_block();
          atomicAdd_block(&pipe.stored_count, 1u);
        }
      }
      if (local_tile == 0 && warp == 2 && lane == 0) trace_stamp(g, 5);
    }
    if (warp == 2 && lane == 0) trace_stamp(g, 2);
  }

  // A role that gave up may have left loads in flight or the partner mid-tile: give outstanding
  // bulk copies time to land (their latency is a few microseconds) before anyone can exit.
  if (*abort_flag) {
    const uint64_t until = ptx::globaltimer() + 200000ull;
    while (ptx::globaltimer() < until) __nanosleep(1000);
  }
  ptx::tc_fence_before_sync();
  ptx2::cluster_sync();                      // the partner no longer reads this CTA's memory or barriers
  if (threadIdx.x == 0) trace_stamp(g, 4);
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx2::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  Policy::finish(p, g, blockIdx.x - aux, gridDim.x - aux, deadline, abort_flag);
}

}  // namespace gemm
}  // namespace pccl
