// Persistent, warp-specialised bf16 GEMM on the 5th-generation tensor cores:
//     C[M,N] = A[M,K] * B[N,K]^T      (A and B row-major, i.e. both K-major; fp32 accumulate)
//
//   warp 0      TMA producer: streams 128x64 A tiles and 256x64 B tiles (128-byte swizzle)
//               from this GPU's HBM into a 4-stage shared-memory ring (plain, non-multicast
//               cp.async.bulk.tensor loads completing on mbarriers);
//   warp 1      MMA issuer: one elected lane issues tcgen05.mma (M128 x N256 x K16) with the
//               accumulator in tensor memory; two 256-column accumulators alternate so the
//               epilogue of tile i overlaps the main loop of tile i+1;
//   warp 6      signal warp (policies that publish per-tile completion): waits until the four
//               epilogue warps have stored a tile, then fences and posts, off their critical path;
//   warps 2-5   epilogue: tcgen05.ld the accumulator (each warp owns 32 TMEM lanes = 32 rows),
//               then hand 32-column row segments to the Policy, which converts and stores
//               them — to local memory, or straight into a peer GPU's memory for the fused
//               GEMM -> reduce-scatter.
//
// A Policy supplies the tile list (optionally sized on the device: ragged expert batches), the
// tile order, an optional "rows ready" wait before a tile's A rows are loaded (all-gather ->
// GEMM), the row of the stacked weight an n-tile starts at (grouped GEMM), the destination /
// scale / validity of each output row, an element-wise transform of the accumulator (SwiGLU),
// and a per-tile completion hook.
// Every wait is bounded; on a timeout the error word is set, all roles leave their loops,
// the CTA waits for its outstanding TMA transactions, frees its TMEM and returns.
// The reference contains no GEMM or tensor-core code; this kernel has no counterpart there.
#pragma once
#include <cuda_bf16.h>

#include "../ptx/tcgen05.cuh"

namespace pccl {
namespace gemm {

constexpr int kBM = 128, kBN = 256, kBK = 64, kStages = 4;
constexpr int kUmmaK = 16;
constexpr int kThreads = 224;                                  // 7 warps: TMA, MMA, 4 epilogue, signal
constexpr int kReducerThreads = 128;                           // + 4 reducer warps for policies that ask for them
constexpr int kMaxThreads = kThreads + kReducerThreads;
constexpr uint32_t kBytesA = kBM * kBK * 2, kBytesB = kBN * kBK * 2;
constexpr uint32_t kStageBytes = kBytesA + kBytesB;
constexpr int kEpiCols = 128;                                   // columns staged per epilogue pass
constexpr uint32_t kEpiWarpBytes = 32 * kEpiCols * 2;           // 32 rows x 256 B per epilogue warp
constexpr uint32_t kSmemBytes = kStages * kStageBytes + 4 * kEpiWarpBytes + 1024;   // + alignment slack
constexpr uint32_t kTmemCols = 512;                             // 2 accumulators x 256 columns

struct Problem {
  int M, N, K;
  int tiles_m, tiles_n;
  int bn;                     // columns per tile: kBN, or what the paired kernel's launcher chose (a multiple of 32)
  uint32_t* error;            // device word: 0 ok, else (code << 8 | role)
  uint64_t timeout_ns;
  // Optional timeline (null = off): kGemmTraceStamps %globaltimer values per CTA:
  // [0] kernel entered, [1] MMA issuer done with its last tile, [2] epilogue warps done,
  // [3] reducer warps done, [4] CTA leaves, [5] first accumulator complete.
  uint64_t* trace;
  // Split tail of the paired kernel (tail_first >= the tile count: off).  Work items [0, tail_first)
  // are whole tiles; each later tile is cut along K into tail_slices items of tail_kb k-blocks whose
  // fp32 partial accumulators meet in tail_ws ([tile][slice][half][128][256] floats) and are summed
  // by the warps that produced them (tail_counters: [0, 64) arrivals, [64, 128) finished, per tile).
  int tail_first, tail_slices, tail_kb, num_items;
  float* tail_ws;
  uint32_t* tail_counters;
};
constexpr int kGemmTraceStamps = 8;
constexpr int kTailMaxTiles = 64;
__device__ __forceinline__ void trace_stamp(const Problem& g, int slot) {
  if (g.trace) g.trace[static_cast<uint64_t>(blockIdx.x) * kGemmTraceStamps + slot] = ptx::globaltimer();
}

enum ErrorCode : uint32_t { kErrProducerWait = 1, kErrMmaWait = 2, kErrEpilogueWait = 3, kErrPolicyWait = 4 };

struct Pipe {
  uint64_t full[kStages], empty[kStages];
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  uint32_t stored_count;       // epilogue-warp completions (4 per tile), monotonic: no phase to alias
};

__device__ __forceinline__ void raise_error(const Problem& g, uint32_t code, uint32_t role) {
  atomicCAS(g.error, 0u, code << 8 | role);
}

__device__ __forceinline__ uint4 pack8_bf16(const float* f);

// What a policy may leave at its default by deriving from this struct.
struct PolicyDefaults {
  // Outputs per 32 accumulator columns: 32 (plain) or 16 (pairwise-combining epilogue, SwiGLU).
  static constexpr int kOutPer32 = 32;
  // true: the destination, validity and scale of a row come from Policy::row_info (rows of one
  // tile may go to unrelated addresses); false: tile_base + row * row_pitch.
  static constexpr bool kRowScatter = false;
  // 4: the CTA carries four more warps that run Policy::reducer_main next to the GEMM roles (work
  // that consumes what peers' epilogues deliver, overlapped with this CTA's own tiles); 0: none.
  static constexpr int kReducerWarps = 0;
  // true: the paired kernel may cut the tiles of its last, partly filled round along K (needs a
  // static tile list, plain row addressing through tile_base / row_pitch and no per-tile signal).
  static constexpr bool kSplitTail = false;
  // true: the paired kernel asks Policy::ragged_pair for the two 128-row blocks of a tile (they need
  // not be neighbours and the second may be absent) and Policy::pair_tiles for the tile count;
  // false: block pair i = blocks 2i, 2i + 1 through Policy::pair_coords.
  static constexpr bool kRaggedPairs = false;
  template <class P>
  __device__ static void reducer_main(const P&, const Problem&, int, int, int, int, uint64_t,
                                      const volatile uint32_t*) {}
  // Row of B (and column of the accumulator grid) where n-tile nb starts.
  template <class P>
  __device__ static int b_row(const P&, const Problem&, int, int nb);
  // 32 accumulator columns -> kOutPer32 values, scaled by the row's factor.
  __device__ static void transform(const float* acc, float scale, float* out) {
#pragma unroll
    for (int i = 0; i < 32; ++i) out[i] = acc[i] * scale;
  }
};

template <class P>
__device__ int PolicyDefaults::b_row(const P&, const Problem& g, int, int nb) { return nb * g.bn; }

struct RowInfo {
  uint8_t* dst;      // address of output column 0 of this row
  float scale;
  uint32_t valid;
};

template <class Policy>
__global__ void __launch_bounds__(kMaxThreads, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const Problem g, const typename Policy::Params p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ Pipe pipe;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const volatile uint32_t* abort_flag = g.error;
  const uint64_t deadline = ptx::globaltimer() + g.timeout_ns;

  // Auxiliary CTAs (e.g. the copiers of all-gather -> GEMM) take no part in the GEMM pipeline.
  const int aux = Policy::aux_ctas(p);
  if (static_cast<int>(blockIdx.x) < aux) {
    Policy::aux_main(p, g, blockIdx.x, aux, deadline, abort_flag, smem);
    return;
  }
  const int cta = blockIdx.x - aux, num_ctas = gridDim.x - aux;
  if (threadIdx.x == 0) trace_stamp(g, 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { ptx::mbar_init(&pipe.full[s], 1); ptx::mbar_init(&pipe.empty[s], 1); }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&pipe.acc_full[a], 1);
      ptx::mbar_init(&pipe.acc_empty[a], 4);
    }
    pipe.stored_count = 0;
    ptx::mbar_init_fence();
    ptx::tma_prefetch_desc(&tma_a);
    ptx::tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&pipe.tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = pipe.tmem_base;

  // Policies with a data-dependent row count (ragged expert batches) size their tile list here;
  // a negative answer (a wait ran out) leaves no tiles and falls through to the TMEM release.
  const int tiles_m = Policy::prepare(p, g, deadline, abort_flag);
  const int num_tiles = tiles_m < 0 ? 0 : tiles_m * g.tiles_n;
  const int k_blocks = (g.K + kBK - 1) / kBK;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      int issued = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += num_ctas) {
        int mb, nb;
        Policy::tile_coords(p, g, tile, &mb, &nb);
        if (!Policy::before_load(p, g, mb, deadline, abort_flag)) { raise_error(g, kErrPolicyWait, 0); break; }
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!ptx::mbar_wait(&pipe.empty[stage], phase ^ 1u, deadline, abort_flag)) {
            raise_error(g, kErrProducerWait, 0); ok = false; break;
          }
          uint8_t* a_dst = smem + stage * kStageBytes;
          uint8_t* b_dst = a_dst + kBytesA;
          ptx::mbar_expect_tx(&pipe.full[stage], kStageBytes);
          ptx::tma_load_2d(a_dst, &tma_a, &pipe.full[stage], kb * kBK, mb * kBM);
          ptx::tma_load_2d(b_dst, &tma_b, &pipe.full[stage], kb * kBK, Policy::b_row(p, g, mb, nb));
          ++issued;
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      // Leaving early: wait (bounded) until the loads already issued have landed, so no
      // bulk copy is still writing this CTA's shared memory when it exits.
      if (!ok || *abort_flag) {
        const uint64_t drain_deadline = ptx::globaltimer() + 50000000ull;
        uint32_t s = stage, ph = phase;
        for (int back = 0; back < kStages && back < issued; ++back) {
          if (s == 0) { s = kStages; ph ^= 1u; }
          --s;
          uint32_t no_abort = 0;
          ptx::mbar_wait(&pipe.full[s], ph, drain_deadline, &no_abort);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = ptx::umma_idesc_f32(kBM, kBN, true);
      uint32_t stage = 0, phase = 0;
      uint32_t local_tile = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += num_ctas, ++local_tile) {
        const uint32_t acc = local_tile & 1u, acc_phase = (local_tile >> 1) & 1u;
        if (!ptx::mbar_wait(&pipe.acc_empty[acc], acc_phase ^ 1u, deadline, abort_flag)) {
          raise_error(g, kErrMmaWait, 1); break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * kBN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!ptx::mbar_wait(&pipe.full[stage], phase, deadline, abort_flag)) {
            raise_error(g, kErrMmaWait, 1); ok = false; break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t a_addr = ptx::smem_u32(smem + stage * kStageBytes);
          const uint32_t b_addr = a_addr + kBytesA;
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            // Advancing K by 16 bf16 = 32 bytes inside the 128-byte swizzled row.
            const uint64_t da = ptx::umma_desc_k_sw128(a_addr + k * kUmmaK * 2);
            const uint64_t db = ptx::umma_desc_k_sw128(b_addr + k * kUmmaK * 2);
            ptx::umma_f16(tmem_d, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          ptx::umma_commit(&pipe.empty[stage]);       // frees the stage when these MMAs retire
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) ptx::umma_commit(&pipe.acc_full[acc]);  // accumulator complete
      }
      trace_stamp(g, 1);
    }
  } else if (warp == 6) {
    // ---------------------------------------------------------------- signal warp
    if (Policy::kSignalsTiles && lane == 0) {
      uint32_t local_tile = 0;
      for (int tile = cta; tile < num_tiles; tile += num_ctas, ++local_tile) {
        // Tile `local_tile` is out when 4 * (local_tile + 1) epilogue warps have reported.
        const uint32_t want = 4u * (local_tile + 1u);
        const volatile uint32_t* count = &pipe.stored_count;
        uint32_t spins = 0;
        bool ok = true;
        while (static_cast<int32_t>(*count - want) < 0) {
          if ((++spins & 255u) == 0u && (*abort_flag || ptx::globaltimer() > deadline)) { ok = false; break; }
        }
        if (!ok) break;
        __threadfence_block();                       // acquire the epilogue warps' stores
        int mb, nb;
        Policy::tile_coords(p, g, tile, &mb, &nb);
        Policy::tile_done(p, g, mb, nb);
      }
    }
  } else if (warp >= 7) {
    // ---------------------------------------------------------------- reducer warps (policies that have them)
    if constexpr (Policy::kReducerWarps > 0)
      Policy::reducer_main(p, g, cta, num_ctas, warp - 7, lane, deadline, abort_flag);
    if (warp == 7 && lane == 0) trace_stamp(g, 3);
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int quarter = warp & 3;                      // TMEM lanes [32*quarter, +32)
    uint32_t local_tile = 0;
    for (int tile = cta; tile < num_tiles; tile += num_ctas, ++local_tile) {
      const uint32_t acc = local_tile & 1u, acc_phase = (local_tile >> 1) & 1u;
      int mb, nb;
      Policy::tile_coords(p, g, tile, &mb, &nb);
      uint32_t ok = 1;
      if (lane == 0) ok = ptx::mbar_wait(&pipe.acc_full[acc], acc_phase, deadline, abort_flag) ? 1u : 0u;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) { if (lane == 0) raise_error(g, kErrEpilogueWait, 2); break; }
      ptx::tc_fence_after_sync();
      constexpr int kOut = Policy::kOutPer32;                  // outputs per 32 accumulator columns
      constexpr int kRowBytes = kEpiCols / 32 * kOut * 2;       // staged bytes per row and pass
      constexpr int kChunks = kRowBytes / 16;                   // 16-byte chunks per staged row
      constexpr int kRowsPerSt = 32 / kChunks;                  // rows written per store instruction
      // The lane that owns TMEM lane (= tile row) quarter*32 + lane looks up that row's destination.
      RowInfo info;
      if constexpr (Policy::kRowScatter) {
        info = Policy::row_info(p, g, mb, quarter * 32 + lane);
      } else {
        info.dst = Policy::tile_base(p, g, mb) + static_cast<int64_t>(quarter * 32 + lane) * Policy::row_pitch(p, g);
        info.scale = 1.f;
        info.valid = mb * kBM + quarter * 32 + lane < g.M ? 1u : 0u;
      }
      const int out_cols = g.N * kOut / 32;
      const uint32_t taddr = tmem_base + acc * kBN + (static_cast<uint32_t>(quarter * 32) << 16);
      // Staging buffer of this warp: 32 rows of kChunks 16-byte chunks, chunk index XOR-swizzled
      // by the row so that both the row-wise writes and the chunk-wise reads spread over banks.
      uint8_t* stage_buf = smem + kStages * kStageBytes + (warp - 2) * kEpiWarpBytes;
#pragma unroll 1
      for (int c0 = 0; c0 < kBN; c0 += kEpiCols) {
#pragma unroll
        for (int q = 0; q < kEpiCols / 32; ++q) {
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
        // kChunks lanes write one row's contiguous bytes; kRowsPerSt rows per instruction.
        const int col_first = (nb * kBN + c0) / 32 * kOut;
#pragma unroll 4
        for (int it = 0; it < 32 / kRowsPerSt; ++it) {
          const int r = it * kRowsPerSt + lane / kChunks, j = lane % kChunks;
          const uint64_t dst_bits = __shfl_sync(0xffffffffu, reinterpret_cast<uint64_t>(info.dst), r);
          const uint32_t row_ok = __shfl_sync(0xffffffffu, info.valid, r);
          const int col = col_first + j * 8;
          const uint4 val = *reinterpret_cast<const uint4*>(stage_buf + r * kRowBytes + ((j ^ (r & (kChunks - 1))) * 16));
          if (row_ok && col < out_cols)
            ptx::st_v4(reinterpret_cast<uint8_t*>(dst_bits) + static_cast<int64_t>(col) * 2, val);
        }
        __syncwarp();
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        ptx::mbar_arrive(&pipe.acc_empty[acc]);
        if (Policy::kSignalsTiles) {                 // release the stores above to the signal warp
          __threadfence_block();
          atomicAdd_block(&pipe.stored_count, 1u);
        }
      }
    }
    if (warp == 2 && lane == 0) trace_stamp(g, 2);
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) trace_stamp(g, 4);
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
  // Work that follows the GEMM on the same CTAs (e.g. the reduction of received partials).
  Policy::finish(p, g, cta, num_ctas, deadline, abort_flag);
}

// ---- the plain policy: C is a row-major bf16 matrix in local memory -------------------------------

__device__ __forceinline__ uint4 pack8_bf16(const float* f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

struct StorePolicy : PolicyDefaults {
  static constexpr bool kSplitTail = true;
  struct Params {
    __nv_bfloat16* c;
    int64_t ldc;
  };
  __device__ static int prepare(const Params&, const Problem& g, uint64_t, const volatile uint32_t*) {
    return g.tiles_m;
  }
  // M-fastest order: consecutive CTAs share the B tile (weights) through L2.
  __device__ static void tile_coords(const Params&, const Problem& g, int tile, int* mb, int* nb) {
    *mb = tile % g.tiles_m;
    *nb = tile / g.tiles_m;
  }
  // The paired kernel's order: pairs of row blocks, M-fastest.
  __device__ static void pair_coords(const Params&, const Problem& g, int tile, int* mb2, int* nb) {
    const int pairs_m = (g.tiles_m + 1) / 2;
    *mb2 = tile % pairs_m;
    *nb = tile / pairs_m;
  }
  __device__ static bool before_load(const Params&, const Problem&, int, uint64_t, const volatile uint32_t*) {
    return true;
  }
  static constexpr bool kSignalsTiles = false;
  // Destination of row mb*128, column 0, and the byte pitch between rows (N % 8 == 0).
  __device__ static uint8_t* tile_base(const Params& p, const Problem&, int mb) {
    return reinterpret_cast<uint8_t*>(p.c + static_cast<int64_t>(mb) * kBM * p.ldc);
  }
  __device__ static int64_t row_pitch(const Params& p, const Problem&) { return p.ldc * 2; }
  __device__ static void tile_done(const Params&, const Problem&, int, int) {}
  __device__ static int aux_ctas(const Params&) { return 0; }
  __device__ static void aux_main(const Params&, const Problem&, int, int, uint64_t, const volatile uint32_t*, uint8_t*) {}
  __device__ static void finish(const Params&, const Problem&, int, int, uint64_t, const volatile uint32_t*) {}
};

}  // namespace gemm
}  // namespace pccl
