// Expert-parallel MoE feed-forward as two policies of the GEMM kernels (one SM per tile or SM pairs).
//
// Tokens arrive in "regions" of the receive buffer, one per (local expert, source rank):
// region = local_expert * world + source, `cap` rows each, of which counts[region] are filled
// (the dispatch kernel of the source ranks wrote rows, row metadata and the count, then posted
// a flag).  Both GEMMs walk only the filled 128-row blocks; the tile list is built on the
// device at kernel start, because the counts are only known there.
//
//   MoeUpPolicy     H = silu(X W1^T) * (X W3^T).  W1 and W3 are interleaved in groups of 16 rows
//       ([16 gate rows | 16 up rows] per 32 rows of the stacked weight), so 32 consecutive
//       accumulator columns hold the gate and up values of the same 16 hidden units and the
//       epilogue emits 16 outputs per 32 columns: the 2F-wide intermediate never reaches memory.
//   MoeDownPolicy   Y = H W2^T; the epilogue scales each row by its router gate and stores it
//       straight into the combine buffer of the rank the token came from (NVLink stores,
//       coalesced per row).  After its tiles the kernel tells every rank it is done, waits for
//       all experts, and sums the two expert outputs of each local token.
//
// Tile order: per local expert, n-tile outer, row block inner, so a wave of CTAs shares a few
// weight tiles and the (L2-resident) activations.  All waits are bounded.
// The reference has no MoE operator; its alltoall template is the nearest relative
// (pccl/dsl/algorithms/ring.py, build_alltoall).
#pragma once
#include "tp_policies.cuh"

namespace pccl {
namespace gemm {

constexpr int kMoeMaxRegions = 64;

struct MoeShape {
  const uint32_t* counts;     // local (symmetric heap): filled rows per region
  const uint32_t* ready;      // local (symmetric heap): [world] dispatch flags, one count per call
  int world, local_experts;   // regions = local_experts * world
  int cap_blocks;             // region capacity in 128-row blocks
  int wait_ready;             // wait for the sources' dispatch flags before reading counts
  uint32_t epoch;
};

// Shared-memory tile index: prefix[r] = filled row blocks in regions [0, r).
struct MoeIndex {
  uint16_t prefix[kMoeMaxRegions + 1];
  uint32_t ok;
  uint32_t pairs;             // sum over local experts of ceil(filled blocks / 2): tiles of the paired kernel per n-tile
};
__device__ __forceinline__ MoeIndex& moe_index() {
  __shared__ MoeIndex index;
  return index;
}

__device__ __forceinline__ int moe_prepare(const MoeShape& s, const Problem& g, uint64_t deadline,
                                           const volatile uint32_t* abort_flag) {
  MoeIndex& ix = moe_index();
  if (threadIdx.x == 0) ix.ok = 1;
  __syncthreads();
  if (s.wait_ready && static_cast<int>(threadIdx.x) < s.world) {
    if (!wait_flag_ge(s.ready + threadIdx.x, s.epoch, deadline, abort_flag)) {
      ix.ok = 0;
      raise_error(g, kErrPolicyWait, 6);
    }
  }
  __syncthreads();
  if (!ix.ok) return -1;
  if (threadIdx.x == 0) {
    const int regions = s.local_experts * s.world;
    uint32_t total = 0;
    for (int r = 0; r < regions; ++r) {
      ix.prefix[r] = static_cast<uint16_t>(total);
      uint32_t rows = ptx::ld_acquire_sys(s.counts + r);
      const uint32_t cap_rows = static_cast<uint32_t>(s.cap_blocks) * kBM;
      if (rows > cap_rows) rows = cap_rows;
      total += (rows + kBM - 1) / kBM;
    }
    ix.prefix[regions] = static_cast<uint16_t>(total);
    uint32_t pairs = 0;
    for (int le = 0; le < s.local_experts; ++le)
      pairs += (static_cast<uint32_t>(ix.prefix[(le + 1) * s.world] - ix.prefix[le * s.world]) + 1u) / 2u;
    ix.pairs = pairs;
  }
  __syncthreads();
  // The rows were written by generic-proxy stores (of other GPUs); TMA reads through the async proxy.
  asm volatile("fence.proxy.async.global;" ::: "memory");
  return ix.prefix[s.local_experts * s.world];
}

// tile -> (row block in the receive buffer, n tile).
__device__ __forceinline__ void moe_tile_coords(const MoeShape& s, const Problem& g, int tile, int* mb, int* nb) {
  const MoeIndex& ix = moe_index();
  int le = 0, first = 0, blocks = 0;
  for (; le < s.local_experts; ++le) {
    first = ix.prefix[le * s.world];
    blocks = ix.prefix[(le + 1) * s.world] - first;
    if (tile < blocks * g.tiles_n) break;
    tile -= blocks * g.tiles_n;
  }
  if (le == s.local_experts) { le = s.local_experts - 1; tile = 0; }     // not reached for tile < num_tiles
  *nb = tile / blocks;
  const int b = first + tile % blocks;
  int region = le * s.world;
  while (region + 1 < (le + 1) * s.world && ix.prefix[region + 1] <= b) ++region;
  *mb = region * s.cap_blocks + (b - ix.prefix[region]);
}

// Paired kernel: tile -> the 128-row block of CTA `half`.  A pair takes two consecutive filled blocks
// of one expert (they share the expert's weight tile); an expert with an odd number of filled
// blocks leaves the second half of its last pair absent.
__device__ __forceinline__ void moe_ragged_pair(const MoeShape& s, const Problem& g, int tile, int half, int* mb,
                                                bool* present, int* nb) {
  const MoeIndex& ix = moe_index();
  int le = 0, first = 0, blocks = 0, pairs = 1;
  for (; le < s.local_experts; ++le) {
    first = ix.prefix[le * s.world];
    blocks = ix.prefix[(le + 1) * s.world] - first;
    pairs = (blocks + 1) / 2;
    if (tile < pairs * g.tiles_n) break;
    tile -= pairs * g.tiles_n;
  }
  if (le == s.local_experts) { le = s.local_experts - 1; tile = 0; pairs = pairs > 0 ? pairs : 1; }   // not reached for tile < pair_tiles
  *nb = tile / pairs;
  const int in_expert = 2 * (tile % pairs) + half;
  *present = in_expert < blocks;
  const int b = first + (*present ? in_expert : in_expert - 1);
  int region = le * s.world;
  while (region + 1 < (le + 1) * s.world && ix.prefix[region + 1] <= b) ++region;
  *mb = region * s.cap_blocks + (b - ix.prefix[region]);
}

// ------------------------------------------------------------------------------------------------
struct MoeUpPolicy : PolicyDefaults {
  struct Params {
    MoeShape shape;
    __nv_bfloat16* h;           // local [regions * cap][F]
    int64_t ldh;
  };
  static constexpr int kOutPer32 = 16;
  static constexpr bool kSignalsTiles = false;
  static constexpr bool kRaggedPairs = true;
  __device__ static void ragged_pair(const Params& p, const Problem& g, int tile, int half, int* mb, bool* present,
                                     int* nb) {
    moe_ragged_pair(p.shape, g, tile, half, mb, present, nb);
  }
  __device__ static int pair_tiles(const Params&, const Problem& g) { return static_cast<int>(moe_index().pairs) * g.tiles_n; }
  __device__ static void pair_coords(const Params&, const Problem&, int, int*, int*) {}

  __device__ static int prepare(const Params& p, const Problem& g, uint64_t deadline, const volatile uint32_t* abort_flag) {
    return moe_prepare(p.shape, g, deadline, abort_flag);
  }
  __device__ static void tile_coords(const Params& p, const Problem& g, int tile, int* mb, int* nb) {
    moe_tile_coords(p.shape, g, tile, mb, nb);
  }
  __device__ static bool before_load(const Params&, const Problem&, int, uint64_t, const volatile uint32_t*) {
    return true;
  }
  // Weights of the local experts are stacked: expert le owns rows [le * N, (le + 1) * N).
  __device__ static int b_row(const Params& p, const Problem& g, int mb, int nb) {
    const int le = mb / p.shape.cap_blocks / p.shape.world;
    return le * g.N + nb * g.bn;
  }
  // acc[0..15] = gate pre-activations, acc[16..31] = up projections of the same 16 units.
  __device__ static void transform(const float* acc, float, float* out) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float gate = acc[i];
      out[i] = gate / (1.f + __expf(-gate)) * acc[16 + i];
    }
  }
  __device__ static uint8_t* tile_base(const Params& p, const Problem&, int mb) {
    return reinterpret_cast<uint8_t*>(p.h + static_cast<int64_t>(mb) * kBM * p.ldh);
  }
  __device__ static int64_t row_pitch(const Params& p, const Problem&) { return p.ldh * 2; }
  __device__ static void tile_done(const Params&, const Problem&, int, int) {}
  __device__ static int aux_ctas(const Params&) { return 0; }
  __device__ static void aux_main(const Params&, const Problem&, int, int, uint64_t, const volatile uint32_t*, uint8_t*) {}
  __device__ static void finish(const Params&, const Problem&, int, int, uint64_t, const volatile uint32_t*) {}
};

// ------------------------------------------------------------------------------------------------
struct MoeDownPolicy : PolicyDefaults {
  struct Params {
    MoeShape shape;
    PeerView peers;
    uint64_t meta_off;          // heap offset of meta[regions][cap] {token * 2 + k, gate bits}
    uint64_t comb_off;          // heap offset of comb[tokens][2][H] bf16 (on the tokens' home rank)
    uint64_t done_off;          // heap offset of u32 done[world]: expert rank r finished call n
    uint32_t* cta_counter;      // local, monotonic
    __nv_bfloat16* out;         // local [tokens][H]
    int tokens;
  };
  static constexpr bool kRowScatter = true;
  static constexpr bool kSignalsTiles = false;
  static constexpr bool kRaggedPairs = true;
  __device__ static void ragged_pair(const Params& p, const Problem& g, int tile, int half, int* mb, bool* present,
                                     int* nb) {
    moe_ragged_pair(p.shape, g, tile, half, mb, present, nb);
  }
  __device__ static int pair_tiles(const Params&, const Problem& g) { return static_cast<int>(moe_index().pairs) * g.tiles_n; }
  __device__ static void pair_coords(const Params&, const Problem&, int, int*, int*) {}

  __device__ static int prepare(const Params& p, const Problem& g, uint64_t deadline, const volatile uint32_t* abort_flag) {
    return moe_prepare(p.shape, g, deadline, abort_flag);
  }
  __device__ static void tile_coords(const Params& p, const Problem& g, int tile, int* mb, int* nb) {
    moe_tile_coords(p.shape, g, tile, mb, nb);
  }
  __device__ static bool before_load(const Params&, const Problem&, int, uint64_t, const volatile uint32_t*) {
    return true;
  }
  __device__ static int b_row(const Params& p, const Problem& g, int mb, int nb) {
    const int le = mb / p.shape.cap_blocks / p.shape.world;
    return le * g.N + nb * g.bn;
  }
  __device__ static RowInfo row_info(const Params& p, const Problem& g, int mb, int row_in_tile) {
    const int region = mb / p.shape.cap_blocks;
    const uint32_t slot = static_cast<uint32_t>(mb % p.shape.cap_blocks) * kBM + row_in_tile;
    RowInfo info{nullptr, 0.f, 0u};
    if (slot < p.shape.counts[region]) {
      const uint2 m = *reinterpret_cast<const uint2*>(
          p.peers.base[p.peers.rank] + p.meta_off +
          (static_cast<uint64_t>(region) * p.shape.cap_blocks * kBM + slot) * sizeof(uint2));
      const int home = region % p.shape.world;
      info.dst = p.peers.base[home] + p.comb_off + static_cast<uint64_t>(m.x) * g.N * 2;
      info.scale = __uint_as_float(m.y);
      info.valid = m.x < static_cast<uint32_t>(2 * p.tokens) ? 1u : 0u;     // never store through a corrupt index
    }
    return info;
  }
  __device__ static uint8_t* tile_base(const Params&, const Problem&, int) { return nullptr; }
  __device__ static int64_t row_pitch(const Params&, const Problem&) { return 0; }
  __device__ static void tile_done(const Params&, const Problem&, int, int) {}
  __device__ static int aux_ctas(const Params&) { return 0; }
  __device__ static void aux_main(const Params&, const Problem&, int, int, uint64_t, const volatile uint32_t*, uint8_t*) {}

  // "All my expert outputs are delivered" -> every rank (posted by the last CTA to get here);
  // then wait for every expert rank and add the two expert rows of each local token.
  __device__ static void finish(const Params& p, const Problem& g, int cta, int num_ctas, uint64_t deadline,
                                const volatile uint32_t* abort_flag) {
    __shared__ uint32_t ok_flag;
    const int me = p.peers.rank, world = p.peers.world;
    if (threadIdx.x == 0) {
      ok_flag = 1;
      // GPU scope suffices here: the CTA that completes the count fences at system scope before it posts,
      // and that fence is cumulative over every arrival it counted (a system fence per CTA is slow while
      // other SMs stream stores over NVLink).
      ptx::fence_gpu();
      const uint32_t arrived = atomicAdd(p.cta_counter, 1u) + 1u;
      if (arrived == p.shape.epoch * static_cast<uint32_t>(num_ctas)) {
        ptx::fence_sys();
        for (int r = 0; r < world; ++r)
          ptx::red_release_sys_add(reinterpret_cast<uint32_t*>(p.peers.base[r] + p.done_off) + me, 1u);
      }
    }
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < world) {
      const uint32_t* done = reinterpret_cast<const uint32_t*>(p.peers.base[me] + p.done_off);
      if (!wait_flag_ge(done + threadIdx.x, p.shape.epoch, deadline, abort_flag)) {
        ok_flag = 0;
        raise_error(g, kErrPolicyWait, 7);
      }
    }
    __syncthreads();
    if (!ok_flag) return;
    const int vecs = g.N / 8;
    const uint8_t* comb = p.peers.base[me] + p.comb_off;
    for (int t = cta; t < p.tokens; t += num_ctas) {
      const uint8_t* row = comb + static_cast<uint64_t>(t) * 2 * g.N * 2;
      for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
        const uint4 a = ptx::ld_local_v4(row + v * 16);
        const uint4 b = ptx::ld_local_v4(row + static_cast<uint64_t>(g.N) * 2 + v * 16);
        const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w};
        float f[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          f[2 * j] = __uint_as_float(wa[j] << 16) + __uint_as_float(wb[j] << 16);
          f[2 * j + 1] = __uint_as_float(wa[j] & 0xffff0000u) + __uint_as_float(wb[j] & 0xffff0000u);
        }
        *reinterpret_cast<uint4*>(p.out + static_cast<int64_t>(t) * g.N + v * 8) = pack8_bf16(f);
      }
    }
  }
};

}  // namespace gemm
}  // namespace pccl
