// Tensor-parallel GEMMs fused with their collective, as policies of umma_gemm_kernel.
//
//   ReduceScatterPolicy   Y = sum_r X_r W_r^T, scattered over rows (tokens).  Every rank computes
//       its full partial product; the epilogue stores each bf16 row segment straight into the
//       *owning* rank's receive slot for this source over NVLink (tiles ordered so the most
//       remote owner comes first and the own rows last), and posts one flag per finished
//       128-row block.  Four extra warps per CTA are reducers from the start: each takes 32-row
//       strips of this rank's own row blocks in the order their partials arrive, waits for the
//       flags of all sources of the block and sums the W slots in rank order (fp32,
//       deterministic), so the reduction runs under the GEMM instead of after it.
//   AllGatherPolicy       Y_r = gather(X) W_r^T.  A few auxiliary CTAs pull the peers' row shards
//       into the *local* gathered matrix with SM loads and publish a ready flag per 128-row
//       block; the GEMM CTAs start with the local shard and wait for a block's flag before
//       its TMA loads (which therefore only ever read this GPU's memory).
//
// Flags count calls (the host passes the call number `epoch`), so nothing is reset between
// calls; receive slots are double-buffered by epoch parity.  All waits are bounded.
// The unfused baseline is cuBLAS + NCCL; the reference has neither operator.
#pragma once
#include <cuda_bf16.h>

#include "../executors/sm100/program.h"
#include "umma_gemm.cuh"

namespace pccl {
namespace gemm {

struct PeerView {
  uint8_t* base[kMaxRanks];     // every rank's symmetric heap as mapped here
  int rank, world;
};

__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t want, uint64_t deadline,
                                             const volatile uint32_t* abort_flag) {
  uint32_t spins = 0;
  while (static_cast<int32_t>(ptx::ld_acquire_sys(flag) - want) < 0) {
    if ((++spins & 63u) == 0u) {
      if (*abort_flag || ptx::globaltimer() > deadline) return false;
      __nanosleep(64);
    }
  }
  return true;
}

// ------------------------------------------------------------------------------------------------
struct ReduceScatterPolicy : PolicyDefaults {
  struct Params {
    PeerView peers;
    uint64_t recv_off;          // heap offset of recv[2][world][rows_per_rank][N] bf16
    uint64_t flags_off;         // heap offset of flags[world][blocks_per_rank] u32
    uint32_t* block_counter;    // local, [tiles_m]: epilogue warps finished per 128-row block (monotonic)
    __nv_bfloat16* out;         // local result [rows_per_rank][N]
    int64_t ldo;
    int rows_per_rank, blocks_per_rank;
    uint32_t epoch;             // 1, 2, 3, ... per call
  };

  __device__ static int prepare(const Params&, const Problem& g, uint64_t, const volatile uint32_t*) {
    return g.tiles_m;
  }
  // Row blocks are visited round-robin over the owners (rank+1, rank+2, ..., rank), so NVLink
  // traffic is spread over the whole GEMM and every owner receives its blocks in order; the
  // n-tiles of one row block are consecutive so that the block's flag is posted early.
  __device__ static void tile_coords(const Params& p, const Problem& g, int tile, int* mb, int* nb) {
    const int block_seq = tile / g.tiles_n;
    const int owner = (p.peers.rank + 1 + block_seq % p.peers.world) % p.peers.world;
    *mb = owner * p.blocks_per_rank + block_seq / p.peers.world;
    *nb = tile % g.tiles_n;
  }
  // The same order for the paired kernel, in units of two row blocks (rows per rank are then a
  // multiple of 256, so a pair never straddles two owners).
  __device__ static void pair_coords(const Params& p, const Problem& g, int tile, int* mb2, int* nb) {
    const int pairs_per_rank = p.blocks_per_rank / 2;
    const int block_seq = tile / g.tiles_n;
    const int owner = (p.peers.rank + 1 + block_seq % p.peers.world) % p.peers.world;
    *mb2 = owner * pairs_per_rank + block_seq / p.peers.world;
    *nb = tile % g.tiles_n;
  }
  __device__ static bool before_load(const Params&, const Problem&, int, uint64_t, const volatile uint32_t*) {
    return true;
  }
  __device__ static uint8_t* slot(const Params& p, const Problem& g, int owner, int src, int local_row) {
    const uint64_t slot_bytes = static_cast<uint64_t>(p.rows_per_rank) * g.N * 2;
    const uint64_t parity = p.epoch & 1u;
    return p.peers.base[owner] + p.recv_off + (parity * p.peers.world + src) * slot_bytes +
           static_cast<uint64_t>(local_row) * g.N * 2;
  }
  static constexpr bool kSignalsTiles = true;
  // A 128-row block never straddles two owners, so its rows are contiguous in one slot.
  __device__ static uint8_t* tile_base(const Params& p, const Problem& g, int mb) {
    return slot(p, g, mb / p.blocks_per_rank, p.peers.rank, (mb % p.blocks_per_rank) * kBM);
  }
  __device__ static int64_t row_pitch(const Params&, const Problem& g) { return static_cast<int64_t>(g.N) * 2; }
  // Called by the signal warp's lane 0 once all four epilogue warps have stored tile (mb, nb)
  // (it acquired their mbarrier arrivals, so the fence below covers their stores).  The call
  // that completes the row block posts the flag at the owner.
  //
  // Fences: a tile's stores only have to be ordered before the block counter at GPU scope; the one
  // CTA that completes the block then fences at system scope before the flag, which by cumulativity
  // covers every tile it counted.  (A system-scope fence per tile measured tens of microseconds
  // each while the other SMs keep streaming stores over NVLink: the flags of the first blocks
  // reached the owner 25-40 us after their data.)
  __device__ static void tile_done(const Params& p, const Problem& g, int mb, int) {
    ptx::fence_gpu();
    const uint32_t target = p.epoch * static_cast<uint32_t>(g.tiles_n);
    const uint32_t seen = atomicAdd(p.block_counter + mb, 1u) + 1u;
    if (seen == target) {
      ptx::fence_sys();
      const int owner = mb / p.blocks_per_rank, local_block = mb % p.blocks_per_rank;
      uint32_t* flag = reinterpret_cast<uint32_t*>(p.peers.base[owner] + p.flags_off) +
                       p.peers.rank * p.blocks_per_rank + local_block;
      ptx::red_release_sys_add(flag, 1u);
    }
  }
  __device__ static int aux_ctas(const Params&) { return 0; }
  __device__ static void aux_main(const Params&, const Problem&, int, int, uint64_t, const volatile uint32_t*, uint8_t*) {}

  // out = sum over the sources' slots, rank order, fp32, for `total` 16-byte vectors of rows
  // [row0, ...) x columns [col0, ...), done by `nthreads` threads of which this is number `tid`.
  // kRV vectors per thread and iteration and kW slots each are loaded before the first add.  Every
  // load is unconditional (lanes past the end re-read the last vector, slots past the world re-read
  // the own one): a conditionally assigned register makes the compiler wait for each load before
  // it issues the next.
  template <int kW>
  __device__ static void sum_slots(const Params& p, const Problem& g, int me, int world, int row0, int col0,
                                   int vec_per_row, int total, int tid, int nthreads) {
    constexpr int kRV = 16 / kW;                  // sixteen 16-byte loads in flight per thread whatever the world size
    for (int i = tid; i < total; i += nthreads * kRV) {
      uint4 raw[kRV][kW];
      int r[kRV], c[kRV];
#pragma unroll
      for (int u = 0; u < kRV; ++u) {
        const int idx = min(i + u * nthreads, total - 1);
        r[u] = row0 + idx / vec_per_row;
        c[u] = col0 + (idx % vec_per_row) * 8;
#pragma unroll
        for (int s = 0; s < kW; ++s)
          raw[u][s] = ptx::ld_local_v4(slot(p, g, me, s < world ? s : me, r[u]) + static_cast<uint64_t>(c[u]) * 2);
      }
#pragma unroll
      for (int u = 0; u < kRV; ++u) {
        if (i + u * nthreads >= total) continue;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int s = 0; s < kW; ++s) {
          if (s >= world) break;
          const uint32_t w[4] = {raw[u][s].x, raw[u][s].y, raw[u][s].z, raw[u][s].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[2 * j] += __uint_as_float(w[j] << 16);
            acc[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
          }
        }
        *reinterpret_cast<uint4*>(p.out + static_cast<int64_t>(r[u]) * p.ldo + c[u]) = pack8_bf16(acc);
      }
    }
  }

  // Reducer warps: item = (local row block, n tile, strip of a few rows), one warp per item, items in
  // the order the blocks complete (every source delivers this rank's blocks in ascending order).
  // A strip is what a warp sums in ONE round of loads (32 lanes x 16 loads in flight): the blocks
  // that complete last are then spread over every reducer warp of the grid and cost one memory
  // round trip.  With 32-row strips 64 warps were left with eight dependent rounds each, 14 us
  // after the last block had arrived (per-CTA timeline, 4 GPUs).
  static constexpr int kReducerWarps = 4;
  __device__ static void reducer_main(const Params& p, const Problem& g, int cta, int num_ctas, int rwarp, int lane,
                                      uint64_t deadline, const volatile uint32_t* abort_flag) {
    const int me = p.peers.rank, world = p.peers.world;
    const uint32_t* flags = reinterpret_cast<const uint32_t*>(p.peers.base[me] + p.flags_off);
    const int loads_per_lane = world <= 2 ? 8 : world <= 4 ? 4 : 2;         // sum_slots' kRV for this world
    int strip_rows = 32 * loads_per_lane * 8 / g.bn;                         // rows of a tile-wide strip in one round
    strip_rows = strip_rows < 1 ? 1 : strip_rows > 32 ? 32 : strip_rows;
    const int strips = (kBM + strip_rows - 1) / strip_rows;
    const int items = p.blocks_per_rank * g.tiles_n * strips;
    int ready_block = -1;
    for (int item = cta * kReducerWarps + rwarp; item < items; item += num_ctas * kReducerWarps) {
      const int block = item / (g.tiles_n * strips), rest = item % (g.tiles_n * strips);
      const int nb = rest / strips, strip = rest % strips;
      if (block != ready_block) {                 // a block this warp has seen complete stays complete
        bool ok = true;
        if (lane < world) ok = wait_flag_ge(flags + lane * p.blocks_per_rank + block, p.epoch, deadline, abort_flag);
        if (!__all_sync(0xffffffffu, ok)) {
          if (lane == 0) raise_error(g, kErrPolicyWait, 3);
          return;
        }
        ready_block = block;
      }
      if (rwarp == 0 && lane == 0) {              // timeline: first and latest item whose partials were all in
        if (item < num_ctas * kReducerWarps) trace_stamp(g, 6);
        trace_stamp(g, 7);
      }
      const int row0 = block * kBM + strip * strip_rows, col0 = nb * g.bn;
      const int rows = min(min(strip_rows, kBM - strip * strip_rows), p.rows_per_rank - row0), cols = min(g.bn, g.N - col0);
      if (rows <= 0 || cols <= 0) continue;
      const int vec_per_row = cols / 8;                    // 8 bf16 per 16 bytes (N % 8 == 0)
      const int total = rows * vec_per_row;
      if (world <= 2) sum_slots<2>(p, g, me, world, row0, col0, vec_per_row, total, lane, 32);
      else if (world <= 4) sum_slots<4>(p, g, me, world, row0, col0, vec_per_row, total, lane, 32);
      else sum_slots<8>(p, g, me, world, row0, col0, vec_per_row, total, lane, 32);
    }
  }
  __device__ static void finish(const Params&, const Problem&, int, int, uint64_t, const volatile uint32_t*) {}
};

// ------------------------------------------------------------------------------------------------
struct AllGatherPolicy : PolicyDefaults {
  static constexpr bool kSplitTail = true;
  struct Params {
    PeerView peers;
    uint64_t gathered_off;      // heap offset of the gathered A [world * rows_per_rank][K] bf16 (per rank)
    uint64_t flags_off;         // heap offset of u32 flags: [0, world) "shard of rank s is in place" (posted
                                // by s at every peer), [world, 2*world) "rank s finished reading my shard"
    uint32_t* ready;            // local, [tiles_m]: gathered row block is complete (epoch counting)
    __nv_bfloat16* c;           // local result [M][N]
    int64_t ldc;
    int rows_per_rank, blocks_per_rank, copy_ctas;
    int copy_parts;             // copier CTAs that share one 128-row block (keeps all copiers busy for small M)
    uint32_t epoch;
  };

  __device__ static int prepare(const Params&, const Problem& g, uint64_t, const volatile uint32_t*) {
    return g.tiles_m;
  }
  // Shards in the order own, rank+1, rank+2, ...  Inside the own shard M-fastest (consecutive CTAs
  // share a weight tile); inside a remote shard N-fastest, rows in the order the copiers deliver
  // them, so that a tile only waits for its own rows (consecutive CTAs then share the A rows).
  __device__ static void tile_coords(const Params& p, const Problem& g, int tile, int* mb, int* nb) {
    const int per_shard = p.blocks_per_rank * g.tiles_n;
    const int step = tile / per_shard, within = tile % per_shard;
    const int shard = (p.peers.rank + step) % p.peers.world;
    if (step == 0) {
      *mb = shard * p.blocks_per_rank + within % p.blocks_per_rank;
      *nb = within / p.blocks_per_rank;
    } else {
      *mb = shard * p.blocks_per_rank + within / g.tiles_n;
      *nb = within % g.tiles_n;
    }
  }
  __device__ static void pair_coords(const Params& p, const Problem& g, int tile, int* mb2, int* nb) {
    const int pairs_per_rank = p.blocks_per_rank / 2;
    const int per_shard = pairs_per_rank * g.tiles_n;
    const int step = tile / per_shard, within = tile % per_shard;
    const int shard = (p.peers.rank + step) % p.peers.world;
    if (step == 0) {
      *mb2 = shard * pairs_per_rank + within % pairs_per_rank;
      *nb = within / pairs_per_rank;
    } else {
      *mb2 = shard * pairs_per_rank + within / g.tiles_n;
      *nb = within % g.tiles_n;
    }
  }
  __device__ static bool before_load(const Params& p, const Problem&, int mb, uint64_t deadline,
                                     const volatile uint32_t* abort_flag) {
    if (mb / p.blocks_per_rank == p.peers.rank) return true;          // the local shard is already there
    const bool ok = wait_flag_ge(p.ready + mb, p.epoch * static_cast<uint32_t>(p.copy_parts), deadline, abort_flag);
    // The rows were written by generic-proxy stores of other CTAs; TMA reads through the async proxy.
    asm volatile("fence.proxy.async.global;" ::: "memory");
    return ok;
  }
  static constexpr bool kSignalsTiles = false;
  __device__ static uint8_t* tile_base(const Params& p, const Problem&, int mb) {
    return reinterpret_cast<uint8_t*>(p.c + static_cast<int64_t>(mb) * kBM * p.ldc);
  }
  __device__ static int64_t row_pitch(const Params& p, const Problem&) { return p.ldc * 2; }
  __device__ static void tile_done(const Params&, const Problem&, int, int) {}
  __device__ static int aux_ctas(const Params& p) { return p.copy_ctas; }

  // Copier CTAs.  CTA 0 first announces "my shard is in place" to every peer.  Then the copiers
  // walk the peers' shards (nearest successor first) in row order: a 128-row block is cut into
  // `copy_parts` parts, part i of the list goes to copier i mod (number of copiers), so at any
  // time all copiers work on the same few blocks and the blocks complete one after another, in
  // the order the GEMM needs them (one copier per block made all blocks complete together, at the
  // end of the copy: most GEMM CTAs then waited 45 us for their first tile in a timeline).  A
  // copier streams its parts through a ring of shared-memory stages without draining between
  // parts: peer memory -> shared memory (bulk copy completing on an mbarrier) -> local gathered
  // matrix (bulk copy in a group), kCopyLag loads in flight; a part is published (ready[mb], and
  // a "read" count at its source) once kDoneLag newer store groups have been committed and the
  // wait for all older groups has returned.  Never a multicast: each copier fetches only its own
  // parts.  Finally CTA 0 waits until every peer has read this rank's shard, so the caller may
  // overwrite its input when the kernel is done.
  static constexpr int kCopyStages = 12, kCopyLag = 8;     // 8 loads of 16 KB in flight, 4 stores pending
  static constexpr int kDoneLag = 3, kDoneFifo = 16;
  static constexpr uint32_t kCopyChunk = 16 * 1024;

  struct CopyPart {
    const uint8_t* from;
    uint8_t* to;
    uint64_t bytes;
    uint32_t chunks;
    int mb, src;
  };
  __device__ static CopyPart copy_part(const Params& p, const Problem& g, int item) {
    const int me = p.peers.rank, world = p.peers.world;
    const uint64_t row_bytes = static_cast<uint64_t>(g.K) * 2;
    const int block_item = item / p.copy_parts, part = item % p.copy_parts;
    CopyPart d;
    d.src = (me + 1 + block_item / p.blocks_per_rank) % world;
    d.mb = d.src * p.blocks_per_rank + block_item % p.blocks_per_rank;
    const uint64_t off = p.gathered_off + static_cast<uint64_t>(d.mb) * kBM * row_bytes;
    const uint64_t rows_here = min(static_cast<int>(kBM), g.M - d.mb * kBM);
    const uint64_t block_vecs = rows_here * row_bytes / 16;
    const uint64_t per_part = (block_vecs + p.copy_parts - 1) / p.copy_parts;
    const uint64_t first = static_cast<uint64_t>(part) * per_part;
    const uint64_t vecs = first >= block_vecs ? 0 : min(per_part, block_vecs - first);
    d.from = p.peers.base[d.src] + off + first * 16;
    d.to = p.peers.base[me] + off + first * 16;
    d.bytes = vecs * 16;
    d.chunks = static_cast<uint32_t>((d.bytes + kCopyChunk - 1) / kCopyChunk);
    return d;
  }

  __device__ static void aux_main(const Params& p, const Problem& g, int cta, int num_ctas, uint64_t deadline,
                                  const volatile uint32_t* abort_flag, uint8_t* smem) {
    __shared__ uint64_t bars[kCopyStages];
    __shared__ int fifo_mb[kDoneFifo], fifo_src[kDoneFifo];
    __shared__ uint32_t fifo_group[kDoneFifo];
    if (threadIdx.x == 0) {
      for (int s = 0; s < kCopyStages; ++s) ptx::mbar_init(&bars[s], 1);
      ptx::mbar_init_fence();
    }
    __syncthreads();
    const int me = p.peers.rank, world = p.peers.world;
    uint32_t* my_flags = reinterpret_cast<uint32_t*>(p.peers.base[me] + p.flags_off);
    if (cta == 0 && static_cast<int>(threadIdx.x) < world && static_cast<int>(threadIdx.x) != me) {
      uint32_t* there = reinterpret_cast<uint32_t*>(p.peers.base[threadIdx.x] + p.flags_off) + me;
      ptx::fence_sys();
      ptx::red_release_sys_add(there, 1u);
    }
    if (threadIdx.x == 0) {
      const int items = (world - 1) * p.blocks_per_rank * p.copy_parts;
      bool ok = true;
      int waited_src = -1;
      auto wait_src = [&](int src) {                       // "shard of rank src is in place"
        if (src == waited_src) return true;
        if (!wait_flag_ge(my_flags + src, p.epoch, deadline, abort_flag)) {
          raise_error(g, kErrPolicyWait, 4);
          return false;
        }
        waited_src = src;
        return true;
      };
      // A part's rows are published locally at once; the "read" counts for its source are added up
      // and posted once, at the end (a system-scope release per part stalled the stream for
      // microseconds each).
      uint32_t parts_read[kMaxRanks] = {};
      auto publish = [&](int mb, int src) {
        ptx::fence_gpu();
        ptx::red_release_gpu_add(p.ready + mb, 1u);
        ++parts_read[src];
      };
      int f_head = 0, f_count = 0;                          // parts stored, not yet known complete
      uint32_t groups = 0;                                  // store groups committed
      auto drain_fifo = [&]() {                             // every committed store has completed
        ptx::bulk_wait_all();
        asm volatile("fence.proxy.async.global;" ::: "memory");
        for (; f_count > 0; --f_count, f_head = (f_head + 1) % kDoneFifo) publish(fifo_mb[f_head], fifo_src[f_head]);
      };
      uint32_t seq_p = 0, seq_c = 0;                        // chunks loaded / stored so far (ring positions)
      int p_item = cta, c_item = cta;
      uint32_t p_chunk = 0, c_chunk = 0;
      bool p_valid = p_item < items, c_valid = c_item < items;
      CopyPart pd{}, cd{};
      if (p_valid) { pd = copy_part(p, g, p_item); ok = wait_src(pd.src); }
      if (c_valid) cd = copy_part(p, g, c_item);
      while (ok) {
        // parts whose last chunk has been stored (or that are empty) join the queue
        while (c_valid && c_chunk == cd.chunks) {
          if (f_count == kDoneFifo) drain_fifo();
          const int slot = (f_head + f_count) % kDoneFifo;
          fifo_mb[slot] = cd.mb; fifo_src[slot] = cd.src; fifo_group[slot] = groups;
          ++f_count;
          c_item += num_ctas; c_valid = c_item < items; c_chunk = 0;
          if (c_valid) cd = copy_part(p, g, c_item);
        }
        while (ok && p_valid && p_chunk == pd.chunks) {
          p_item += num_ctas; p_valid = p_item < items; p_chunk = 0;
          if (p_valid) { pd = copy_part(p, g, p_item); ok = wait_src(pd.src); }
        }
        if (!ok) break;
        // publish the oldest part once kDoneLag newer groups exist: waiting for "all but the newest
        // kDoneLag groups" then covers its stores and does not stall the stream
        if (f_count > 0 && groups - fifo_group[f_head] >= static_cast<uint32_t>(kDoneLag)) {
          ptx::bulk_wait_group<kDoneLag>();
          asm volatile("fence.proxy.async.global;" ::: "memory");
          while (f_count > 0 && groups - fifo_group[f_head] >= static_cast<uint32_t>(kDoneLag)) {
            publish(fifo_mb[f_head], fifo_src[f_head]);
            f_head = (f_head + 1) % kDoneFifo; --f_count;
          }
        }
        if (p_valid && seq_p - seq_c < static_cast<uint32_t>(kCopyLag)) {
          // produce: the store that last read this stage (kCopyStages chunks ago) must be done reading
          const uint32_t len = static_cast<uint32_t>(min(static_cast<uint64_t>(kCopyChunk), pd.bytes - static_cast<uint64_t>(p_chunk) * kCopyChunk));
          ptx::bulk_wait_read<kCopyStages - kCopyLag>();
          ptx::mbar_expect_tx(&bars[seq_p % kCopyStages], len);
          ptx::bulk_load(smem + (seq_p % kCopyStages) * kCopyChunk, pd.from + static_cast<uint64_t>(p_chunk) * kCopyChunk, len,
                         &bars[seq_p % kCopyStages]);
          ++seq_p; ++p_chunk;
          continue;
        }
        if (seq_c < seq_p) {
          // consume: wait for the oldest load, store it
          const uint32_t len = static_cast<uint32_t>(min(static_cast<uint64_t>(kCopyChunk), cd.bytes - static_cast<uint64_t>(c_chunk) * kCopyChunk));
          if (!ptx::mbar_wait(&bars[seq_c % kCopyStages], (seq_c / kCopyStages) & 1u, deadline, abort_flag)) {
            raise_error(g, kErrPolicyWait, 8);
            ok = false;
            break;
          }
          ptx::bulk_store(cd.to + static_cast<uint64_t>(c_chunk) * kCopyChunk, smem + (seq_c % kCopyStages) * kCopyChunk, len);
          ptx::bulk_commit();
          ++groups; ++seq_c; ++c_chunk;
          continue;
        }
        break;                                              // nothing left to load, nothing in flight
      }
      if (ok) {
        drain_fifo();
        for (int r = 0; r < world; ++r)
          if (parts_read[r])
            ptx::red_release_sys_add(reinterpret_cast<uint32_t*>(p.peers.base[r] + p.flags_off) + world + me, parts_read[r]);
      } else {
        // Leaving early: wait (bounded) for the loads still writing this CTA's shared memory.
        const uint64_t drain = ptx::globaltimer() + 50000000ull;
        uint32_t no_abort = 0;
        for (uint32_t c = seq_c; c < seq_p; ++c) ptx::mbar_wait(&bars[c % kCopyStages], (c / kCopyStages) & 1u, drain, &no_abort);
        ptx::bulk_wait_all();
      }
    }
    __syncthreads();
    if (cta == 0 && !*abort_flag) {
      // Every peer posts blocks_per_rank * copy_parts "read" counts per call.
      if (static_cast<int>(threadIdx.x) < world && static_cast<int>(threadIdx.x) != me) {
        const uint32_t want = p.epoch * static_cast<uint32_t>(p.blocks_per_rank * p.copy_parts);
        if (!wait_flag_ge(my_flags + world + threadIdx.x, want, deadline, abort_flag))
          raise_error(g, kErrPolicyWait, 5);
      }
    }
  }
  __device__ static void finish(const Params&, const Problem&, int, int, uint64_t, const volatile uint32_t*) {}
};

// All-gather -> GEMM with the SwiGLU of a gated feed-forward in the epilogue: the weight stacks the
// gate and up projections interleaved in groups of 16 rows (16 gate rows, then the 16 up rows of
// the same hidden units), so every 32 accumulator columns hold both halves of 16 outputs and the
// kernel writes act[M][N / 2] = silu(gate) * up directly.  The [M][N] pre-activation never
// reaches memory and the element-wise kernel between the two GEMMs of the block disappears.
struct AllGatherSwigluPolicy : AllGatherPolicy {
  static constexpr int kOutPer32 = 16;
  static constexpr bool kSplitTail = false;        // the split tail sums plain accumulators only
  __device__ static void transform(const float* acc, float, float* out) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float gate = acc[i];
      out[i] = gate / (1.f + __expf(-gate)) * acc[16 + i];
    }
  }
};

}  // namespace gemm
}  // namespace pccl
