#include "signal_board.h"

#include <chrono>
#include <cstring>

#include "../common/util.h"
#include "../engine/cuda_driver.h"
#include "../engine/engine.h"
#include "../ptx/sync.cuh"

namespace pccl {

namespace {

enum : int { kKindGather = 0, kKindBroadcast = 1, kKindGatherRelease = 2 };

struct BoardParams {
  uint8_t* base[kMaxRanks];      // every rank's heap as mapped here
  uint64_t slots_off;
  int rank, world, kind, root;
  uint32_t round;                // gather round number (kinds 0 and 2) or broadcast round number (kind 1)
  uint32_t release_round;        // kind 2: round number of the leader's release on the broadcast slots
  uint32_t payload[kBoardWords];
  uint32_t release[kBoardWords]; // kind 2, on the root: the record to release with once all arrived
  int compare_begin, compare_end; // kind 2: payload words [begin, end) must be equal on all ranks for release[0] to stay set
  uint32_t* host_records;        // mapped pinned [world + 1][kBoardSlotWords]; row `world` = the release
  uint32_t* host_done;           // mapped pinned: completion word
  uint32_t* host_status;         // mapped pinned: 0 ok, 1 + source rank on a timeout
  uint64_t timeout_ns;
};

__device__ __forceinline__ uint32_t* slot_of(uint8_t* heap, uint64_t slots_off, int world, int kind, uint32_t parity,
                                             int source) {
  return reinterpret_cast<uint32_t*>(heap + slots_off) +
         ((static_cast<uint64_t>(kind) * 2 + parity) * world + source) * kBoardSlotWords;
}

__device__ __forceinline__ void send_record(uint32_t* dst, const uint32_t* words, int rank, uint32_t round) {
#pragma unroll
  for (int w = 0; w < kBoardWords; ++w) ptx::st_relaxed_sys(dst + w, words[w]);
  ptx::st_relaxed_sys(dst + kBoardWords, static_cast<uint32_t>(rank));
  // Release: the record words above are visible before the round number.
  ptx::st_release_sys(dst + kBoardWords + 1, round);
}

// Bounded wait for `round` in a slot of this rank's memory; then the slot is copied to host memory
// as four 16-byte stores.
__device__ __forceinline__ bool receive_record(const uint32_t* src, uint32_t round, uint64_t deadline,
                                               uint32_t* host_row, uint32_t* keep) {
  uint32_t spins = 0;
  while (ptx::ld_acquire_sys(src + kBoardWords + 1) != round) {
    if ((++spins & 31u) == 0u && ptx::globaltimer() > deadline) return false;
  }
  uint4 v[kBoardSlotWords / 4];
#pragma unroll
  for (int q = 0; q < kBoardSlotWords / 4; ++q) v[q] = ptx::ld_local_v4(src + 4 * q);
#pragma unroll
  for (int q = 0; q < kBoardSlotWords / 4; ++q) reinterpret_cast<uint4*>(host_row)[q] = v[q];
  if (keep) {
#pragma unroll
    for (int q = 0; q < kBoardSlotWords / 4; ++q) reinterpret_cast<uint4*>(keep)[q] = v[q];
  }
  return true;
}

// One CTA, one warp.  Lane t < world sends to peer t and then receives from source t.
__global__ void __launch_bounds__(32) ocs_board_kernel(const BoardParams p) {
  __shared__ __align__(16) uint32_t seen[kMaxRanks][kBoardSlotWords];
  const int lane = static_cast<int>(threadIdx.x);
  const bool gathers = p.kind != kKindBroadcast;
  const uint64_t deadline = ptx::globaltimer() + p.timeout_ns;
  if (lane < p.world && (gathers || p.rank == p.root))
    send_record(slot_of(p.base[lane], p.slots_off, p.world, gathers ? kKindGather : kKindBroadcast, p.round & 1u,
                        p.rank), p.payload, p.rank, p.round);
  bool ok = true;
  const bool receives = lane < p.world && (gathers || lane == p.root);
  if (receives)
    ok = receive_record(slot_of(p.base[p.rank], p.slots_off, p.world, gathers ? kKindGather : kKindBroadcast,
                                p.round & 1u, lane),
                        p.round, deadline, p.host_records + lane * kBoardSlotWords, seen[lane]);
  uint32_t failed = __ballot_sync(0xffffffffu, receives && !ok);
  if (p.kind == kKindGatherRelease && failed == 0u) {
    // Everyone has arrived.  The leader compares the agreed words of all records with its own and
    // releases; every rank then waits for that one record.
    __syncwarp();
    if (p.rank == p.root) {
      bool same = true;
      if (lane < p.world)
        for (int w = p.compare_begin; w < p.compare_end; ++w) same &= seen[lane][w] == p.payload[w];
      const bool all_same = __all_sync(0xffffffffu, same);
      if (lane < p.world) {
        uint32_t words[kBoardWords];
#pragma unroll
        for (int w = 0; w < kBoardWords; ++w) words[w] = p.release[w];
        if (!all_same) words[0] = 0u;
        send_record(slot_of(p.base[lane], p.slots_off, p.world, kKindBroadcast, p.release_round & 1u, p.rank), words,
                    p.rank, p.release_round);
      }
    }
    bool got = true;
    if (lane == 0)
      got = receive_record(slot_of(p.base[p.rank], p.slots_off, p.world, kKindBroadcast, p.release_round & 1u, p.root),
                           p.release_round, deadline, p.host_records + p.world * kBoardSlotWords, nullptr);
    if (__ballot_sync(0xffffffffu, !got)) failed = 1u << p.root;
  }
  if (lane == 0) {
    *reinterpret_cast<volatile uint32_t*>(p.host_status) = failed ? static_cast<uint32_t>(__ffs(failed)) : 0u;
    __threadfence_system();                     // records and status reach host memory before the completion word
    *reinterpret_cast<volatile uint32_t*>(p.host_done) = p.round | (static_cast<uint32_t>(p.kind) << 30);
  }
}

}  // namespace

SignalBoard::SignalBoard(RankContext& ctx) : ctx_(ctx), rank_(ctx.rank()), world_(ctx.world()) {
  slots_bytes_ = static_cast<size_t>(2) * 2 * world_ * kBoardSlotWords * sizeof(uint32_t);
  slots_off_ = ctx_.arena_alloc(slots_bytes_, 256);
  PCCL_CUDA(cudaMemset(ctx_.heap().data(rank_) + slots_off_, 0, slots_bytes_));
  const size_t host_bytes = (static_cast<size_t>(world_ + 1) * kBoardSlotWords + 2) * sizeof(uint32_t);
  PCCL_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&host_block_), host_bytes, cudaHostAllocMapped));
  std::memset(host_block_, 0, host_bytes);
  PCCL_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&host_block_dev_), host_block_, 0));
  int least = 0, greatest = 0;
  PCCL_CUDA(cudaDeviceGetStreamPriorityRange(&least, &greatest));
  PCCL_CUDA(cudaStreamCreateWithPriority(&stream_, cudaStreamNonBlocking, greatest));
  PCCL_CUDA(cudaDeviceSynchronize());
}

SignalBoard::~SignalBoard() {
  if (stream_) { cudaStreamSynchronize(stream_); cudaStreamDestroy(stream_); }
  if (host_block_) cudaFreeHost(host_block_);
}

void SignalBoard::reset() {
  PCCL_CUDA(cudaStreamSynchronize(stream_));
  PCCL_CUDA(cudaMemset(ctx_.heap().data(rank_) + slots_off_, 0, slots_bytes_));
  PCCL_CUDA(cudaDeviceSynchronize());
  std::memset(host_block_, 0, (static_cast<size_t>(world_ + 1) * kBoardSlotWords + 2) * sizeof(uint32_t));
  gather_round_ = bcast_round_ = 0;
}

BoardStatus SignalBoard::run(int kind, int root, const uint32_t* payload, uint32_t round, uint64_t timeout_us,
                             const uint32_t* release, uint32_t release_round, int compare_begin, int compare_end) {
  BoardParams p{};
  for (int r = 0; r < world_; ++r) {
    PCCL_CHECK(ctx_.heap().has_peer(r), "OCS signal board: rank " << r << " is not connected");
    p.base[r] = ctx_.heap().data(r);
  }
  p.slots_off = slots_off_;
  p.rank = rank_; p.world = world_; p.kind = kind; p.root = root;
  p.round = round;
  p.release_round = release_round;
  p.compare_begin = compare_begin; p.compare_end = compare_end;
  if (payload) std::memcpy(p.payload, payload, sizeof p.payload);
  if (release) std::memcpy(p.release, release, sizeof p.release);
  p.host_records = host_block_dev_;
  p.host_done = host_block_dev_ + (world_ + 1) * kBoardSlotWords;
  p.host_status = p.host_done + 1;
  p.timeout_ns = timeout_us * 1000ull;
  volatile uint32_t* done = host_block_ + (world_ + 1) * kBoardSlotWords;
  volatile uint32_t* status = done + 1;
  const uint32_t want = round | (static_cast<uint32_t>(kind) << 30);
  const auto t0 = std::chrono::steady_clock::now();
  ocs_board_kernel<<<1, 32, 0, stream_>>>(p);
  PCCL_CUDA(cudaGetLastError());
  // The kernel's own limit ends its wait; the host allows it a margin on top.
  const auto host_deadline = t0 + std::chrono::microseconds(timeout_us + 2000000);
  BoardStatus out;
  uint32_t polls = 0;
  while (*done != want) {
    if ((++polls & 1023u) == 0u && std::chrono::steady_clock::now() > host_deadline) {
      out.ok = false;
      out.host_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
      return out;
    }
#if defined(__x86_64__)
    __builtin_ia32_pause();
#endif
  }
  out.host_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
  const uint32_t st = *status;
  if (st != 0) { out.ok = false; out.missing_rank = static_cast<int>(st) - 1; }
  return out;
}

BoardStatus SignalBoard::gather_release(int root, const std::array<uint32_t, kBoardWords>& mine,
                                        const std::array<uint32_t, kBoardWords>& release, int compare_begin,
                                        int compare_end, std::vector<std::array<uint32_t, kBoardWords>>* records,
                                        std::array<uint32_t, kBoardWords>* released, uint64_t timeout_us) {
  PCCL_CHECK(root >= 0 && root < world_, "OCS signal board: root " << root << " outside the world");
  PCCL_CHECK(compare_begin >= 0 && compare_begin <= compare_end && compare_end <= kBoardWords,
             "OCS signal board: compared words outside the record");
  const uint32_t g = ++gather_round_, b = ++bcast_round_;
  const BoardStatus st = run(kKindGatherRelease, root, mine.data(), g, timeout_us, release.data(), b, compare_begin,
                             compare_end);
  if (st.ok) {
    if (records) {
      records->resize(world_);
      for (int r = 0; r < world_; ++r)
        std::memcpy((*records)[r].data(), host_block_ + r * kBoardSlotWords, kBoardWords * sizeof(uint32_t));
    }
    if (released) std::memcpy(released->data(), host_block_ + world_ * kBoardSlotWords, kBoardWords * sizeof(uint32_t));
  }
  return st;
}

BoardStatus SignalBoard::all_gather(const std::array<uint32_t, kBoardWords>& mine,
                                    std::vector<std::array<uint32_t, kBoardWords>>* records, uint64_t timeout_us) {
  const BoardStatus st = run(kKindGather, 0, mine.data(), ++gather_round_, timeout_us, nullptr, 0, 0, 0);
  if (st.ok && records) {
    records->resize(world_);
    for (int r = 0; r < world_; ++r)
      std::memcpy((*records)[r].data(), host_block_ + r * kBoardSlotWords, kBoardWords * sizeof(uint32_t));
  }
  return st;
}

BoardStatus SignalBoard::broadcast(int root, std::array<uint32_t, kBoardWords>* record, uint64_t timeout_us) {
  PCCL_CHECK(root >= 0 && root < world_, "OCS signal board: root " << root << " outside the world");
  const BoardStatus st = run(kKindBroadcast, root, record->data(), ++bcast_round_, timeout_us, nullptr, 0, 0, 0);
  if (st.ok) std::memcpy(record->data(), host_block_ + root * kBoardSlotWords, kBoardWords * sizeof(uint32_t));
  return st;
}

BoardStatus SignalBoard::barrier(uint64_t timeout_us) {
  std::array<uint32_t, kBoardWords> none{};
  return all_gather(none, nullptr, timeout_us);
}

}  // namespace pccl
