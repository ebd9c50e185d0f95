// OCS control-plane exchange over NVLink: the fast connector's native half.
//
// An OCS barrier has two rounds of tiny messages: every rank contributes its READY record and
// sees everyone's (an all-gather of a few words), then the leader's switch result is delivered to
// all (a broadcast).  The reference does both with pickled-object collectives on the host
// (pccl/ocs/runtime.py:139-203: all_gather_object + broadcast_object_list, hundreds of
// microseconds).  Here each round is one single-CTA kernel: a thread per peer stores this rank's
// record into a slot of the peer's symmetric memory (plain stores followed by a release store of
// the round number), a thread per source waits (bounded) for that source's round number with
// acquire loads, and the received records are written to pinned host memory mapped into the GPU,
// followed by a completion word the host spins on.  No stream synchronisation, no host collective.
//
// Slots are double-buffered by round parity: a rank can run at most one round ahead of a peer
// (finishing round n needs every peer's record of round n), so parity n is never overwritten
// while a peer still reads it.  Every device wait has a time limit; when it runs out the kernel
// reports which source was missing and returns, and the host raises.
#pragma once
#include <cuda_runtime.h>

#include <array>
#include <cstdint>
#include <vector>

namespace pccl {

class RankContext;

constexpr int kBoardWords = 14;          // payload words (u32) per record
constexpr int kBoardSlotWords = 16;      // payload + source rank + round number

struct BoardStatus {
  bool ok = true;
  int missing_rank = -1;                 // first source whose record did not arrive in time
  double host_us = 0.0;                  // launch to completion as seen by the host
};

class SignalBoard {
 public:
  // Collective: every rank constructs its board at the same point (the slots come from the
  // symmetric arena) and synchronises the ranks before the first round.
  explicit SignalBoard(RankContext& ctx);
  ~SignalBoard();
  SignalBoard(const SignalBoard&) = delete;
  SignalBoard& operator=(const SignalBoard&) = delete;

  // Every rank passes its record; on return `records[r]` holds rank r's (this rank's included).
  BoardStatus all_gather(const std::array<uint32_t, kBoardWords>& mine,
                         std::vector<std::array<uint32_t, kBoardWords>>* records, uint64_t timeout_us);
  // `record` travels from `root` to every rank (in place).
  BoardStatus broadcast(int root, std::array<uint32_t, kBoardWords>* record, uint64_t timeout_us);
  // Both rounds of an OCS barrier in one launch, for a leader that has nothing to do on the host
  // between them: all-gather of the READY records, then the leader (`root`) sends `release` to
  // everyone once all records are in.  The leader compares words [compare_begin, compare_end) of
  // every record with its own and clears word 0 of the release when they differ.
  BoardStatus gather_release(int root, const std::array<uint32_t, kBoardWords>& mine,
                             const std::array<uint32_t, kBoardWords>& release, int compare_begin, int compare_end,
                             std::vector<std::array<uint32_t, kBoardWords>>* records,
                             std::array<uint32_t, kBoardWords>* released, uint64_t timeout_us);
  // A barrier with no payload: one all-gather round.
  BoardStatus barrier(uint64_t timeout_us);

  // After a failed round the ranks are out of step: zero the slots and restart the round count.
  // Collective, between two host barriers.
  void reset();
  int world() const { return world_; }
  uint64_t rounds() const { return gather_round_ + bcast_round_; }

 private:
  BoardStatus run(int kind, int root, const uint32_t* payload, uint32_t round, uint64_t timeout_us,
                  const uint32_t* release, uint32_t release_round, int compare_begin, int compare_end);

  RankContext& ctx_;
  int rank_, world_;
  uint64_t slots_off_ = 0;               // symmetric: u32 [2 kinds][2 parities][world][kBoardSlotWords]
  size_t slots_bytes_ = 0;
  uint32_t* host_block_ = nullptr;       // pinned, mapped: [world + 1][kBoardSlotWords] records, release | done | status
  uint32_t* host_block_dev_ = nullptr;
  cudaStream_t stream_ = nullptr;
  uint32_t gather_round_ = 0, bcast_round_ = 0;
};

}  // namespace pccl
