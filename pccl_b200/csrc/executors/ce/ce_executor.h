// Copy-engine executor: a host-driven way to run a lowered plan.
//
// Every chain of the program gets its own CUDA stream.  Pull copies are issued as
// cudaMemcpyAsync from the peer's mapped heap (the DMA engines move the bytes, no SM is used);
// everything between two copies of a chain (signal waits and posts, reductions) runs as a
// small launch of the plan interpreter over just those steps.  The caller's stream forks into
// the chain streams and joins them again with events, so the operation keeps stream semantics.
// Chosen when a plan contains `ce.copy` operations or PCCL_EXECUTOR=ce.
// Restriction: chains must not depend on one another (true for every template); such plans
// stay on the SM executor.
// (The reference lets its persistent kernel enqueue copy commands to a host proxy thread and
// spin on a host flag: csrc/plugins/host/ce_proxy.cc:23-86, cuda_executor.cu:763-794.)
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <vector>

#include "../../engine/plan.h"
#include "../sm100/program.h"

namespace pccl {

struct CeItem {
  enum Part : uint8_t { kWholeSteps, kWaitsOfCopy, kNotifiesOfCopy };
  bool is_copy = false;
  Part part = kWholeSteps;          // kernel items: whole steps, or one half of a DMA'd copy step
  // copy
  int src_rank = 0;
  uint64_t src_off = 0, dst_off = 0, bytes = 0;
  // kernel segment: steps [step_begin, step_begin + step_count) of the chain
  uint32_t step_begin = 0, step_count = 0, ctas = 1;
  uint32_t barriers_per_launch = 0;
  RankProgram* d_program = nullptr;     // one-chain program for this segment
  uint32_t* counters = nullptr;         // its chain_sync / chain_progress pair
};

class CeSchedule {
 public:
  CeSchedule() = default;
  ~CeSchedule();
  CeSchedule(const CeSchedule&) = delete;
  CeSchedule& operator=(const CeSchedule&) = delete;

  // True if the lowered program can run on this executor (no cross-chain dependencies).
  static bool supports(const LoweredProgram& lp);
  // Build the per-chain item lists.  `base` is the op's full program (pointers valid on device);
  // copies smaller than `min_copy_bytes` stay inside kernel segments.
  void build(const LoweredProgram& lp, const RankProgram& base, uint64_t min_copy_bytes);
  // Enqueue one execution.  data[r] = rank r's heap base as mapped here.
  void run(uint8_t* const* data, int self, uint32_t launch_index, cudaStream_t stream);
  void reset_counters();
  size_t num_copies() const { return copies_; }
  size_t num_segments() const { return segments_; }

 private:
  uint32_t dtype_ = 0;                  // element type of the plan (selects the kernel instance)
  void clear();
  std::vector<std::vector<CeItem>> chains_;
  std::vector<cudaStream_t> streams_;
  std::vector<cudaEvent_t> done_;
  cudaEvent_t fork_ = nullptr;
  void* d_chain_tables_ = nullptr;
  size_t copies_ = 0, segments_ = 0;
};

}  // namespace pccl
