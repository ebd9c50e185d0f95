// Plan loading, validation and lowering.
//
// load_plan      JSON text (version-2 device plan) -> Plan (host representation).
//                Accepts every executor string and primitive name the reference
//                emits, including bare "notify" / "wait_notify" / "noop"
//                (reference: csrc/engine/graph_builder.cc:12-107 and the channel
//                parsers csrc/plugins/cuda/channels/*.h for the field mapping).
// validate_plan  one rank's plan on its own: bounds of every range, peer and signal id.
// check_world    all ranks' plans together: abstract execution of the signal protocol (deadlock,
//                signals left over, posts nobody consumes) and a 16-byte alignment report.
// lower_plan     Plan -> LoweredProgram: chains of steps in plan order (program.h).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "../common/json.h"
#include "../executors/sm100/program.h"

namespace pccl {

enum class Primitive {
  kNoop, kNotify, kWait, kCopy, kReduce, kPut, kReduceMulti, kMmReduce, kMmStore, kMmAllreduce, kCeCopy,
};

struct PlanOp {
  int index = 0;
  Primitive primitive = Primitive::kNoop;
  std::string primitive_name, executor;
  int channel = 0;
  std::vector<int> deps, next;
  // data parameters, in elements
  int peer = -1;                  // source_rank / target_rank
  std::vector<int> sources;       // reduce_multi
  int64_t off_src = 0, off_dst = 0, off_remote = 0, count = 0;
  uint8_t red_op = kRedSum;
  bool avg = false;
  uint32_t signal_id = 0;
};

struct Plan {
  int version = 2;
  uint8_t dtype = kF32;
  std::string dtype_name;
  int64_t numel = 0;
  std::string collective_type, algorithm;
  std::vector<PlanOp> ops;
  bool uses_avg = false;
  bool has_ce_ops = false;
  int num_channels = 1;
};

Plan load_plan(const std::string& json_text);

struct PlanLimits {
  int rank = 0, world = 1;
  int64_t buffer_elems = 0;       // elements of the plan dtype that fit the data region
};
// Throws pccl::Error describing the first violation.
void validate_plan(const Plan& plan, const PlanLimits& limits);

// Result of executing the signal protocol of all ranks' plans together, data left out: an operation
// runs when its dependencies ran, a wait_notify when its semaphore is positive.
struct WorldReport {
  bool deadlock = false;          // some rank could not finish
  std::string detail;             // who is blocked on what (deadlock), or which signals are left over
  int leftover_signals = 0;       // semaphores non-zero at the end: the plan cannot be re-run without a reset
  int misaligned_ops = 0;         // data operations whose offsets or size are not multiples of 16 bytes
                                  // (they run on the element-wise path, and never on multimem)
  int64_t notifies = 0, waits = 0;
};
// `plans[r]` is rank r's plan.  Never throws for protocol errors: the caller decides.
WorldReport check_world(const std::vector<Plan>& plans);

struct LowerOptions {
  int rank = 0, world = 1;
  bool multicast = false;         // NVLS mapping available
  uint32_t total_ctas = 16;       // CTA budget for the whole program
  uint32_t max_ctas_per_chain = 64;
  bool defer_barriers = true;             // merge runs of independent copies / puts into barrier-free runs
  uint64_t min_bytes_per_cta = 64 << 10;   // do not spread less than this over another CTA
  bool force_copy_engine = false; // route pull copies to the copy-engine executor
  // Append an all-pairs barrier after the last step.  Pull-style templates (ring, tree,
  // halving-doubling) let a rank finish while a neighbour still reads its buffer; the
  // barrier keeps the next operation's input copy from overwriting data in use.
  bool closing_barrier = false;
};

struct LoweredProgram {
  std::vector<Step> steps;
  std::vector<SigRef> sigs;
  std::vector<ChainDep> deps;
  std::vector<Chain> chains;
  uint32_t total_ctas = 0;
  bool uses_multicast = false;
  uint64_t max_step_bytes = 0;
};

LoweredProgram lower_plan(const Plan& plan, const LowerOptions& opt);

const char* primitive_label(Primitive p);

}  // namespace pccl
