// Device-visible description of one rank's lowered plan: the "step program".
//
// A plan (JSON) is lowered on the host into *chains*: linear sequences of steps
// that run in order on a dedicated group of CTAs.  A step is
//     [wait on signals / on other chains]  ->  [one data operation]  ->  [post signals]
// in exactly the order the plan lists them.  Plans whose channels are linear
// (every reference template) map one channel to one chain; arbitrary DAGs are
// split into several chains with cross-chain progress counters, so DAG
// semantics hold without a device-side scheduler.  (The reference instead
// interprets a DAG with ready-queues, ~1.2 us per primitive, or a "fused" list
// limited to 128 steps / 8 channels that posts a step's notify before its wait:
// csrc/engine/graph_builder.cc:163-316, csrc/plugins/cuda/cuda_executor.cu:963-1057.)
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define PCCL_HD __host__ __device__
#else
#define PCCL_HD
#endif

namespace pccl {

constexpr int kMaxRanks = 8;            // GPUs in one NVSwitch domain addressed by a plan
constexpr uint32_t kSignalSlots = 65536;  // counting semaphores per rank (32 channels x 1000 ids fit)
constexpr int kMaxVirtualRanks = 8;     // ranks emulated by one launch on one GPU (tests)

enum StepKind : uint8_t {
  kStepNoop = 0,
  kStepCopy,         // self[off1] = rank[peer][off0]
  kStepReduce,       // self[off2] = rank[peer][off0] (op) self[off1]
  kStepPut,          // rank[peer][off1] = self[off0]
  kStepReduceMulti,  // self[off2] = (op) over set bits r of peer_mask: rank[r][off0]
  kStepMmReduce,     // self[off2] = multimem.ld_reduce(mc[off0])
  kStepMmStore,      // multimem.st(mc[off1]) = self[off0]
  kStepMmAllreduce,  // multimem.st(mc[off0]) = multimem.ld_reduce(mc[off0])
  kStepScale,        // self[off0] *= scale   (the final 1/N of an "avg" reduction)
};

enum RedOp : uint8_t { kRedSum = 0, kRedMax = 1, kRedMin = 2 };
enum DType : uint8_t { kF32 = 0, kF16 = 1, kBF16 = 2, kE4M3 = 3, kE5M2 = 4 };

PCCL_HD inline int dtype_bytes(uint8_t d) { return d == kF32 ? 4 : (d <= kBF16 ? 2 : 1); }

struct SigRef {       // one semaphore operation
  int32_t rank;       // notify: rank whose slot is incremented; wait: informational
  uint32_t slot;      // index into that rank's signal array
};

struct ChainDep {     // "chain `chain` must have finished `steps_done` steps of this launch"
  uint32_t chain;
  uint32_t steps_done;
};

struct Step {
  uint8_t kind, red_op, n_wait, n_notify;
  uint8_t n_dep, writes_remote;
  uint8_t defer_barrier;   // 1: the next step is an independent copy / put, no completion barrier here
  uint8_t reserved;
  int32_t peer;
  uint32_t peer_mask;
  uint32_t sig_begin;    // waits are sigs[sig_begin .. +n_wait), notifies follow
  uint32_t dep_begin;
  float scale;
  uint64_t off0, off1, off2;   // byte offsets into a rank's data region
  uint64_t bytes;
};
static_assert(sizeof(Step) == 64, "Step is one 64-byte record");

struct Chain {
  uint32_t step_begin, step_count;
  uint32_t first_cta, num_ctas;
  uint32_t barriers_per_launch;   // channel barriers one launch performs (for monotonic counters)
  uint32_t reserved[3];
};

// Written by the first device thread that gives up waiting; read by the host
// after the launch.  code 0 = success.
struct DeviceStatus {
  uint32_t abort;      // raised once; every wait polls it
  uint32_t code;       // 1 = signal wait timed out, 2 = chain barrier timed out, 3 = chain dep timed out
  int32_t rank;
  uint32_t chain, step;
  uint32_t slot;       // signal slot (code 1)
  uint32_t observed;   // value seen when giving up
  uint32_t expected;
};

enum StatusCode : uint32_t { kOk = 0, kSignalTimeout = 1, kBarrierTimeout = 2, kDepTimeout = 3 };

struct RankProgram {
  int32_t rank, world;
  uint32_t dtype, num_chains;
  uint8_t* data[kMaxRanks];        // every rank's data region as mapped into this GPU
  uint32_t* signals[kMaxRanks];    // every rank's signal array
  uint8_t* mc_data;                // multicast alias of the data region (null without NVLS)
  const Step* steps;
  const SigRef* sigs;
  const ChainDep* deps;
  const Chain* chains;
  uint32_t* chain_sync;            // [num_chains] monotonically increasing barrier counters
  uint32_t* chain_progress;        // [num_chains] monotonically increasing finished-step counters
  DeviceStatus* status;            // device copy: abort flag polled by every wait
  DeviceStatus* host_status;       // pinned host mirror, written once by the failing thread
  uint64_t timeout_ns;
  // Optional timeline of the most recent launch (null = tracing off): kTraceStamps
  // %globaltimer values per step, written by thread 0 of the chain's lead CTA.
  uint64_t* trace;
};

// Stamps of one step: [0] step reached, [1] waits satisfied and followers released (data starts),
// [2] completion barrier passed (every CTA's data is written), [3] signals posted.
constexpr int kTraceStamps = 4;

struct LaunchParams {
  const RankProgram* programs;     // [gridDim.y]
  uint32_t launch_index;           // number of earlier launches of this op since the last reset
};

// Threads per interpreter CTA.  256 rather than 512: the data movers keep two register tiles of
// 16-byte loads in flight per thread, which needs the 255-register budget.
constexpr uint32_t kInterpThreads = 256;

// Host-callable launchers (defined in interp_kernel.cu).
struct LaunchConfig { uint32_t ctas, threads, virtual_ranks; bool cooperative; uint32_t dtype; };
int launch_plan_interp(const LaunchParams& params, const LaunchConfig& cfg, void* stream);
int plan_interp_max_ctas(int threads);
// Data-mover tuning: bit 0 = two register tiles in flight per thread, bit 1 = strong peer loads.
int set_mover_tuning(uint32_t word);
// ptr[0..bytes) *= scale, interpreted as `dtype` (the epilogue of an "avg" reduction).
int launch_scale(void* ptr, uint64_t bytes, uint32_t dtype, float scale, void* stream);

}  // namespace pccl
