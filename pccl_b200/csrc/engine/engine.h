// The engine: registers plans, owns the symmetric heap, launches executors.
//
//   RankContext   everything one rank needs: heap, registered operations, device
//                 tables, status block.  Free of process-level assumptions, so a
//                 LocalCluster can hold several in one process.
//   Engine        the per-process singleton behind pccl.engine (rank from $RANK):
//                 RankContext + fd server + endpoint exchange + NVLS bring-up.
//                 Verb names follow the reference (regOp / exeOp / exeOpAsync /
//                 syncOp / resetSignals / exportEndpoint / updateEndpoint,
//                 reference: include/engine/engine.h:21-46, csrc/engine_c.cc:166-678).
//   LocalCluster  N virtual ranks on one GPU executed by one cooperative launch;
//                 exercises exactly the device code of the multi-GPU path.
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../common/fd_socket.h"
#include "../common/json.h"
#include "../executors/ce/ce_executor.h"
#include "heap.h"
#include "plan.h"

namespace pccl {

struct OpStats {
  uint64_t calls = 0, bytes = 0;
  std::string algorithm, collective;
  uint32_t chains = 0, ctas = 0, steps = 0;
  bool multicast = false, copy_engine = false;
};

struct RegisteredOp {
  std::string name;
  Plan plan;
  LoweredProgram lowered;
  void* d_tables = nullptr;             // steps | sigs | deps | chains in one allocation
  size_t tables_bytes = 0;
  RankProgram host_program{};           // pointers filled for this rank
  RankProgram* d_program = nullptr;     // device copy (Engine mode)
  uint32_t* chain_sync = nullptr;       // control-area counters
  uint32_t* chain_progress = nullptr;
  uint64_t* d_trace = nullptr;          // kTraceStamps timestamps per step when tracing is on
  uint32_t launch_index = 0;
  uint32_t threads = kInterpThreads;
  std::unique_ptr<CeSchedule> ce;       // set when the copy-engine executor runs this operation
  OpStats stats;
};

struct IoSegment { size_t heap_offset, user_offset, bytes; };

// One step of the most recent launch as the device saw it (times in ns since the launch's first stamp).
struct TraceStep {
  uint32_t chain, step, kind, ctas;
  uint64_t bytes;
  uint64_t t[kTraceStamps];
};

class RankContext {
 public:
  RankContext(int rank, int world, int device, size_t buffer_bytes, size_t arena_bytes, bool shareable);
  ~RankContext();

  int rank() const { return rank_; }
  int world() const { return world_; }
  SymmetricHeap& heap() { return heap_; }
  size_t buffer_bytes() const { return buffer_bytes_; }

  // Load + validate + lower + upload.  Re-registering a name replaces it.
  RegisteredOp& register_op(const std::string& name, const std::string& json_text);
  RegisteredOp& op(const std::string& name);
  bool has_op(const std::string& name) const { return ops_.count(name) != 0; }
  // (Re)build device tables; called lazily when peers / NVLS changed after registration.
  void upload(RegisteredOp& op);

  std::vector<IoSegment> input_segments(const RegisteredOp& op, size_t user_bytes) const;
  std::vector<IoSegment> output_segments(const RegisteredOp& op, size_t user_bytes) const;
  void stage_in(const RegisteredOp& op, const void* user, size_t bytes, cudaStream_t stream);
  void stage_out(const RegisteredOp& op, void* user, size_t bytes, cudaStream_t stream);
  void scale_output(RegisteredOp& op, void* user, size_t bytes, cudaStream_t stream);

  DeviceStatus* device_status() const { return d_status_; }
  const DeviceStatus* host_status() const { return h_status_; }
  void clear_status();
  // Throws TimeoutError describing the recorded failure, if any (and clears it).
  void check_status(const std::string& op_name);
  // Zero signals, counters, status; launch indices restart.  Collective: all ranks
  // must call it between two host barriers.
  void reset();
  void reset_op_counters(RegisteredOp& op);

  // Device timeline (optional, PCCL_TRACE=1 or set_trace): every step of a launch stamps
  // %globaltimer four times; read_trace returns the most recent launch of `op` after a
  // synchronize.  The replacement for an external timeline profiler (the reference relies on
  // nsys + tests/parse_nsys.py:18-143).
  void set_trace(bool on) { if (on != trace_) { trace_ = on; tables_dirty_ = true; } }
  bool tracing() const { return trace_; }
  std::vector<TraceStep> read_trace(const RegisteredOp& op);

  uint64_t timeout_ns() const { return timeout_ns_; }
  void set_timeout_ms(uint64_t ms) { timeout_ns_ = ms * 1000000ull; tables_dirty_ = true; }
  // Upper bound of CTAs per launch for programs of this rank (0 = PCCL_NUM_BLOCKS, default 128).
  void set_cta_cap(uint32_t cap) { cta_cap_ = cap; }
  void mark_dirty() { tables_dirty_ = true; }
  bool dirty() const { return tables_dirty_; }
  void clear_dirty() { tables_dirty_ = false; }

  // Arena: bump allocation of symmetric memory for fused operators (same offset on every rank
  // provided every rank allocates in the same order).
  size_t arena_alloc(size_t bytes, size_t align = 1024);
  void arena_reset() { arena_used_ = 0; }
  size_t arena_offset() const { return buffer_bytes_; }

  std::map<std::string, std::unique_ptr<RegisteredOp>>& ops() { return ops_; }

 private:
  int rank_, world_, device_;
  size_t buffer_bytes_, arena_bytes_, arena_used_ = 0;
  SymmetricHeap heap_;
  std::map<std::string, std::unique_ptr<RegisteredOp>> ops_;
  DeviceStatus* d_status_ = nullptr;     // in the control area
  DeviceStatus* h_status_ = nullptr;     // pinned host mirror written by the failing thread
  DeviceStatus* h_status_dev_ = nullptr; // device-visible address of the mirror
  uint64_t timeout_ns_;
  bool tables_dirty_ = false;
  bool trace_ = false;
  uint32_t cta_cap_ = 0;
  friend class Engine;
  friend class LocalCluster;
};

class Engine {
 public:
  static Engine& instance();
  static bool instantiated();

  bool regOp(const std::string& name, const std::string& filename);
  bool regOpFromString(const std::string& name, const std::string& json_text);
  // in/out are device pointers; byte counts are the user tensors' sizes.
  void exeOp(const std::string& name, const void* in, size_t in_bytes, void* out, size_t out_bytes,
             cudaStream_t stream, bool sync);
  void syncOp(const std::string& name, cudaStream_t stream);
  void resetSignals(const std::string& name);
  void reset();
  std::string exportEndpoint();
  bool updateEndpoint(int rank, const std::string& endpoint_json);

  // NVLS bring-up in three host-synchronised stages (the caller barriers between them):
  //   0: rank 0 creates + publishes the multicast object     1: everyone imports + adds its device
  //   2: everyone binds its heap and maps the multicast address.
  // Returns false when NVLS is unavailable or disabled; the caller must make the decision
  // collective (all ranks or none).
  bool nvlsStage(int stage);
  void nvlsDisable();
  bool nvlsActive() { return ctx_->heap().multicast_ready(); }

  RankContext& context() { return *ctx_; }
  int rank() const { return rank_; }
  int world() const { return world_; }
  std::string statsJson();

 private:
  Engine();
  int rank_, world_, device_;
  std::string job_, node_id_;
  std::unique_ptr<RankContext> ctx_;
  FdServer fd_server_;
  bool nvls_wanted_ = false;
};

class LocalCluster {
 public:
  LocalCluster(int world, int device, size_t buffer_bytes);
  ~LocalCluster();
  int world() const { return world_; }
  void regOp(const std::string& name, const std::vector<std::string>& json_per_rank);
  // One cooperative launch runs all ranks.  inputs/outputs are device pointers per rank.
  void exeOp(const std::string& name, const std::vector<const void*>& in, const std::vector<size_t>& in_bytes,
             const std::vector<void*>& out, const std::vector<size_t>& out_bytes, cudaStream_t stream);
  void reset();
  void set_timeout_ms(uint64_t ms);
  void set_ctas(uint32_t ctas) { ctas_override_ = ctas; }
  // regOp runs all ranks' signal protocol abstractly and refuses a plan set that would deadlock;
  // off only for tests of the device-side wait limit, which need such a plan to reach the GPU.
  void set_protocol_check(bool on) { protocol_check_ = on; }
  RankContext& context(int r) { return *ranks_[r]; }
  // Status of the last launch per rank: code 0 = ok.
  std::vector<DeviceStatus> last_status() const { return last_status_; }

 private:
  int world_, device_;
  std::vector<std::unique_ptr<RankContext>> ranks_;
  std::map<std::string, RankProgram*> d_programs_;     // [world] arrays
  std::vector<DeviceStatus> last_status_;
  uint32_t ctas_override_ = 0;
  bool protocol_check_ = true;
};

}  // namespace pccl
