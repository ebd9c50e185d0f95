#include "engine.h"

#include "../common/launch.h"

#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <fstream>
#include <sstream>

namespace pccl {

namespace {

std::string read_file(const std::string& path) {
  std::ifstream in(path, std::ios::binary);
  PCCL_CHECK(in.good(), "cannot open plan file '" << path << "'");
  std::ostringstream ss;
  ss << in.rdbuf();
  return ss.str();
}

std::string boot_id() {
  std::ifstream in("/proc/sys/kernel/random/boot_id");
  std::string id;
  std::getline(in, id);
  return id.empty() ? "unknown-node" : id;
}

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// CTA budget for a program: enough CTAs to saturate NVLink for big steps, few for small ones.
uint32_t auto_ctas(const Plan& plan, uint32_t cap) {
  uint64_t moved = 0;
  for (const PlanOp& op : plan.ops)
    if (op.count > 0) moved = std::max<uint64_t>(moved, static_cast<uint64_t>(op.count) * dtype_bytes(plan.dtype));
  const uint64_t per_channel = std::max<uint64_t>(1, moved / (16 << 10));
  const uint64_t want = per_channel * static_cast<uint64_t>(plan.num_channels);
  return static_cast<uint32_t>(std::min<uint64_t>(std::max<uint64_t>(want, plan.num_channels), cap));
}

const char* status_text(uint32_t code) {
  switch (code) {
    case kSignalTimeout: return "timed out waiting for a signal";
    case kBarrierTimeout: return "timed out in an intra-GPU chain barrier";
    case kDepTimeout: return "timed out waiting for another chain";
    default: return "unknown device status";
  }
}

}  // namespace

// ---- RankContext -------------------------------------------------------------------------------

RankContext::RankContext(int rank, int world, int device, size_t buffer_bytes, size_t arena_bytes,
                         bool shareable)
    : rank_(rank), world_(world), device_(device), buffer_bytes_(round_up(buffer_bytes, 4096)),
      arena_bytes_(round_up(arena_bytes, 4096)) {
  PCCL_CHECK(world >= 1 && world <= kMaxRanks, "world size " << world << " outside 1.." << kMaxRanks);
  PCCL_CHECK(rank >= 0 && rank < world, "rank " << rank << " outside world of " << world);
  timeout_ns_ = static_cast<uint64_t>(Environs::get_int("PCCL_WAIT_TIMEOUT_MS", 10000)) * 1000000ull;
  heap_.set_self(rank);
  heap_.allocate(device, buffer_bytes_ + arena_bytes_, shareable);
  d_status_ = reinterpret_cast<DeviceStatus*>(heap_.control_alloc(sizeof(DeviceStatus)));
  PCCL_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&h_status_), sizeof(DeviceStatus), cudaHostAllocMapped));
  std::memset(h_status_, 0, sizeof(DeviceStatus));
  PCCL_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&h_status_dev_), h_status_, 0));
  trace_ = Environs::get_flag("PCCL_TRACE", false);
  PCCL_CHECK(set_mover_tuning(static_cast<uint32_t>(Environs::get_int("PCCL_MOVER_TUNING", 0))) == 0,
             "cannot set the data-mover tuning word");
}

RankContext::~RankContext() {
  for (auto& kv : ops_) {
    RegisteredOp& op = *kv.second;
    if (op.d_tables) cudaFree(op.d_tables);
    if (op.d_program) cudaFree(op.d_program);
    if (op.chain_sync) cudaFree(op.chain_sync);
    if (op.d_trace) cudaFree(op.d_trace);
  }
  if (h_status_) cudaFreeHost(h_status_);
}

RegisteredOp& RankContext::op(const std::string& name) {
  auto it = ops_.find(name);
  PCCL_CHECK(it != ops_.end(), "operation '" << name << "' is not registered");
  return *it->second;
}

RegisteredOp& RankContext::register_op(const std::string& name, const std::string& json_text) {
  auto fresh = std::make_unique<RegisteredOp>();
  fresh->name = name;
  fresh->plan = load_plan(json_text);
  PlanLimits limits;
  limits.rank = rank_;
  limits.world = world_;
  limits.buffer_elems = static_cast<int64_t>(buffer_bytes_ / dtype_bytes(fresh->plan.dtype));
  validate_plan(fresh->plan, limits);
  auto old = ops_.find(name);
  if (old != ops_.end()) {
    RegisteredOp& o = *old->second;
    if (o.d_tables) cudaFree(o.d_tables);
    if (o.d_program) cudaFree(o.d_program);
    if (o.chain_sync) cudaFree(o.chain_sync);
    if (o.d_trace) cudaFree(o.d_trace);
    ops_.erase(old);
  }
  RegisteredOp& ref = *fresh;
  ops_[name] = std::move(fresh);
  upload(ref);
  return ref;
}

void RankContext::upload(RegisteredOp& op) {
  PCCL_CUDA(cudaSetDevice(device_));
  LowerOptions lo;
  lo.rank = rank_;
  lo.world = world_;
  lo.multicast = heap_.multicast_ready();
  uint32_t cap = cta_cap_ ? cta_cap_ : static_cast<uint32_t>(Environs::get_int("PCCL_NUM_BLOCKS", 128));
  // Never more CTAs than can be resident at once (the interpreter's CTAs wait on one another).
  const int resident = plan_interp_max_ctas(kInterpThreads);
  if (resident > 0) cap = std::min<uint32_t>(cap, static_cast<uint32_t>(resident));
  const int64_t forced = Environs::get_int("PCCL_FORCE_BLOCKS", 0);
  lo.total_ctas = forced > 0 ? std::min<uint32_t>(static_cast<uint32_t>(forced), cap) : auto_ctas(op.plan, cap);
  lo.min_bytes_per_cta = static_cast<uint64_t>(Environs::get_int("PCCL_MIN_BYTES_PER_BLOCK", 16 << 10));
  // Templates of this library end with their own barrier; everything else gets one appended.
  const std::string& algo = op.plan.algorithm;
  const bool self_fenced = algo == "oneshot" || algo == "twoshot" || algo == "direct" || algo == "nvls" || algo == "hybrid";
  lo.defer_barriers = Environs::get_flag("PCCL_DEFER_BARRIERS", true);
  lo.closing_barrier = !self_fenced && !op.plan.collective_type.empty() &&
                       Environs::get_flag("PCCL_CLOSING_BARRIER", true);
  op.lowered = lower_plan(op.plan, lo);
  const LoweredProgram& lp = op.lowered;

  // One device allocation: steps | sigs | deps | chains.
  const size_t steps_b = round_up(lp.steps.size() * sizeof(Step), 128);
  const size_t sigs_b = round_up(lp.sigs.size() * sizeof(SigRef) + 8, 128);
  const size_t deps_b = round_up(lp.deps.size() * sizeof(ChainDep) + 8, 128);
  const size_t chains_b = round_up(lp.chains.size() * sizeof(Chain), 128);
  const size_t total = steps_b + sigs_b + deps_b + chains_b;
  if (op.d_tables == nullptr || op.tables_bytes < total) {
    if (op.d_tables) cudaFree(op.d_tables);
    PCCL_CUDA(cudaMalloc(&op.d_tables, total));
    op.tables_bytes = total;
  }
  std::vector<uint8_t> staging(total, 0);
  std::memcpy(staging.data(), lp.steps.data(), lp.steps.size() * sizeof(Step));
  std::memcpy(staging.data() + steps_b, lp.sigs.data(), lp.sigs.size() * sizeof(SigRef));
  std::memcpy(staging.data() + steps_b + sigs_b, lp.deps.data(), lp.deps.size() * sizeof(ChainDep));
  std::memcpy(staging.data() + steps_b + sigs_b + deps_b, lp.chains.data(), lp.chains.size() * sizeof(Chain));
  PCCL_CUDA(cudaMemcpy(op.d_tables, staging.data(), total, cudaMemcpyHostToDevice));

  // Counters: [chain_sync | chain_progress], zeroed; the launch index restarts with them.
  if (op.chain_sync) cudaFree(op.chain_sync);
  const size_t counters = std::max<size_t>(1, lp.chains.size());
  PCCL_CUDA(cudaMalloc(reinterpret_cast<void**>(&op.chain_sync), 2 * counters * sizeof(uint32_t)));
  PCCL_CUDA(cudaMemset(op.chain_sync, 0, 2 * counters * sizeof(uint32_t)));
  op.chain_progress = op.chain_sync + counters;
  op.launch_index = 0;

  RankProgram& P = op.host_program;
  std::memset(&P, 0, sizeof P);
  P.rank = rank_;
  P.world = world_;
  P.dtype = op.plan.dtype;
  P.num_chains = static_cast<uint32_t>(lp.chains.size());
  for (int r = 0; r < world_; ++r) {
    if (!heap_.has_peer(r)) continue;       // not yet exchanged: upload() runs again later
    P.data[r] = heap_.data(r);
    P.signals[r] = heap_.signals(r);
  }
  P.mc_data = heap_.multicast_ready() ? heap_.mc_base() : nullptr;
  auto* base = static_cast<uint8_t*>(op.d_tables);
  P.steps = reinterpret_cast<const Step*>(base);
  P.sigs = reinterpret_cast<const SigRef*>(base + steps_b);
  P.deps = reinterpret_cast<const ChainDep*>(base + steps_b + sigs_b);
  P.chains = reinterpret_cast<const Chain*>(base + steps_b + sigs_b + deps_b);
  P.chain_sync = op.chain_sync;
  P.chain_progress = op.chain_progress;
  P.status = d_status_;
  P.host_status = h_status_dev_;
  P.timeout_ns = timeout_ns_;
  if (op.d_trace) { cudaFree(op.d_trace); op.d_trace = nullptr; }
  if (trace_ && !lp.steps.empty()) {
    const size_t bytes = lp.steps.size() * kTraceStamps * sizeof(uint64_t);
    PCCL_CUDA(cudaMalloc(reinterpret_cast<void**>(&op.d_trace), bytes));
    PCCL_CUDA(cudaMemset(op.d_trace, 0, bytes));
  }
  P.trace = op.d_trace;
  if (op.d_program == nullptr) PCCL_CUDA(cudaMalloc(reinterpret_cast<void**>(&op.d_program), sizeof(RankProgram)));
  PCCL_CUDA(cudaMemcpy(op.d_program, &P, sizeof P, cudaMemcpyHostToDevice));

  // Copy-engine executor: plans that ask for it (ce.copy operations) or PCCL_EXECUTOR=ce.
  op.ce.reset();
  const bool want_ce = op.plan.has_ce_ops || Environs::get("PCCL_EXECUTOR") == "ce";
  if (want_ce) {
    bool peers_ready = true;
    for (int r = 0; r < world_; ++r) peers_ready &= heap_.has_peer(r);
    if (!CeSchedule::supports(lp)) {
      PCCL_LOG_WARN("operation '" << op.name << "' has cross-chain dependencies; staying on the SM executor");
    } else if (peers_ready) {
      op.ce = std::make_unique<CeSchedule>();
      op.ce->build(lp, P, static_cast<uint64_t>(Environs::get_int("PCCL_CE_MIN_BYTES", 64 << 10)));
    }
  }
  op.stats.copy_engine = op.ce != nullptr;
  op.stats.algorithm = op.plan.algorithm;
  op.stats.collective = op.plan.collective_type;
  op.stats.chains = P.num_chains;
  op.stats.ctas = lp.total_ctas;
  op.stats.steps = static_cast<uint32_t>(lp.steps.size());
  op.stats.multicast = lp.uses_multicast;
}

std::vector<IoSegment> RankContext::input_segments(const RegisteredOp& op, size_t user_bytes) const {
  const size_t esize = dtype_bytes(op.plan.dtype);
  const size_t n = static_cast<size_t>(op.plan.numel) * esize;
  if (op.plan.collective_type == "allgather") {
    const size_t shard = n / world_;
    return {{static_cast<size_t>(rank_) * shard, 0, std::min(user_bytes, shard)}};
  }
  return {{0, 0, user_bytes}};
}

std::vector<IoSegment> RankContext::output_segments(const RegisteredOp& op, size_t user_bytes) const {
  const size_t esize = dtype_bytes(op.plan.dtype);
  const size_t n = static_cast<size_t>(op.plan.numel) * esize;
  const std::string& kind = op.plan.collective_type;
  if (kind == "reduce_scatter") {
    const size_t shard = n / world_;
    return {{static_cast<size_t>(rank_) * shard, 0, std::min(user_bytes, shard)}};
  }
  if (kind == "alltoall") {
    // Own chunk stays in place; chunk p of the result was pulled into scratch at n + p*chunk.
    const size_t chunk = n / world_;
    std::vector<IoSegment> segs;
    for (int p = 0; p < world_; ++p) {
      const size_t from = p == rank_ ? static_cast<size_t>(rank_) * chunk : n + static_cast<size_t>(p) * chunk;
      segs.push_back({from, static_cast<size_t>(p) * chunk, chunk});
    }
    return segs;
  }
  if (kind == "allreduce" || kind == "allgather") return {{0, 0, std::min(user_bytes, n)}};
  return {{0, 0, user_bytes}};
}

void RankContext::stage_in(const RegisteredOp& op, const void* user, size_t bytes, cudaStream_t stream) {
  for (const IoSegment& s : input_segments(op, bytes)) {
    PCCL_CHECK(s.heap_offset + s.bytes <= buffer_bytes_, "input of " << bytes << " bytes does not fit the "
                                                                     << buffer_bytes_ << "-byte working buffer");
    uint8_t* dst = heap_.data(rank_) + s.heap_offset;
    const uint8_t* src = static_cast<const uint8_t*>(user) + s.user_offset;
    if (dst == src || s.bytes == 0) continue;     // the tensor already lives in the working buffer
    PCCL_CUDA(cudaMemcpyAsync(dst, src, s.bytes, cudaMemcpyDeviceToDevice, stream));
  }
}

void RankContext::stage_out(const RegisteredOp& op, void* user, size_t bytes, cudaStream_t stream) {
  for (const IoSegment& s : output_segments(op, bytes)) {
    PCCL_CHECK(s.user_offset + s.bytes <= bytes, "output tensor of " << bytes << " bytes is too small");
    const uint8_t* src = heap_.data(rank_) + s.heap_offset;
    uint8_t* dst = static_cast<uint8_t*>(user) + s.user_offset;
    if (dst == src || s.bytes == 0) continue;
    PCCL_CUDA(cudaMemcpyAsync(dst, src, s.bytes, cudaMemcpyDeviceToDevice, stream));
  }
}

void RankContext::scale_output(RegisteredOp& op, void* user, size_t bytes, cudaStream_t stream) {
  if (!op.plan.uses_avg) return;
  // After stage_out the result lives in `user` (or in place in the heap): scale it there.
  const std::vector<IoSegment> segs = output_segments(op, bytes);
  size_t out_bytes = 0;
  for (const IoSegment& s : segs) out_bytes = std::max(out_bytes, s.user_offset + s.bytes);
  PCCL_CHECK(launch_scale(user, out_bytes, op.plan.dtype, 1.0f / static_cast<float>(world_), stream) == 0,
             "scale kernel launch failed");
}

void RankContext::clear_status() {
  std::memset(h_status_, 0, sizeof(DeviceStatus));
  PCCL_CUDA(cudaMemset(d_status_, 0, sizeof(DeviceStatus)));
}

void RankContext::check_status(const std::string& op_name) {
  if (h_status_->code == kOk) return;
  const DeviceStatus st = *h_status_;
  std::ostringstream msg;
  msg << "operation '" << op_name << "' on rank " << st.rank << ": " << status_text(st.code) << " (chain "
      << st.chain << ", step " << st.step;
  if (st.code == kSignalTimeout) msg << ", signal slot " << st.slot;
  msg << ", observed " << st.observed << ", expected " << st.expected << ") after "
      << timeout_ns_ / 1000000ull << " ms; call reset() on every rank before reusing the engine";
  clear_status();
  throw TimeoutError(msg.str());
}

std::vector<TraceStep> RankContext::read_trace(const RegisteredOp& op) {
  std::vector<TraceStep> out;
  if (op.d_trace == nullptr) return out;
  const LoweredProgram& lp = op.lowered;
  std::vector<uint64_t> raw(lp.steps.size() * kTraceStamps);
  PCCL_CUDA(cudaMemcpy(raw.data(), op.d_trace, raw.size() * sizeof(uint64_t), cudaMemcpyDeviceToHost));
  uint64_t origin = ~0ull;
  for (uint64_t v : raw) if (v != 0 && v < origin) origin = v;
  for (size_t c = 0; c < lp.chains.size(); ++c) {
    const Chain& ch = lp.chains[c];
    for (uint32_t k = 0; k < ch.step_count; ++k) {
      const Step& s = lp.steps[ch.step_begin + k];
      TraceStep t{};
      t.chain = static_cast<uint32_t>(c); t.step = k; t.kind = s.kind; t.ctas = ch.num_ctas; t.bytes = s.bytes;
      for (int i = 0; i < kTraceStamps; ++i) {
        const uint64_t v = raw[(ch.step_begin + k) * kTraceStamps + i];
        t.t[i] = v ? v - origin : 0;
      }
      out.push_back(t);
    }
  }
  return out;
}

void RankContext::reset_op_counters(RegisteredOp& op) {
  const size_t counters = std::max<size_t>(1, op.lowered.chains.size());
  PCCL_CUDA(cudaMemset(op.chain_sync, 0, 2 * counters * sizeof(uint32_t)));
  if (op.ce) op.ce->reset_counters();
  op.launch_index = 0;
}

void RankContext::reset() {
  PCCL_CUDA(cudaSetDevice(device_));
  PCCL_CUDA(cudaDeviceSynchronize());
  PCCL_CUDA(cudaMemset(heap_.signals(rank_), 0, static_cast<size_t>(kSignalSlots) * sizeof(uint32_t)));
  for (auto& kv : ops_) reset_op_counters(*kv.second);
  clear_status();
}

size_t RankContext::arena_alloc(size_t bytes, size_t align) {
  const size_t at = round_up(arena_used_, align);
  PCCL_CHECK(at + bytes <= arena_bytes_, "symmetric arena exhausted: " << at + bytes << " > " << arena_bytes_
                                                                        << " bytes (raise PCCL_ARENA_SIZE)");
  arena_used_ = at + bytes;
  return buffer_bytes_ + at;
}

// ---- Engine -----------------------------------------------------------------------------------------

namespace { bool g_engine_built = false; }

bool Engine::instantiated() { return g_engine_built; }

Engine& Engine::instance() {
  static Engine engine;
  return engine;
}

Engine::Engine() {
  Environs::register_option("RANK", "rank of this process (required)");
  Environs::register_option("WORLD_SIZE", "number of ranks (default 1)");
  Environs::register_option("PCCL_BUFFER_SIZE", "bytes of the plan working buffer (default 1G)");
  Environs::register_option("PCCL_ARENA_SIZE", "bytes of symmetric memory for fused operators (default 1G)");
  Environs::register_option("PCCL_NUM_BLOCKS", "upper bound of CTAs per launch (default 128, never more than can be resident at once)");
  Environs::register_option("PCCL_FORCE_BLOCKS", "exact CTA count per launch (overrides the heuristic)");
  Environs::register_option("PCCL_WAIT_TIMEOUT_MS", "budget of device-side waits per launch (default 10000)");
  Environs::register_option("PCCL_NVLS_ENABLE", "0 disables NVLS multicast (default: on when supported)");
  Environs::register_option("PCCL_DISABLE_NVLS", "1 disables NVLS multicast");
  Environs::register_option("PCCL_LOG_LEVEL", "TRACE|DEBUG|INFO|WARN|ERROR|CRITICAL (default WARN)");
  Environs::register_option("PCCL_JOB_ID", "namespace of the fd-passing sockets (default MASTER_ADDR:MASTER_PORT)");

  rank_ = static_cast<int>(std::stol(Environs::require("RANK")));
  world_ = static_cast<int>(Environs::get_int("WORLD_SIZE", 1));
  PCCL_CUDA(cudaGetDevice(&device_));
  job_ = FdServer::default_job_id();
  node_id_ = boot_id();
  size_t buffer = static_cast<size_t>(Environs::get_int("PCCL_BUFFER_SIZE", 1ll << 30));
  buffer = std::max<size_t>(buffer, 1 << 20);
  const size_t arena = static_cast<size_t>(Environs::get_int("PCCL_ARENA_SIZE", 1ll << 30));
  ctx_ = std::make_unique<RankContext>(rank_, world_, device_, buffer, arena, /*shareable=*/true);
  if (world_ > 1) {
    fd_server_.start(job_, rank_);
    const int fd = ctx_->heap().export_fd();
    fd_server_.publish("heap", fd);
    close(fd);
  }
  nvls_wanted_ = world_ > 1 && Environs::get_flag("PCCL_NVLS_ENABLE", true) &&
                 !Environs::get_flag("PCCL_DISABLE_NVLS", false) &&
                 SymmetricHeap::multicast_supported(device_);
  g_engine_built = true;
  PCCL_LOG_INFO("engine up: rank " << rank_ << "/" << world_ << " device " << device_ << " buffer "
                                   << buffer << " arena " << arena << " nvls_wanted " << nvls_wanted_);
}

bool Engine::regOp(const std::string& name, const std::string& filename) {
  try {
    return regOpFromString(name, read_file(filename));
  } catch (const Error& e) {
    PCCL_LOG_WARN("regOp('" << name << "', '" << filename << "') failed: " << e.what());
    return false;
  }
}

bool Engine::regOpFromString(const std::string& name, const std::string& json_text) {
  try {
    NvtxRange range("regOp");
    ctx_->register_op(name, json_text);
    return true;
  } catch (const std::exception& e) {
    PCCL_LOG_WARN("registering '" << name << "' failed: " << e.what());
    return false;
  }
}

void Engine::exeOp(const std::string& name, const void* in, size_t in_bytes, void* out, size_t out_bytes,
                   cudaStream_t stream, bool sync) {
  RegisteredOp& op = ctx_->op(name);
  if (ctx_->dirty()) {
    for (auto& kv : ctx_->ops()) ctx_->upload(*kv.second);
    ctx_->clear_dirty();
  }
  for (int r = 0; r < world_; ++r)
    PCCL_CHECK(ctx_->heap().has_peer(r), "rank " << r << " has not been connected; call initialize_engine first");
  {
    NvtxRange range("d2d_input_copy");
    ctx_->stage_in(op, in, in_bytes, stream);
  }
  {
    NvtxRange range("execute");
    if (op.ce) {
      op.ce->run(op.host_program.data, rank_, op.launch_index, stream);
    } else {
      LaunchParams lp{op.d_program, op.launch_index};
      // Chains use multi-CTA barriers and lead-CTA waits on peers: every CTA must be resident, also
      // next to a compute kernel that holds part of the GPU, hence a cooperative launch.
      // (A plan with more chains than resident CTAs cannot be launched that way; it keeps the
      // ordinary launch and needs the GPU to itself.)
      const uint32_t grid = std::max<uint32_t>(1, op.lowered.total_ctas);
      const bool coop = cooperative_launches() && static_cast<int>(grid) <= plan_interp_max_ctas(op.threads);
      LaunchConfig cfg{grid, op.threads, 1, coop, op.host_program.dtype};
      const int err = launch_plan_interp(lp, cfg, stream);
      PCCL_CHECK(err == 0, "kernel launch failed: " << cudaGetErrorString(static_cast<cudaError_t>(err)));
    }
    ++op.launch_index;
  }
  {
    NvtxRange range("d2d_output_copy");
    ctx_->stage_out(op, out, out_bytes, stream);
    ctx_->scale_output(op, out, out_bytes, stream);
  }
  op.stats.calls += 1;
  op.stats.bytes += in_bytes;
  if (sync) syncOp(name, stream);
}

void Engine::syncOp(const std::string& name, cudaStream_t stream) {
  PCCL_CUDA(cudaStreamSynchronize(stream));
  ctx_->check_status(name);
}

void Engine::resetSignals(const std::string& name) {
  PCCL_CUDA(cudaDeviceSynchronize());
  PCCL_CUDA(cudaMemset(ctx_->heap().signals(rank_), 0, static_cast<size_t>(kSignalSlots) * sizeof(uint32_t)));
  if (ctx_->has_op(name)) ctx_->reset_op_counters(ctx_->op(name));
  ctx_->clear_status();
}

void Engine::reset() { ctx_->reset(); }

std::string Engine::exportEndpoint() {
  json::Value ep = json::Value::object();
  ep.set("version", 1);
  ep.set("rank", rank_);
  ep.set("world", world_);
  ep.set("node_id", node_id_);
  ep.set("job", job_);
  ep.set("pid", static_cast<int64_t>(getpid()));
  ep.set("device", device_);
  ep.set("buffer_bytes", static_cast<uint64_t>(ctx_->buffer_bytes()));
  ep.set("heap_bytes", static_cast<uint64_t>(ctx_->heap().layout().total_bytes));
  ep.set("heap_entry", "heap");
  ep.set("multicast_supported", SymmetricHeap::multicast_supported(device_));
  return ep.dump();
}

bool Engine::updateEndpoint(int rank, const std::string& endpoint_json) {
  try {
    if (rank == rank_) return true;
    const json::Value ep = json::parse(endpoint_json);
    PCCL_CHECK(ep.get_string("node_id", "") == node_id_,
               "rank " << rank << " runs on another node; only single-node peers are mapped");
    PCCL_CHECK(static_cast<size_t>(ep.get_int("heap_bytes", 0)) == ctx_->heap().layout().total_bytes,
               "rank " << rank << " uses a different heap size (PCCL_BUFFER_SIZE / PCCL_ARENA_SIZE must match)");
    if (ctx_->heap().has_peer(rank)) return true;
    const int fd = FdServer::fetch(ep.get_string("job", job_), rank, ep.get_string("heap_entry", "heap"));
    PCCL_CHECK(fd >= 0, "could not obtain rank " << rank << "'s heap descriptor");
    ctx_->heap().map_peer(rank, fd);
    ctx_->mark_dirty();
    return true;
  } catch (const std::exception& e) {
    PCCL_LOG_ERROR("updateEndpoint(" << rank << ") failed: " << e.what());
    return false;
  }
}

bool Engine::nvlsStage(int stage) {
  if (!nvls_wanted_) return false;
  try {
    SymmetricHeap& heap = ctx_->heap();
    if (stage == 0) {
      if (rank_ == 0) {
        const int fd = heap.multicast_create(world_);
        fd_server_.publish("nvls_mc", fd);
        close(fd);
      }
    } else if (stage == 1) {
      if (rank_ != 0) {
        const int fd = FdServer::fetch(job_, 0, "nvls_mc");
        PCCL_CHECK(fd >= 0, "could not obtain the multicast descriptor from rank 0");
        heap.multicast_import(fd);
      }
      heap.multicast_add_device();
    } else {
      heap.multicast_bind_and_map();
      ctx_->mark_dirty();
    }
    return true;
  } catch (const std::exception& e) {
    PCCL_LOG_WARN("NVLS stage " << stage << " failed, falling back to peer loads: " << e.what());
    return false;
  }
}

void Engine::nvlsDisable() {
  nvls_wanted_ = false;
  ctx_->heap().multicast_release();
  ctx_->mark_dirty();
}

std::string Engine::statsJson() {
  json::Value all = json::Value::object();
  for (auto& kv : ctx_->ops()) {
    const OpStats& s = kv.second->stats;
    json::Value o = json::Value::object();
    o.set("calls", s.calls);
    o.set("bytes", s.bytes);
    o.set("algorithm", s.algorithm);
    o.set("collective", s.collective);
    o.set("chains", static_cast<int64_t>(s.chains));
    o.set("ctas", static_cast<int64_t>(s.ctas));
    o.set("steps", static_cast<int64_t>(s.steps));
    o.set("multicast", s.multicast);
    o.set("copy_engine", s.copy_engine);
    all.set(kv.first, o);
  }
  return all.dump();
}

// ---- LocalCluster --------------------------------------------------------------------------------------

LocalCluster::LocalCluster(int world, int device, size_t buffer_bytes) : world_(world), device_(device) {
  PCCL_CHECK(world >= 1 && world <= kMaxVirtualRanks, "cluster size " << world << " outside 1.." << kMaxVirtualRanks);
  for (int r = 0; r < world; ++r)
    ranks_.push_back(std::make_unique<RankContext>(r, world, device, buffer_bytes, 4096, /*shareable=*/false));
  for (int r = 0; r < world; ++r)
    for (int p = 0; p < world; ++p)
      if (p != r) ranks_[r]->heap().alias_peer(p, ranks_[p]->heap());
  last_status_.resize(world);
}

LocalCluster::~LocalCluster() {
  for (auto& kv : d_programs_) cudaFree(kv.second);
}

void LocalCluster::regOp(const std::string& name, const std::vector<std::string>& json_per_rank) {
  PCCL_CHECK(static_cast<int>(json_per_rank.size()) == world_, "need one plan per rank");
  if (protocol_check_) {
    // All ranks' plans are at hand: run their signal protocol abstractly before anything launches.
    std::vector<Plan> all;
    for (const std::string& text : json_per_rank) all.push_back(load_plan(text));
    const WorldReport rep = check_world(all);
    PCCL_CHECK(!rep.deadlock, "operation '" << name << "' would deadlock: " << rep.detail);
    if (rep.leftover_signals)
      PCCL_LOG_WARN("operation '" << name << "' leaves " << rep.leftover_signals
                                  << " signals non-zero (reset_signals needed between runs): " << rep.detail);
  }
  // All virtual ranks must be co-resident in one cooperative launch.
  const int resident = plan_interp_max_ctas(kInterpThreads);
  PCCL_CHECK(resident > 0, "no CUDA device");
  const uint32_t per_rank = std::max<uint32_t>(1, ctas_override_ ? std::min<uint32_t>(ctas_override_, resident / world_)
                                                                 : static_cast<uint32_t>(resident / world_));
  for (int r = 0; r < world_; ++r) {
    RankContext& ctx = *ranks_[r];
    ctx.set_cta_cap(per_rank);
    RegisteredOp& op = ctx.register_op(name, json_per_rank[r]);
    PCCL_CHECK(op.lowered.total_ctas <= per_rank,
               "plan needs " << op.lowered.total_ctas << " CTAs per rank (at least one per chain) but only "
                             << per_rank << " fit next to the other virtual ranks");
  }
  RankProgram* d = nullptr;
  auto it = d_programs_.find(name);
  if (it != d_programs_.end()) d = it->second;
  else PCCL_CUDA(cudaMalloc(reinterpret_cast<void**>(&d), sizeof(RankProgram) * world_));
  std::vector<RankProgram> host(world_);
  for (int r = 0; r < world_; ++r) host[r] = ranks_[r]->op(name).host_program;
  PCCL_CUDA(cudaMemcpy(d, host.data(), sizeof(RankProgram) * world_, cudaMemcpyHostToDevice));
  d_programs_[name] = d;
}

void LocalCluster::exeOp(const std::string& name, const std::vector<const void*>& in,
                         const std::vector<size_t>& in_bytes, const std::vector<void*>& out,
                         const std::vector<size_t>& out_bytes, cudaStream_t stream) {
  PCCL_CHECK(static_cast<int>(in.size()) == world_ && static_cast<int>(out.size()) == world_,
             "need one input and one output per rank");
  uint32_t ctas = 1, launch_index = 0;
  for (int r = 0; r < world_; ++r) {
    RegisteredOp& op = ranks_[r]->op(name);
    ranks_[r]->stage_in(op, in[r], in_bytes[r], stream);
    ctas = std::max(ctas, op.lowered.total_ctas);
    launch_index = op.launch_index;
  }
  LaunchParams lp{d_programs_.at(name), launch_index};
  LaunchConfig cfg{ctas, kInterpThreads, static_cast<uint32_t>(world_), true,
                   ranks_[0]->op(name).host_program.dtype};
  const int err = launch_plan_interp(lp, cfg, stream);
  PCCL_CHECK(err == 0, "cooperative launch failed: " << cudaGetErrorString(static_cast<cudaError_t>(err)));
  for (int r = 0; r < world_; ++r) {
    RegisteredOp& op = ranks_[r]->op(name);
    ++op.launch_index;
    ranks_[r]->stage_out(op, out[r], out_bytes[r], stream);
    ranks_[r]->scale_output(op, out[r], out_bytes[r], stream);
  }
  PCCL_CUDA(cudaStreamSynchronize(stream));
  bool failed = false;
  for (int r = 0; r < world_; ++r) {
    last_status_[r] = *ranks_[r]->host_status();
    failed |= last_status_[r].code != kOk;
  }
  if (failed) {
    for (int r = 0; r < world_; ++r)
      if (last_status_[r].code != kOk) ranks_[r]->check_status(name);   // throws TimeoutError
  }
}

void LocalCluster::reset() {
  for (auto& r : ranks_) r->reset();
}

void LocalCluster::set_timeout_ms(uint64_t ms) {
  for (auto& r : ranks_) {
    r->set_timeout_ms(ms);
    for (auto& kv : r->ops()) r->upload(*kv.second);
    r->clear_dirty();
  }
  for (auto& kv : d_programs_) {
    std::vector<RankProgram> host(world_);
    for (int r = 0; r < world_; ++r) host[r] = ranks_[r]->op(kv.first).host_program;
    PCCL_CUDA(cudaMemcpy(kv.second, host.data(), sizeof(RankProgram) * world_, cudaMemcpyHostToDevice));
  }
}

}  // namespace pccl
