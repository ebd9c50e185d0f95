#include "plan.h"

#include <algorithm>
#include <map>
#include <set>
#include <sstream>

#include "../common/util.h"

namespace pccl {

namespace {

uint8_t parse_dtype(const std::string& name) {
  if (name == "float32" || name == "torch.float32") return kF32;
  if (name == "float16" || name == "torch.float16") return kF16;
  if (name == "bfloat16" || name == "torch.bfloat16") return kBF16;
  if (name == "float8_e4m3" || name == "torch.float8_e4m3fn") return kE4M3;
  if (name == "float8_e5m2" || name == "torch.float8_e5m2") return kE5M2;
  throw Error("plan: unsupported dtype '" + name + "'");
}

Primitive parse_primitive(const std::string& name) {
  static const std::map<std::string, Primitive> table = {
      {"noop", Primitive::kNoop},
      {"notify", Primitive::kNotify}, {"sm.notify", Primitive::kNotify},
      {"wait_notify", Primitive::kWait}, {"sm.wait_notify", Primitive::kWait},
      {"sm.copy", Primitive::kCopy}, {"tma.copy", Primitive::kCopy}, {"rdma.read", Primitive::kCopy},
      {"ce.copy", Primitive::kCeCopy},
      {"sm.reduce", Primitive::kReduce}, {"tma.reduce", Primitive::kReduce},
      {"sm.put", Primitive::kPut}, {"rdma.write", Primitive::kPut},
      {"sm.reduce_multi", Primitive::kReduceMulti},
      {"multimem.reduce", Primitive::kMmReduce}, {"multimem.store", Primitive::kMmStore},
      {"multimem.allreduce", Primitive::kMmAllreduce},
  };
  auto it = table.find(name);
  if (it == table.end()) throw Error("plan: unknown primitive '" + name + "'");
  return it->second;
}

bool known_executor(const std::string& e) {
  static const std::set<std::string> names = {"cuda_sm", "cuda_tma", "cuda_ce", "cuda_multimem",
                                              "cuda_rdma", "host"};
  return names.count(e) != 0;
}

bool is_data(Primitive p) {
  return p != Primitive::kNoop && p != Primitive::kNotify && p != Primitive::kWait;
}

}  // namespace

const char* primitive_label(Primitive p) {
  switch (p) {
    case Primitive::kNoop: return "noop";
    case Primitive::kNotify: return "notify";
    case Primitive::kWait: return "wait_notify";
    case Primitive::kCopy: return "copy";
    case Primitive::kReduce: return "reduce";
    case Primitive::kPut: return "put";
    case Primitive::kReduceMulti: return "reduce_multi";
    case Primitive::kMmReduce: return "multimem.reduce";
    case Primitive::kMmStore: return "multimem.store";
    case Primitive::kMmAllreduce: return "multimem.allreduce";
    case Primitive::kCeCopy: return "ce.copy";
  }
  return "?";
}

Plan load_plan(const std::string& text) {
  const json::Value doc = json::parse(text);
  PCCL_CHECK(doc.is_object(), "plan: top level must be an object");
  Plan plan;
  plan.version = static_cast<int>(doc.get_int("version", 2));
  // A phased (version 3) manifest has no top-level operations: the host must
  // split it into phases first.
  PCCL_CHECK(doc.contains("operations"), "plan: no top-level 'operations' (a phased OCS manifest must be "
                                         "split into per-phase plans before registration)");
  if (const json::Value* info = doc.find("tensor_info")) {
    plan.dtype_name = info->get_string("dtype", "float32");
    plan.dtype = parse_dtype(plan.dtype_name);
    plan.numel = 1;
    if (const json::Value* shape = info->find("shape"))
      for (const auto& extent : shape->items()) plan.numel *= extent.as_int();
  } else {
    plan.dtype_name = "float32";
  }
  plan.collective_type = doc.get_string("collective_type", "");
  plan.algorithm = doc.get_string("algorithm", "");

  const auto& ops = doc.at("operations").items();
  plan.ops.reserve(ops.size());
  int max_channel = 0;
  for (size_t i = 0; i < ops.size(); ++i) {
    const json::Value& o = ops[i];
    PlanOp op;
    PCCL_CHECK(o.contains("index") && o.contains("executor") && o.contains("primitive"),
               "plan: operation " << i << " needs index, executor and primitive");
    op.index = static_cast<int>(o.at("index").as_int());
    PCCL_CHECK(op.index == static_cast<int>(i), "plan: operation indices must be 0..n-1 in order");
    op.executor = o.at("executor").as_string();
    PCCL_CHECK(known_executor(op.executor), "plan: unknown executor '" << op.executor << "'");
    op.primitive_name = o.at("primitive").as_string();
    op.primitive = parse_primitive(op.primitive_name);
    op.channel = static_cast<int>(o.get_int("channel", 0));
    PCCL_CHECK(op.channel >= 0 && op.channel < 4096, "plan: channel " << op.channel << " out of range");
    max_channel = std::max(max_channel, op.channel);
    if (const json::Value* d = o.find("dependencies"))
      for (const auto& v : d->items()) op.deps.push_back(static_cast<int>(v.as_int()));
    if (const json::Value* n = o.find("next_ops"))
      for (const auto& v : n->items()) op.next.push_back(static_cast<int>(v.as_int()));
    for (int d : op.deps)
      PCCL_CHECK(d >= 0 && d < op.index, "plan: operation " << i << " depends on " << d
                                                             << ", which is not an earlier operation");
    static const json::Value kEmpty = json::Value::object();
    const json::Value* pp = o.find("params");
    const json::Value& p = pp ? *pp : kEmpty;
    const std::string red = p.get_string("reduce_op", "sum");
    if (red == "sum") op.red_op = kRedSum;
    else if (red == "avg") { op.red_op = kRedSum; op.avg = true; }
    else if (red == "max") op.red_op = kRedMax;
    else if (red == "min") op.red_op = kRedMin;
    else throw Error("plan: unknown reduce_op '" + red + "'");
    switch (op.primitive) {
      case Primitive::kNotify:
        op.signal_id = static_cast<uint32_t>(p.get_int("signal_id", 0));
        op.peer = static_cast<int>(p.get_int("target_rank", -1));
        break;
      case Primitive::kWait:
        op.signal_id = static_cast<uint32_t>(p.get_int("signal_id", 0));
        op.peer = static_cast<int>(p.get_int("source_rank", -1));
        break;
      case Primitive::kCopy:
      case Primitive::kCeCopy:
      case Primitive::kMmStore:
        op.peer = static_cast<int>(p.get_int("source_rank", -1));
        op.off_src = p.get_int("src_offset", 0);
        op.off_dst = p.get_int("dst_offset", 0);
        op.count = p.get_int("size", 0);
        break;
      case Primitive::kPut:
        op.peer = static_cast<int>(p.get_int("target_rank", -1));
        op.off_src = p.get_int("src_offset", 0);
        op.off_dst = p.get_int("dst_offset", 0);
        op.count = p.get_int("size", 0);
        break;
      case Primitive::kReduce:
      case Primitive::kMmReduce:
        op.peer = static_cast<int>(p.get_int("source_rank", -1));
        op.off_src = p.get_int("src_offset", 0);
        op.off_dst = p.get_int("dst_offset", 0);
        op.off_remote = p.get_int("remote_offset", 0);
        op.count = p.get_int("count", 0);
        break;
      case Primitive::kReduceMulti:
        if (const json::Value* s = p.find("source_ranks"))
          for (const auto& v : s->items()) op.sources.push_back(static_cast<int>(v.as_int()));
        op.off_dst = p.get_int("dst_offset", 0);
        op.off_remote = p.get_int("remote_offset", 0);
        op.count = p.get_int("count", 0);
        break;
      case Primitive::kMmAllreduce:
        op.off_remote = p.get_int("offset", 0);
        op.count = p.get_int("count", 0);
        break;
      case Primitive::kNoop:
        break;
    }
    plan.uses_avg |= op.avg;
    plan.has_ce_ops |= op.primitive == Primitive::kCeCopy;
    plan.ops.push_back(std::move(op));
  }
  plan.num_channels = max_channel + 1;
  return plan;
}

void validate_plan(const Plan& plan, const PlanLimits& lim) {
  auto fail = [&](const PlanOp& op, const std::string& what) {
    throw Error("plan: operation " + std::to_string(op.index) + " (" + op.primitive_name + "): " + what);
  };
  auto check_rank = [&](const PlanOp& op, int r, const char* what) {
    if (r < 0 || r >= lim.world)
      fail(op, std::string(what) + " " + std::to_string(r) + " is outside the world of " + std::to_string(lim.world));
  };
  auto check_range = [&](const PlanOp& op, int64_t off, const char* what) {
    if (off < 0 || op.count < 0 || off + op.count > lim.buffer_elems)
      fail(op, std::string(what) + " range [" + std::to_string(off) + ", " + std::to_string(off + op.count) +
                   ") exceeds the " + std::to_string(lim.buffer_elems) + "-element buffer");
  };
  for (const PlanOp& op : plan.ops) {
    switch (op.primitive) {
      case Primitive::kNotify:
      case Primitive::kWait:
        check_rank(op, op.peer, op.primitive == Primitive::kNotify ? "target_rank" : "source_rank");
        if (op.signal_id >= kSignalSlots - kMaxRanks)
          fail(op, "signal_id " + std::to_string(op.signal_id) + " exceeds the " +
                       std::to_string(kSignalSlots - kMaxRanks) + " usable signal slots");
        break;
      case Primitive::kCopy: case Primitive::kCeCopy: case Primitive::kPut: case Primitive::kMmStore:
        check_rank(op, op.peer, "peer rank");
        check_range(op, op.off_src, "source");
        check_range(op, op.off_dst, "destination");
        break;
      case Primitive::kReduce: case Primitive::kMmReduce:
        check_rank(op, op.peer, "source_rank");
        check_range(op, op.off_src, "local source");
        check_range(op, op.off_dst, "destination");
        check_range(op, op.off_remote, "remote source");
        break;
      case Primitive::kReduceMulti:
        if (op.sources.empty()) fail(op, "source_ranks is empty");
        for (int r : op.sources) check_rank(op, r, "source rank");
        check_range(op, op.off_dst, "destination");
        check_range(op, op.off_remote, "remote source");
        break;
      case Primitive::kMmAllreduce:
        check_range(op, op.off_remote, "range");
        break;
      case Primitive::kNoop:
        break;
    }
  }
}

WorldReport check_world(const std::vector<Plan>& plans) {
  WorldReport rep;
  const int world = static_cast<int>(plans.size());
  struct RankState {
    std::vector<int> missing;       // unmet dependencies per operation
    std::vector<char> done;
    std::vector<int> ready;
    std::map<uint32_t, int64_t> signals;
    size_t finished = 0;
  };
  std::vector<RankState> st(world);
  for (int r = 0; r < world; ++r) {
    const Plan& plan = plans[r];
    st[r].missing.resize(plan.ops.size());
    st[r].done.assign(plan.ops.size(), 0);
    const int esize = dtype_bytes(plan.dtype);
    for (size_t i = 0; i < plan.ops.size(); ++i) {
      const PlanOp& op = plan.ops[i];
      st[r].missing[i] = static_cast<int>(op.deps.size());
      if (op.deps.empty()) st[r].ready.push_back(static_cast<int>(i));
      if (op.primitive == Primitive::kNotify) ++rep.notifies;
      if (op.primitive == Primitive::kWait) ++rep.waits;
      if (is_data(op.primitive)) {
        const int64_t fields[4] = {op.off_src, op.off_dst, op.off_remote, op.count};
        for (int64_t f : fields)
          if ((f * esize) % 16 != 0) { ++rep.misaligned_ops; break; }
      }
    }
  }
  // Successor lists from the dependency lists (next_ops in the file may be truncated or absent).
  std::vector<std::vector<std::vector<int>>> succ(world);
  for (int r = 0; r < world; ++r) {
    succ[r].resize(plans[r].ops.size());
    for (const PlanOp& op : plans[r].ops)
      for (int d : op.deps) succ[r][d].push_back(op.index);
  }
  bool progressed = true;
  while (progressed) {
    progressed = false;
    for (int r = 0; r < world; ++r) {
      RankState& s = st[r];
      for (size_t k = 0; k < s.ready.size();) {
        const int i = s.ready[k];
        const PlanOp& op = plans[r].ops[i];
        if (op.primitive == Primitive::kWait) {
          auto it = s.signals.find(op.signal_id);
          if (it == s.signals.end() || it->second <= 0) { ++k; continue; }
          --it->second;
        } else if (op.primitive == Primitive::kNotify) {
          if (op.peer >= 0 && op.peer < world) ++st[op.peer].signals[op.signal_id];
        }
        s.done[i] = 1;
        ++s.finished;
        s.ready.erase(s.ready.begin() + static_cast<long>(k));
        for (int n : succ[r][i])
          if (--s.missing[n] == 0) s.ready.push_back(n);
        progressed = true;
      }
    }
  }
  std::ostringstream detail;
  for (int r = 0; r < world; ++r) {
    if (st[r].finished == plans[r].ops.size()) continue;
    rep.deadlock = true;
    detail << "rank " << r << " blocked at";
    int shown = 0;
    for (int i : st[r].ready) {
      const PlanOp& op = plans[r].ops[i];
      detail << " op " << i << " (" << op.primitive_name;
      if (op.primitive == Primitive::kWait) detail << " signal " << op.signal_id << " from rank " << op.peer;
      detail << ")";
      if (++shown == 4) break;
    }
    detail << "; ";
  }
  for (int r = 0; r < world; ++r)
    for (const auto& kv : st[r].signals)
      if (kv.second != 0) {
        if (rep.leftover_signals < 4 && !rep.deadlock)
          detail << "rank " << r << " signal " << kv.first << " left at " << kv.second << "; ";
        ++rep.leftover_signals;
      }
  rep.detail = detail.str();
  return rep;
}

// ---- lowering ---------------------------------------------------------------------------------

namespace {

struct ChainBuilder {
  int channel = 0;
  std::vector<int> ops;            // plan op indices in order
};

uint64_t bytes_of(const Plan& plan, int64_t elems) { return static_cast<uint64_t>(elems) * dtype_bytes(plan.dtype); }

bool mm_dtype_ok(uint8_t dtype, uint8_t red_op) {
  if (dtype == kF32) return red_op == kRedSum;
  return dtype == kF16 || dtype == kBF16;
}

}  // namespace

LoweredProgram lower_plan(const Plan& plan, const LowerOptions& opt) {
  LoweredProgram out;
  const size_t n = plan.ops.size();
  const int esize = dtype_bytes(plan.dtype);

  // 1. Chain decomposition: an operation extends the chain of a dependency when
  //    that dependency is still the chain's tail and shares its channel.
  std::vector<ChainBuilder> chains;
  std::vector<int> chain_of(n, -1), pos_in_chain(n, -1);
  std::vector<int> tail_of_chain;
  for (size_t i = 0; i < n; ++i) {
    const PlanOp& op = plan.ops[i];
    int chosen = -1;
    for (int d : op.deps) {
      const int c = chain_of[d];
      if (tail_of_chain[c] == d && chains[c].channel == op.channel) { chosen = c; break; }
    }
    if (chosen < 0) {
      chains.push_back(ChainBuilder{op.channel, {}});
      tail_of_chain.push_back(-1);
      chosen = static_cast<int>(chains.size()) - 1;
    }
    chain_of[i] = chosen;
    pos_in_chain[i] = static_cast<int>(chains[chosen].ops.size());
    chains[chosen].ops.push_back(static_cast<int>(i));
    tail_of_chain[chosen] = static_cast<int>(i);
  }

  // 2. Fold each chain's operations into steps: waits*, one data op, notifies*.
  //    step_of_op lets cross-chain dependencies refer to finished *steps*.
  std::vector<int> step_of_op(n, -1);          // step index within its chain
  struct PendingStep {
    std::vector<SigRef> waits, notifies;
    std::vector<std::pair<int, int>> deps;     // (plan op index depended on) resolved later
    std::vector<int> dep_ops;
    Step step{};
    bool has_data = false;
  };
  std::vector<std::vector<PendingStep>> chain_steps(chains.size());

  auto new_step = [&](int c) -> PendingStep& {
    chain_steps[c].emplace_back();
    PendingStep& s = chain_steps[c].back();
    s.step.kind = kStepNoop;
    s.step.scale = 1.0f;
    s.step.peer = -1;
    return s;
  };

  auto fill_data = [&](PendingStep& ps, const PlanOp& op, Primitive prim) {
    Step& s = ps.step;
    ps.has_data = true;
    s.red_op = op.red_op;
    s.bytes = bytes_of(plan, op.count);
    switch (prim) {
      case Primitive::kCopy: case Primitive::kCeCopy:
        s.kind = kStepCopy; s.peer = op.peer;
        s.off0 = bytes_of(plan, op.off_src); s.off1 = bytes_of(plan, op.off_dst);
        break;
      case Primitive::kPut:
        s.kind = kStepPut; s.peer = op.peer; s.writes_remote = op.peer != opt.rank;
        s.off0 = bytes_of(plan, op.off_src); s.off1 = bytes_of(plan, op.off_dst);
        break;
      case Primitive::kReduce:
        s.kind = kStepReduce; s.peer = op.peer;
        s.off0 = bytes_of(plan, op.off_remote); s.off1 = bytes_of(plan, op.off_src);
        s.off2 = bytes_of(plan, op.off_dst);
        break;
      case Primitive::kReduceMulti:
        s.kind = kStepReduceMulti;
        for (int r : op.sources) s.peer_mask |= 1u << r;
        s.off0 = bytes_of(plan, op.off_remote); s.off2 = bytes_of(plan, op.off_dst);
        break;
      case Primitive::kMmReduce:
        s.kind = kStepMmReduce;
        s.off0 = bytes_of(plan, op.off_remote); s.off2 = bytes_of(plan, op.off_dst);
        break;
      case Primitive::kMmStore:
        s.kind = kStepMmStore; s.writes_remote = 1;
        s.off0 = bytes_of(plan, op.off_src); s.off1 = bytes_of(plan, op.off_dst);
        break;
      case Primitive::kMmAllreduce:
        s.kind = kStepMmAllreduce; s.writes_remote = 1;
        s.off0 = bytes_of(plan, op.off_remote);
        break;
      default: break;
    }
  };

  const uint32_t all_ranks_mask = opt.world >= 32 ? 0xffffffffu : ((1u << opt.world) - 1u);

  for (size_t c = 0; c < chains.size(); ++c) {
    enum { kFresh, kWaiting, kHasData, kNotifying } state = kFresh;
    PendingStep* cur = nullptr;
    for (int oi : chains[c].ops) {
      const PlanOp& op = plan.ops[oi];
      // Dependencies on operations of *other* chains (or non-adjacent ones) become chain deps.
      std::vector<int> cross;
      for (int d : op.deps)
        if (chain_of[d] != static_cast<int>(c)) cross.push_back(d);
      const bool data = is_data(op.primitive);
      // A step is [waits][one data op][notifies].  Dependencies on other chains may only sit
      // at the very start of a step: attaching them later could make this step wait for a
      // chain that itself waits for an earlier part of this step.
      bool start_new = cur == nullptr;
      if (!start_new) {
        if (!cross.empty() && state != kFresh) start_new = true;
        else if (op.primitive == Primitive::kWait && (state == kHasData || state == kNotifying)) start_new = true;
        else if (data && (state == kHasData || state == kNotifying)) start_new = true;
      }
      if (start_new) { cur = &new_step(static_cast<int>(c)); state = kFresh; }
      for (int d : cross) cur->dep_ops.push_back(d);

      if (op.primitive == Primitive::kWait) {
        cur->waits.push_back(SigRef{op.peer, op.signal_id});
        state = kWaiting;
      } else if (op.primitive == Primitive::kNotify) {
        cur->notifies.push_back(SigRef{op.peer, op.signal_id});
        state = kNotifying;
      } else if (data) {
        // Multicast steps fall back to SM steps when NVLS is absent, the dtype has no
        // in-switch form, or the range is not 16-byte aligned.
        Primitive prim = op.primitive;
        const bool aligned = bytes_of(plan, op.count) % 16 == 0 && bytes_of(plan, op.off_remote) % 16 == 0 &&
                             bytes_of(plan, op.off_src) % 16 == 0 && bytes_of(plan, op.off_dst) % 16 == 0;
        const bool mm_ok = opt.multicast && aligned;
        if (prim == Primitive::kMmReduce && !(mm_ok && mm_dtype_ok(plan.dtype, op.red_op))) {
          fill_data(*cur, op, Primitive::kReduceMulti);
          cur->step.peer_mask = all_ranks_mask;
        } else if (prim == Primitive::kMmStore && !mm_ok) {
          // One put per peer, plus a local copy when source and destination differ.
          bool first = true;
          for (int i = 0; i < opt.world; ++i) {
            const int r = (opt.rank + 1 + i) % opt.world;
            if (r == opt.rank && op.off_src == op.off_dst) continue;
            if (!first) { cur = &new_step(static_cast<int>(c)); }
            first = false;
            PlanOp put = op;
            put.peer = r;
            fill_data(*cur, put, Primitive::kPut);
          }
          if (first) cur->has_data = false;
        } else if (prim == Primitive::kMmAllreduce && !(mm_ok && mm_dtype_ok(plan.dtype, op.red_op))) {
          PlanOp red = op;
          red.off_dst = op.off_remote;
          fill_data(*cur, red, Primitive::kReduceMulti);
          cur->step.peer_mask = all_ranks_mask;
          // The reduced slice is then pushed to every peer.  Readers of the same
          // offsets on the peers only ever read their *own* slices, so no barrier
          // is needed between the two halves.
          for (int i = 1; i < opt.world; ++i) {
            const int r = (opt.rank + i) % opt.world;
            cur = &new_step(static_cast<int>(c));
            PlanOp put = op;
            put.peer = r;
            put.off_src = put.off_dst = op.off_remote;
            fill_data(*cur, put, Primitive::kPut);
          }
        } else {
          fill_data(*cur, op, prim);
          out.uses_multicast |= prim == Primitive::kMmReduce || prim == Primitive::kMmStore ||
                                prim == Primitive::kMmAllreduce;
        }
        state = kHasData;
      }
      step_of_op[oi] = static_cast<int>(chain_steps[c].size()) - 1;
    }
  }

  // 2b. Closing barrier on reserved signal slots (top of the signal space, one per sender).
  if (opt.closing_barrier && opt.world > 1 && !chains.empty()) {
    PendingStep& post = new_step(0);
    for (size_t c = 1; c < chains.size(); ++c)
      if (!chains[c].ops.empty()) post.dep_ops.push_back(chains[c].ops.back());
    for (int i = 1; i < opt.world; ++i) {
      const int peer = (opt.rank + i) % opt.world;
      post.notifies.push_back(SigRef{peer, kSignalSlots - kMaxRanks + static_cast<uint32_t>(opt.rank)});
    }
    PendingStep& wait = new_step(0);
    for (int i = 1; i < opt.world; ++i) {
      const int peer = (opt.rank + i) % opt.world;
      wait.waits.push_back(SigRef{peer, kSignalSlots - kMaxRanks + static_cast<uint32_t>(peer)});
    }
  }

  // 3. CTA budget: chains with data share the budget in proportion to their largest step.
  std::vector<uint64_t> weight(chains.size(), 0);
  uint64_t total_weight = 0;
  for (size_t c = 0; c < chains.size(); ++c) {
    for (const auto& ps : chain_steps[c]) weight[c] = std::max<uint64_t>(weight[c], ps.step.bytes);
    total_weight += weight[c];
    out.max_step_bytes = std::max(out.max_step_bytes, weight[c]);
  }
  const uint32_t budget = std::max<uint32_t>(opt.total_ctas, static_cast<uint32_t>(chains.size()));
  std::vector<uint32_t> ctas(chains.size(), 1);
  uint32_t spare = budget - static_cast<uint32_t>(chains.size());
  if (total_weight > 0 && spare > 0) {
    for (size_t c = 0; c < chains.size(); ++c) {
      if (!weight[c]) continue;
      uint64_t want = static_cast<uint64_t>(spare) * weight[c] / total_weight;
      const uint64_t useful = weight[c] / std::max<uint64_t>(1, opt.min_bytes_per_cta);
      want = std::min<uint64_t>(want, useful ? useful - 1 : 0);
      ctas[c] = static_cast<uint32_t>(std::min<uint64_t>(1 + want, opt.max_ctas_per_chain));
    }
  }

  // 4. Emit flat tables.
  uint32_t next_cta = 0;
  for (size_t c = 0; c < chains.size(); ++c) {
    Chain ch{};
    ch.step_begin = static_cast<uint32_t>(out.steps.size());
    ch.step_count = static_cast<uint32_t>(chain_steps[c].size());
    ch.first_cta = next_cta;
    ch.num_ctas = ctas[c];
    next_cta += ctas[c];
    // Runs of independent pulls (peer -> distinct local ranges) or puts (local -> peers) need no
    // completion barrier between them: nothing signals in between and no step reads what the
    // previous one wrote.  Only for plans without cross-chain dependencies (progress counters
    // are published per step).
    auto independent = [&](const Step& a, const Step& b, int self_rank) {
      if (a.kind != b.kind || (a.kind != kStepCopy && a.kind != kStepPut)) return false;
      if (a.kind == kStepCopy) {
        if (a.peer == self_rank || b.peer == self_rank) return false;           // a local source may alias
        return a.off1 + a.bytes <= b.off1 || b.off1 + b.bytes <= a.off1;          // disjoint local destinations
      }
      return a.peer != b.peer || a.off1 + a.bytes <= b.off1 || b.off1 + b.bytes <= a.off1;
    };
    bool chain_has_deps = false;
    for (auto& ps : chain_steps[c]) chain_has_deps |= !ps.dep_ops.empty();
    const size_t first_step_of_chain = out.steps.size();
    uint32_t barriers = 0;
    for (auto& ps : chain_steps[c]) {
      Step s = ps.step;
      if (!ps.has_data) { s.kind = kStepNoop; s.bytes = 0; }
      s.n_wait = static_cast<uint8_t>(ps.waits.size());
      s.n_notify = static_cast<uint8_t>(ps.notifies.size());
      PCCL_CHECK(ps.waits.size() < 256 && ps.notifies.size() < 256 && ps.dep_ops.size() < 256,
                 "plan: more than 255 signal operations folded into one step");
      s.sig_begin = static_cast<uint32_t>(out.sigs.size());
      out.sigs.insert(out.sigs.end(), ps.waits.begin(), ps.waits.end());
      out.sigs.insert(out.sigs.end(), ps.notifies.begin(), ps.notifies.end());
      s.dep_begin = static_cast<uint32_t>(out.deps.size());
      for (int d : ps.dep_ops)
        out.deps.push_back(ChainDep{static_cast<uint32_t>(chain_of[d]), static_cast<uint32_t>(step_of_op[d] + 1)});
      s.n_dep = static_cast<uint8_t>(ps.dep_ops.size());
      out.steps.push_back(s);
    }
    const bool any_deps = [&] { for (auto& cs : chain_steps) for (auto& ps : cs) if (!ps.dep_ops.empty()) return true; return false; }();
    for (size_t k = first_step_of_chain; k < out.steps.size(); ++k) {
      Step& s = out.steps[k];
      if (!any_deps && !chain_has_deps && opt.defer_barriers && k + 1 < out.steps.size() && s.n_notify == 0) {
        const Step& next = out.steps[k + 1];
        if (next.n_wait == 0 && next.n_dep == 0 && independent(s, next, opt.rank)) s.defer_barrier = 1;
      }
      if (ch.num_ctas > 1) {
        if (s.n_wait + s.n_dep) ++barriers;
        if (s.kind != kStepNoop && !s.defer_barrier) ++barriers;
      }
    }
    ch.barriers_per_launch = barriers;
    out.chains.push_back(ch);
  }
  out.total_ctas = next_cta;
  (void)esize;
  return out;
}

}  // namespace pccl
