#include "ce_executor.h"

#include <cstring>

#include "../../engine/cuda_driver.h"

namespace pccl {

CeSchedule::~CeSchedule() { clear(); }

void CeSchedule::clear() {
  for (auto& chain : chains_)
    for (CeItem& it : chain) {
      if (it.d_program) cudaFree(it.d_program);
      if (it.counters) cudaFree(it.counters);
    }
  chains_.clear();
  for (cudaStream_t s : streams_) cudaStreamDestroy(s);
  for (cudaEvent_t e : done_) cudaEventDestroy(e);
  streams_.clear();
  done_.clear();
  if (fork_) { cudaEventDestroy(fork_); fork_ = nullptr; }
  if (d_chain_tables_) { cudaFree(d_chain_tables_); d_chain_tables_ = nullptr; }
  copies_ = segments_ = 0;
}

bool CeSchedule::supports(const LoweredProgram& lp) {
  for (const Step& s : lp.steps)
    if (s.n_dep) return false;
  return true;
}

void CeSchedule::build(const LoweredProgram& lp, const RankProgram& base, uint64_t min_copy_bytes) {
  dtype_ = base.dtype;
  clear();
  PCCL_CHECK(supports(lp), "the copy-engine executor cannot run plans whose chains depend on one another");
  // One Chain record per segment, all in one device table.
  std::vector<Chain> seg_chains;
  chains_.resize(lp.chains.size());
  for (size_t c = 0; c < lp.chains.size(); ++c) {
    const Chain& ch = lp.chains[c];
    uint32_t seg_begin = ch.step_begin;
    auto flush = [&](uint32_t end) {
      if (end <= seg_begin) return;
      CeItem it;
      it.step_begin = seg_begin;
      it.step_count = end - seg_begin;
      it.ctas = ch.num_ctas;
      uint32_t barriers = 0;
      for (uint32_t k = seg_begin; k < end; ++k) {
        const Step& s = lp.steps[k];
        if (ch.num_ctas > 1) {
          if (s.n_wait + s.n_dep) ++barriers;
          if (s.kind != kStepNoop) ++barriers;
        }
      }
      it.barriers_per_launch = barriers;
      chains_[c].push_back(it);
      ++segments_;
    };
    for (uint32_t k = ch.step_begin; k < ch.step_begin + ch.step_count; ++k) {
      const Step& s = lp.steps[k];
      const bool dma = s.kind == kStepCopy && s.bytes >= min_copy_bytes;
      if (!dma) continue;
      // A copy step is [waits] copy [notifies]: the waits end the previous segment, the
      // notifies open the next one.  Both halves are expressed as no-op steps that keep
      // the step's signal lists, so they need their own Step records: emitted below.
      flush(k);
      CeItem pre;             // waits of step k
      pre.step_begin = k; pre.step_count = 1; pre.ctas = 1;
      CeItem cp;
      cp.is_copy = true;
      cp.src_rank = s.peer; cp.src_off = s.off0; cp.dst_off = s.off1; cp.bytes = s.bytes;
      if (s.n_wait) { pre.part = CeItem::kWaitsOfCopy; chains_[c].push_back(pre); ++segments_; }
      chains_[c].push_back(cp);
      ++copies_;
      if (s.n_notify) { CeItem post = pre; post.part = CeItem::kNotifiesOfCopy; chains_[c].push_back(post); ++segments_; }
      seg_begin = k + 1;
    }
    flush(ch.step_begin + ch.step_count);
  }

  // Materialise device programs for kernel segments.  Waits-only / notifies-only halves of a
  // copy step get a private copy of the step with the data part (and the other half) removed.
  std::vector<Step> extra_steps;
  for (auto& chain : chains_)
    for (CeItem& it : chain) {
      if (it.is_copy) continue;
      const bool waits_only = it.part == CeItem::kWaitsOfCopy, notifies_only = it.part == CeItem::kNotifiesOfCopy;
      Chain rec{};
      rec.step_count = it.step_count;
      rec.first_cta = 0;
      rec.num_ctas = it.ctas;
      rec.barriers_per_launch = it.barriers_per_launch;
      if (waits_only || notifies_only) {
        Step s = lp.steps[it.step_begin];
        s.kind = kStepNoop;
        s.bytes = 0;
        if (waits_only) s.n_notify = 0;
        else { s.sig_begin += s.n_wait; s.n_wait = 0; s.n_dep = 0; }
        rec.step_begin = 0x80000000u | static_cast<uint32_t>(extra_steps.size());   // patched below
        extra_steps.push_back(s);
      } else {
        rec.step_begin = it.step_begin;
      }
      seg_chains.push_back(rec);
    }
  // Device layout: [extra steps][segment chain records].
  const size_t steps_bytes = (extra_steps.size() * sizeof(Step) + 127) / 128 * 128;
  const size_t total = steps_bytes + seg_chains.size() * sizeof(Chain) + 128;
  PCCL_CUDA(cudaMalloc(&d_chain_tables_, total));
  auto* d_base = static_cast<uint8_t*>(d_chain_tables_);
  if (!extra_steps.empty())
    PCCL_CUDA(cudaMemcpy(d_base, extra_steps.data(), extra_steps.size() * sizeof(Step), cudaMemcpyHostToDevice));
  const Step* d_extra = reinterpret_cast<const Step*>(d_base);
  Chain* d_chains = reinterpret_cast<Chain*>(d_base + steps_bytes);

  size_t idx = 0;
  for (auto& chain : chains_)
    for (CeItem& it : chain) {
      if (it.is_copy) continue;
      Chain rec = seg_chains[idx];
      RankProgram prog = base;
      if (rec.step_begin & 0x80000000u) {
        // The private step lives in the extra table: point `steps` there, index 0-based.
        prog.steps = d_extra + (rec.step_begin & 0x7fffffffu);
        rec.step_begin = 0;
      }
      PCCL_CUDA(cudaMemcpy(d_chains + idx, &rec, sizeof(Chain), cudaMemcpyHostToDevice));
      PCCL_CUDA(cudaMalloc(reinterpret_cast<void**>(&it.counters), 2 * sizeof(uint32_t)));
      PCCL_CUDA(cudaMemset(it.counters, 0, 2 * sizeof(uint32_t)));
      prog.num_chains = 1;
      prog.chains = d_chains + idx;
      prog.chain_sync = it.counters;
      prog.chain_progress = it.counters + 1;
      PCCL_CUDA(cudaMalloc(reinterpret_cast<void**>(&it.d_program), sizeof(RankProgram)));
      PCCL_CUDA(cudaMemcpy(it.d_program, &prog, sizeof(RankProgram), cudaMemcpyHostToDevice));
      ++idx;
    }

  streams_.resize(chains_.size());
  done_.resize(chains_.size());
  for (size_t c = 0; c < chains_.size(); ++c) {
    PCCL_CUDA(cudaStreamCreateWithFlags(&streams_[c], cudaStreamNonBlocking));
    PCCL_CUDA(cudaEventCreateWithFlags(&done_[c], cudaEventDisableTiming));
  }
  PCCL_CUDA(cudaEventCreateWithFlags(&fork_, cudaEventDisableTiming));
}

void CeSchedule::run(uint8_t* const* data, int self, uint32_t launch_index, cudaStream_t stream) {
  PCCL_CUDA(cudaEventRecord(fork_, stream));
  for (size_t c = 0; c < chains_.size(); ++c) {
    cudaStream_t cs = streams_[c];
    PCCL_CUDA(cudaStreamWaitEvent(cs, fork_, 0));
    for (const CeItem& it : chains_[c]) {
      if (it.is_copy) {
        PCCL_CUDA(cudaMemcpyAsync(data[self] + it.dst_off, data[it.src_rank] + it.src_off, it.bytes,
                                  cudaMemcpyDeviceToDevice, cs));
      } else {
        LaunchParams lp{it.d_program, launch_index};
        LaunchConfig cfg{it.ctas, kInterpThreads, 1, false, dtype_};
        const int err = launch_plan_interp(lp, cfg, cs);
        PCCL_CHECK(err == 0, "copy-engine executor: segment launch failed: "
                                 << cudaGetErrorString(static_cast<cudaError_t>(err)));
      }
    }
    PCCL_CUDA(cudaEventRecord(done_[c], cs));
    PCCL_CUDA(cudaStreamWaitEvent(stream, done_[c], 0));
  }
}

void CeSchedule::reset_counters() {
  for (auto& chain : chains_)
    for (CeItem& it : chain)
      if (it.counters) cudaMemset(it.counters, 0, 2 * sizeof(uint32_t));
}

}  // namespace pccl
