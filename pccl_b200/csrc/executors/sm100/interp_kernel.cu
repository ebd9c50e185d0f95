// plan_interp_kernel: one persistent launch executes a rank's whole step program.
//
// Grid: x = CTAs of this rank, partitioned over the program's chains;
//       y = virtual rank (1 in production; >1 only when several ranks are
//           emulated on one GPU in a single cooperative launch, for tests).
// Per step, in plan order:
//   1. lane i of the chain's lead CTA waits for signal i (bounded acquire spin,
//      then consumes one count) / for dependency i on another chain;
//   2. a chain-wide barrier releases the other CTAs (skipped for 1-CTA chains
//      and for steps without waits);
//   3. all CTAs of the chain move their share of the data;
//   4. a second chain-wide barrier (with the fence scope the step needs)
//      establishes that every CTA's writes are done;
//   5. lane i of the lead CTA posts signal i with red.release.sys, and the
//      chain's progress counter is bumped for dependent chains.
// Any wait that exhausts its budget records a DeviceStatus, raises the abort
// flag and every CTA leaves; the context stays usable.
// (Replaces the reference's cuda_executor_kernel and fused_allreduce_kernel:
// csrc/plugins/cuda/cuda_executor.cu:526-918, 963-1057.)
#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include "dataops.cuh"
#include "program.h"

namespace pccl {

namespace {

struct WaitCtx {
  DeviceStatus* status;
  DeviceStatus* host_status;
  uint64_t deadline;
  int32_t rank;
  uint32_t chain, step;
};

__device__ __forceinline__ bool aborted(const DeviceStatus* st) {
  return ptx::ld_relaxed_sys(&st->abort) != 0;
}

__device__ __noinline__ void give_up(const WaitCtx& w, uint32_t code, uint32_t slot, uint32_t observed,
                                     uint32_t expected) {
  // First failure wins the record; everyone sees the flag.
  if (atomicCAS(&w.status->abort, 0u, 1u) == 0u) {
    w.status->code = code;
    w.status->rank = w.rank;
    w.status->chain = w.chain;
    w.status->step = w.step;
    w.status->slot = slot;
    w.status->observed = observed;
    w.status->expected = expected;
    if (w.host_status) {
      DeviceStatus rec = *w.status;
      rec.abort = 1;
      *w.host_status = rec;
    }
    __threadfence_system();
  }
}

// Spin until pred(value) holds.  Polls the clock and the abort flag every 64 probes.
template <class Load, class Pred>
__device__ __forceinline__ bool bounded_spin(const WaitCtx& w, Load load, Pred pred, uint32_t code,
                                             uint32_t slot, uint32_t expected) {
  uint32_t probes = 0;
  for (;;) {
    uint32_t v = load();
    if (pred(v)) return true;
    if ((++probes & 63u) == 0u) {
      if (aborted(w.status)) return false;
      if (ptx::globaltimer() > w.deadline) {
        give_up(w, code, slot, v, expected);
        return false;
      }
      __nanosleep(32);
    }
  }
}

// Barrier over the CTAs of one chain on a monotonically increasing counter.
// `target` is the absolute count that marks completion of this barrier.
__device__ __forceinline__ bool chain_barrier(uint32_t* counter, uint32_t target, bool sys_fence,
                                              const WaitCtx& w, uint32_t* smem_flag) {
  __syncthreads();
  if (threadIdx.x == 0) {
    if (sys_fence) ptx::fence_sys(); else ptx::fence_gpu();
    ptx::red_release_gpu_add(counter, 1u);
    bool ok = bounded_spin(
        w, [&] { return ptx::ld_acquire_gpu(counter); },
        [&](uint32_t v) { return static_cast<int32_t>(v - target) >= 0; }, kBarrierTimeout, 0, target);
    *smem_flag = ok ? 1u : 0u;
  }
  __syncthreads();
  return *smem_flag != 0u;
}

// Fill the shared source table for one step (one thread), return the destination.
__device__ __forceinline__ uint8_t* describe_step(const RankProgram& P, const Step& s, SrcTable* t) {
  uint8_t* self = P.data[P.rank];
  t->count = 1;
  t->remote_mask = 0;
  switch (s.kind) {
    case kStepCopy:
      t->ptr[0] = P.data[s.peer] + s.off0;
      t->remote_mask = s.peer != P.rank;
      return self + s.off1;
    case kStepPut:
      t->ptr[0] = self + s.off0;
      return P.data[s.peer] + s.off1;
    case kStepReduce:
      t->ptr[0] = P.data[s.peer] + s.off0;
      t->ptr[1] = self + s.off1;
      t->remote_mask = s.peer != P.rank;
      t->count = 2;
      return self + s.off2;
    case kStepReduceMulti: {
      int n = 0;
      // Start with the rank after this one so simultaneous readers spread over sources.
      for (int i = 0; i < P.world; ++i) {
        const int r = (P.rank + 1 + i) % P.world;
        if (s.peer_mask >> r & 1u) {
          t->ptr[n] = P.data[r] + s.off0;
          t->remote_mask |= static_cast<uint32_t>(r != P.rank) << n;
          ++n;
        }
      }
      t->count = n;
      return self + s.off2;
    }
    case kStepMmReduce:
      t->ptr[0] = P.mc_data + s.off0;
      return self + s.off2;
    case kStepMmStore:
      t->ptr[0] = self + s.off0;
      return P.mc_data + s.off1;
    case kStepMmAllreduce:
      t->ptr[0] = P.mc_data + s.off0;
      return P.mc_data + s.off0;
    case kStepScale:
      t->ptr[0] = self + s.off0;
      return self + s.off0;
    default:
      t->count = 0;
      return nullptr;
  }
}

template <int DT>
__device__ __forceinline__ void run_typed(const Step& s, const SrcTable& t, uint8_t* dst, uint32_t cta,
                                          uint32_t nctas) {
  switch (s.kind) {
    case kStepReduce:
    case kStepReduceMulti:
      reduce_range<DT>(t, dst, s.bytes, s.red_op, 1.0f, cta, nctas);
      break;
    case kStepScale:
      reduce_range<DT>(t, dst, s.bytes, kRedSum, s.scale, cta, nctas);
      break;
    default:
      break;
  }
}

template <int DT>
__device__ __forceinline__ void run_multimem(const Step& s, const SrcTable& t, uint8_t* dst, uint32_t cta,
                                             uint32_t nctas) {
  if (s.kind == kStepMmReduce) mm_reduce_range<DT, false>(t.ptr[0], dst, s.bytes, s.red_op, cta, nctas);
  else mm_reduce_range<DT, true>(t.ptr[0], dst, s.bytes, s.red_op, cta, nctas);
}

template <int DT>
__device__ __forceinline__ void run_step_data(const RankProgram& P, const Step& s, const SrcTable& t,
                                              uint8_t* dst, uint32_t cta, uint32_t nctas) {
  if (t.count == 0 || dst == nullptr) return;
  switch (s.kind) {
    case kStepCopy:
    case kStepPut:
      copy_range<false>(t, dst, s.bytes, cta, nctas);
      return;
    case kStepMmStore:
      if (P.mc_data) copy_range<true>(t, dst, s.bytes, cta, nctas);
      return;
    case kStepMmReduce:
    case kStepMmAllreduce:
      if (!P.mc_data) return;            // the host never lowers multimem steps without NVLS
      // multimem arithmetic exists for f32 / f16 / bf16 only; the host lowers fp8 to SM steps.
      if constexpr (DT == kF32 || DT == kBF16 || DT == kF16) run_multimem<DT>(s, t, dst, cta, nctas);
      return;
    default:
      break;
  }
  run_typed<DT>(s, t, dst, cta, nctas);
}

}  // namespace

// One instance per element type: the data movers are inlined, so the register allocator sees
// the whole loop nest (separately compiled movers spilled their load tiles at every call).
template <int DT>
__global__ void __launch_bounds__(kInterpThreads, 1) plan_interp_kernel(const LaunchParams lp) {
  const RankProgram& P = lp.programs[blockIdx.y];
  __shared__ uint32_t s_ok;
  __shared__ uint32_t s_chain;
  __shared__ SrcTable s_src;
  __shared__ uint8_t* s_dst;

  // Which chain does this CTA serve?
  if (threadIdx.x == 0) {
    uint32_t found = 0xffffffffu;
    for (uint32_t c = 0; c < P.num_chains; ++c) {
      const Chain& ch = P.chains[c];
      if (blockIdx.x >= ch.first_cta && blockIdx.x < ch.first_cta + ch.num_ctas) { found = c; break; }
    }
    s_chain = found;
  }
  __syncthreads();
  const uint32_t chain_id = s_chain;
  if (chain_id == 0xffffffffu) return;          // spare CTA
  const Chain chain = P.chains[chain_id];
  const uint32_t cta = blockIdx.x - chain.first_cta;
  const bool lead = cta == 0;
  const bool multi_cta = chain.num_ctas > 1;

  uint32_t* sync_counter = P.chain_sync + chain_id;
  uint32_t barrier_no = lp.launch_index * chain.barriers_per_launch;   // barriers completed so far
  const uint32_t progress_base = lp.launch_index * chain.step_count;

  WaitCtx w;
  w.status = P.status;
  w.host_status = P.host_status;
  w.deadline = ptx::globaltimer() + P.timeout_ns;
  w.rank = P.rank;
  w.chain = chain_id;

  uint32_t* my_signals = P.signals[P.rank];
  // Timeline stamps of this chain's steps (lead CTA, thread 0), when tracing is on.
  uint64_t* trace = (P.trace != nullptr && lead && threadIdx.x == 0)
                        ? P.trace + static_cast<uint64_t>(chain.step_begin) * kTraceStamps : nullptr;

  for (uint32_t k = 0; k < chain.step_count; ++k) {
    const Step s = P.steps[chain.step_begin + k];
    w.step = k;
    if (trace) trace[k * kTraceStamps + 0] = ptx::globaltimer();

    // 1. waits (lead CTA, one lane per wait)
    const uint32_t nwait = s.n_wait + s.n_dep;
    if (nwait) {
      if (lead) {
        bool ok = true;
        for (uint32_t i = threadIdx.x; i < nwait; i += blockDim.x) {
          if (i < s.n_wait) {
            const SigRef ref = P.sigs[s.sig_begin + i];
            uint32_t* slot = my_signals + ref.slot;
            // Consume exactly one count: compare-and-swap so that two waiters of one
            // slot can never both pass on a single post.
            ok = bounded_spin(
                w, [&] { return ptx::ld_acquire_sys(slot); },
                [&](uint32_t v) {
                  return static_cast<int32_t>(v) > 0 && atomicCAS(slot, v, v - 1u) == v;
                },
                kSignalTimeout, ref.slot, 1);
          } else {
            const ChainDep d = P.deps[s.dep_begin + (i - s.n_wait)];
            const uint32_t need = lp.launch_index * P.chains[d.chain].step_count + d.steps_done;
            const uint32_t* prog = P.chain_progress + d.chain;
            ok = bounded_spin(
                w, [&] { return ptx::ld_acquire_gpu(prog); },
                [&](uint32_t v) { return static_cast<int32_t>(v - need) >= 0; }, kDepTimeout, d.chain,
                need);
          }
          if (!ok) break;
        }
        // Combine the lanes' outcomes: any failure already raised the abort flag.
        __syncthreads();
        if (threadIdx.x == 0) s_ok = aborted(P.status) ? 0u : 1u;
        __syncthreads();
        if (!s_ok && !multi_cta) return;
      }
      // 2. release the followers
      if (multi_cta) {
        ++barrier_no;
        if (!chain_barrier(sync_counter, barrier_no * chain.num_ctas, false, w, &s_ok)) return;
        if (aborted(P.status)) return;
      }
    }

    if (trace) trace[k * kTraceStamps + 1] = ptx::globaltimer();

    // 3. data
    if (s.kind != kStepNoop && s.bytes) {
      if (threadIdx.x == 0) s_dst = describe_step(P, s, &s_src);
      __syncthreads();
      run_step_data<DT>(P, s, s_src, s_dst, cta, chain.num_ctas);
    }

    // 4. completion barrier
    const bool publishes = s.n_notify != 0;
    if (multi_cta) {
      if (s.kind != kStepNoop && !s.defer_barrier) {
        ++barrier_no;
        if (!chain_barrier(sync_counter, barrier_no * chain.num_ctas, s.writes_remote != 0, w, &s_ok))
          return;
      } else if (s.defer_barrier) {
        __syncthreads();                       // the shared step descriptor is about to be rewritten
      }
    } else {
      __syncthreads();
    }

    if (trace) trace[k * kTraceStamps + 2] = ptx::globaltimer();

    // 5. notifies + progress (lead CTA)
    if (lead) {
      if (publishes && threadIdx.x < s.n_notify) {
        // This lane did not write the data itself; the release below is cumulative over what the
        // barrier above made visible to it (an explicit system fence in front of it doubled the cost
        // of a post: 2 us each in a timeline).
        const SigRef ref = P.sigs[s.sig_begin + s.n_wait + threadIdx.x];
        ptx::red_release_sys_add(P.signals[ref.rank] + ref.slot, 1u);
      }
      if (threadIdx.x == 0) {
        // Read by other chains of this GPU only: GPU scope.  (A system-scope release here waited for
        // the acknowledgement of the notify just posted over NVLink: 3 us per step in a timeline.)
        ptx::st_release_gpu(P.chain_progress + chain_id, progress_base + k + 1);
      }
    }
    if (trace) trace[k * kTraceStamps + 3] = ptx::globaltimer();
  }
}

__global__ void __launch_bounds__(kInterpThreads, 1) scale_kernel(uint8_t* ptr, uint64_t bytes, uint32_t dtype, float scale) {
  __shared__ SrcTable t;
  if (threadIdx.x == 0) { t.ptr[0] = ptr; t.count = 1; t.remote_mask = 0; }
  __syncthreads();
  switch (dtype) {
    case kF32: reduce_range<kF32>(t, ptr, bytes, kRedSum, scale, blockIdx.x, gridDim.x); break;
    case kF16: reduce_range<kF16>(t, ptr, bytes, kRedSum, scale, blockIdx.x, gridDim.x); break;
    case kBF16: reduce_range<kBF16>(t, ptr, bytes, kRedSum, scale, blockIdx.x, gridDim.x); break;
    case kE4M3: reduce_range<kE4M3>(t, ptr, bytes, kRedSum, scale, blockIdx.x, gridDim.x); break;
    default: reduce_range<kE5M2>(t, ptr, bytes, kRedSum, scale, blockIdx.x, gridDim.x); break;
  }
}

int launch_scale(void* ptr, uint64_t bytes, uint32_t dtype, float scale, void* stream) {
  if (bytes == 0) return 0;
  const uint32_t ctas = static_cast<uint32_t>(bytes / (256 << 10)) + 1;
  scale_kernel<<<ctas > 128 ? 128 : ctas, kInterpThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint8_t*>(ptr), bytes, dtype, scale);
  return static_cast<int>(cudaGetLastError());
}

namespace {
const void* interp_entry(uint32_t dtype) {
  switch (dtype) {
    case kF32: return reinterpret_cast<const void*>(plan_interp_kernel<kF32>);
    case kF16: return reinterpret_cast<const void*>(plan_interp_kernel<kF16>);
    case kBF16: return reinterpret_cast<const void*>(plan_interp_kernel<kBF16>);
    case kE4M3: return reinterpret_cast<const void*>(plan_interp_kernel<kE4M3>);
    default: return reinterpret_cast<const void*>(plan_interp_kernel<kE5M2>);
  }
}
}  // namespace

int set_mover_tuning(uint32_t word) {
  return static_cast<int>(cudaMemcpyToSymbol(g_mover_tuning, &word, sizeof word));
}

int plan_interp_max_ctas(int threads) {
  // Asked on every launch: remember the answer per device (the block size is always kInterpThreads).
  static int cached[64] = {};
  int dev = 0, sms = 0, per_sm = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  const bool cacheable = dev >= 0 && dev < 64 && threads == static_cast<int>(kInterpThreads);
  if (cacheable && cached[dev] > 0) return cached[dev];
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, plan_interp_kernel<kF32>, threads, 0) != cudaSuccess)
    return 0;
  if (cacheable) cached[dev] = sms * per_sm;
  return sms * per_sm;
}

int launch_plan_interp(const LaunchParams& params, const LaunchConfig& cfg, void* stream) {
  dim3 grid(cfg.ctas, cfg.virtual_ranks, 1), block(cfg.threads, 1, 1);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LaunchParams copy = params;
  void* args[] = {&copy};
  // Virtual ranks wait on one another inside a single launch: co-residency must be guaranteed.
  if (cfg.cooperative)
    return static_cast<int>(cudaLaunchCooperativeKernel(interp_entry(cfg.dtype), grid, block, args, 0, st));
  return static_cast<int>(cudaLaunchKernel(interp_entry(cfg.dtype), grid, block, args, 0, st));
}

}  // namespace pccl
