// Launching kernels whose CTAs wait on one another or on CTAs of the same kernel on a peer GPU.
//
// Such a kernel is only live if every CTA of its grid is resident at the same time: a CTA that
// spins on a flag keeps its SM, and the flag may be posted only once a CTA that has not started
// yet has run.  With the GPU to itself a grid no larger than (SMs x resident CTAs per SM) is
// resident as a whole, but next to another kernel that holds SMs (a GEMM overlapped with a
// gradient all-reduce) an ordinary launch starts whichever CTAs fit and the rest never run.
// A cooperative launch starts the grid only when all of it fits, so these kernels are launched
// cooperatively, with the grid clamped to what can be resident.  (The reference launches its
// persistent kernels with <<<>>> and relies on a small fixed grid:
// csrc/plugins/cuda/cuda_device.cc:287-324.)
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "util.h"

namespace pccl {

// Largest grid of which every CTA is resident at once; 0 when the kernel does not fit at all.
inline uint32_t coresident_limit(int ctas_per_sm, int sms) {
  if (ctas_per_sm <= 0 || sms <= 0) return 0;
  return static_cast<uint32_t>(ctas_per_sm) * static_cast<uint32_t>(sms);
}

// min(requested, limit), never 0 when the kernel fits.
inline uint32_t clamp_coresident(uint32_t requested, int ctas_per_sm, int sms) {
  const uint32_t limit = coresident_limit(ctas_per_sm, sms);
  if (limit == 0) return 0;
  if (requested == 0) return 1;
  return requested < limit ? requested : limit;
}

// PCCL_COOPERATIVE=0 falls back to ordinary launches (the grid is still clamped).
inline bool cooperative_launches() {
  static const bool on = Environs::get_flag("PCCL_COOPERATIVE", true);
  return on;
}

// Resident-CTA limit of `kernel` on the current device for this block size and dynamic shared
// memory.  The occupancy query costs about a microsecond, which a 5-microsecond collective would
// notice, so answers are remembered per (kernel, device, threads, shared memory).
template <class Kernel>
uint32_t max_coresident(Kernel kernel, int threads, size_t smem) {
  struct Entry { const void* fn; int dev, threads; size_t smem; uint32_t limit; };
  static thread_local Entry cache[8] = {};
  static thread_local int used = 0, next = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  const void* fn = reinterpret_cast<const void*>(kernel);
  for (int i = 0; i < used; ++i)
    if (cache[i].fn == fn && cache[i].dev == dev && cache[i].threads == threads && cache[i].smem == smem)
      return cache[i].limit;
  int sms = 0, per_sm = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess) return 0;
  const uint32_t limit = coresident_limit(per_sm, sms);
  cache[next] = Entry{fn, dev, threads, smem, limit};
  next = (next + 1) % 8;
  if (used < 8) ++used;
  return limit;
}

// Launch `kernel` with all CTAs co-resident; `args` points at the kernel's arguments in order.
// `exact_grid`: the grid size is part of the kernel's protocol (completion counts), so a grid
// that cannot be resident is an error instead of being clamped.  Returns the grid used.
template <class Kernel>
uint32_t launch_coresident_args(Kernel kernel, uint32_t grid, int threads, size_t smem, cudaStream_t stream,
                                void** args, bool exact_grid = false) {
  const uint32_t limit = max_coresident(kernel, threads, smem);
  PCCL_CHECK(limit > 0, "kernel does not fit on this device (" << threads << " threads, " << smem
                                                                << " bytes of shared memory)");
  if (grid > limit) {
    PCCL_CHECK(!exact_grid, "a grid of " << grid << " CTAs cannot be resident at once (limit " << limit
                                         << "); its CTAs wait on one another, so it is refused");
    grid = limit;
  }
  if (grid == 0) grid = 1;
  cudaError_t err;
  if (cooperative_launches())
    err = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), dim3(grid), dim3(threads), args, smem,
                                      stream);
  else
    err = cudaLaunchKernel(reinterpret_cast<const void*>(kernel), dim3(grid), dim3(threads), args, smem, stream);
  PCCL_CHECK(err == cudaSuccess, "kernel launch failed: " << cudaGetErrorString(err));
  return grid;
}

// The common case of a kernel with one parameter block.
template <class Kernel, class Params>
uint32_t launch_coresident(Kernel kernel, uint32_t grid, int threads, size_t smem, cudaStream_t stream,
                           const Params& params, bool exact_grid = false) {
  Params copy = params;
  void* args[] = {&copy};
  return launch_coresident_args(kernel, grid, threads, smem, stream, args, exact_grid);
}

}  // namespace pccl
