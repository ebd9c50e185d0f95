// Launchers of the tcgen05 GEMM kernels: tensor-map construction and launch.
#include <cuda.h>

#include <algorithm>
#include <mutex>
#include <vector>

#include "../common/launch.h"
#include "../engine/cuda_driver.h"
#include "gemm_host.h"
#include "moe_policies.cuh"
#include "tp_policies.cuh"
#include "umma_gemm.cuh"
#include "umma_gemm2.cuh"

namespace pccl {
namespace gemm {

namespace {

uint32_t* g_error = nullptr;
std::once_flag g_error_once, g_tail_once;
float* g_tail_ws = nullptr;            // split-tail workspace and counters of the paired kernel (allocated on first use)
uint32_t* g_tail_counters = nullptr;
uint64_t* g_trace = nullptr;          // [kTraceCtas][kGemmTraceStamps], allocated by gemm_trace_enable
constexpr int kTraceCtas = 256;

// 2-D bf16 tensor map over a row-major matrix: inner dimension = columns, box = kBK x box_rows,
// 128-byte swizzle (the layout tcgen05.mma's SWIZZLE_128B descriptor expects).
CUtensorMap encode_map(const MatrixDesc& m, uint32_t box_rows);

// Encoding a tensor map costs a few microseconds of host time; operands of a layer recur
// call after call, so the last few maps are kept.
CUtensorMap make_map(const MatrixDesc& m, uint32_t box_rows) {
  struct Key {
    const void* ptr; int rows, cols; int64_t ld; uint32_t box;
    bool operator==(const Key& o) const {
      return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box == o.box;
    }
  };
  struct Entry { Key key; CUtensorMap map; };
  static std::mutex mu;
  static Entry cache[16];
  static int used = 0, next = 0;
  const Key key{m.ptr, m.rows, m.cols, m.ld, box_rows};
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < used; ++i)
    if (cache[i].key == key) return cache[i].map;
  Entry& e = cache[next];
  next = (next + 1) % 16;
  if (used < 16) ++used;
  e.key = key;
  e.map = encode_map(m, box_rows);
  return e.map;
}

CUtensorMap encode_map(const MatrixDesc& m, uint32_t box_rows) {
  PCCL_CHECK(reinterpret_cast<uintptr_t>(m.ptr) % 16 == 0, "GEMM operand must be 16-byte aligned");
  PCCL_CHECK(m.ld % 8 == 0, "GEMM operand leading dimension must be a multiple of 8 elements");
  CUtensorMap map;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(m.cols), static_cast<cuuint64_t>(m.rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(m.ld) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), box_rows};
  const cuuint32_t elem[2] = {1, 1};
  PCCL_CU(DriverApi::get().cuTensorMapEncodeTiled(
      &map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(m.ptr), dims, strides, box, elem,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  return map;
}

int sm_count() {
  static int sms = [] {
    int dev = 0, n = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
  }();
  return sms;
}

template <class Policy>
void launch(const MatrixDesc& a, const MatrixDesc& b, const typename Policy::Params& params, int ctas,
            uint64_t timeout_ms, cudaStream_t stream, int aux_ctas = 0, int groups = 1) {
  // groups > 1: B stacks `groups` weight matrices of N rows each and the tile list is built on
  // the device, so the grid is not trimmed to a tile count known here.
  PCCL_CHECK(a.cols == b.cols, "GEMM: A and B disagree on K (" << a.cols << " vs " << b.cols << ")");
  PCCL_CHECK(a.cols % 8 == 0, "GEMM: K must be a multiple of 8");
  PCCL_CHECK(b.rows % groups == 0 && b.rows / groups % 8 == 0, "GEMM: N must be a multiple of 8");
  Problem g;
  g.M = a.rows; g.N = b.rows / groups; g.K = a.cols;
  g.tiles_m = (g.M + kBM - 1) / kBM;
  g.tiles_n = (g.N + kBN - 1) / kBN;
  g.bn = kBN;
  g.trace = g_trace;
  g.tail_first = g.num_items = g.tiles_m * g.tiles_n;         // the one-SM kernel never splits
  g.tail_slices = 1; g.tail_kb = 0; g.tail_ws = nullptr; g.tail_counters = nullptr;
  g.error = error_word();
  g.timeout_ns = timeout_ms * 1000000ull;
  const CUtensorMap ta = make_map(a, kBM), tb = make_map(b, kBN);
  static std::once_flag attr_once;
  auto kernel = umma_gemm_kernel<Policy>;
  PCCL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
  const int tiles = g.tiles_m * g.tiles_n;
  // `grid` counts all CTAs (one per SM at most: CTAs wait on one another through flags);
  // `aux_ctas` of them do not run GEMM tiles.
  int grid = ctas > 0 ? ctas : sm_count();
  if (grid > sm_count()) grid = sm_count();
  if (groups == 1 && grid - aux_ctas > tiles) grid = tiles + aux_ctas;
  if (grid - aux_ctas < 1) grid = aux_ctas + 1;
  // Policies make CTAs wait on flags posted by other CTAs of this launch (reducers, copiers) and by
  // the same kernel on the peers, so the grid must be resident as a whole.
  CUtensorMap ta_arg = ta, tb_arg = tb;
  Problem g_arg = g;
  typename Policy::Params params_arg = params;
  void* args[] = {&ta_arg, &tb_arg, &g_arg, &params_arg};
  launch_coresident_args(kernel, static_cast<uint32_t>(grid), kThreads + 32 * Policy::kReducerWarps, kSmemBytes, stream,
                         args, true);
  (void)attr_once;
}

// Tile width of the paired kernel.  Measured on 8192 x 1792 x 4096: 256 columns 1198 TFLOP/s, 224 the
// same, 128 784, 96 638, 64 462.  A 256 x 256 x 16 step reads 8 KB of shared memory per SM in the 64
// clocks its MMA takes; a narrower tile still reads the same 4 KB of A per step while its MMA
// shrinks, so it turns shared-memory bound and a round costs almost the same however narrow the
// tile.  Narrow tiles therefore never pay for the better fit of their tile count to the SM pairs:
// the width stays 256 unless PCCL_GEMM_TILE_N (a multiple of 32) says otherwise.
int pick_tile_n(int, int, int) { return kBN; }

// The two-SM kernel: clusters of two CTAs, each CTA loading 128-row boxes of A and of B.
template <class Policy>
void launch_pair(const MatrixDesc& a, const MatrixDesc& b, const typename Policy::Params& params, int ctas,
                 uint64_t timeout_ms, cudaStream_t stream, bool cooperative, int aux_ctas = 0, int groups = 1) {
  // groups > 1: B stacks `groups` weight matrices of N rows each and the tile list is built on the
  // device (ragged pairs), so the grid is not trimmed to a tile count known here.
  PCCL_CHECK(a.cols == b.cols, "GEMM: A and B disagree on K (" << a.cols << " vs " << b.cols << ")");
  PCCL_CHECK(a.cols % 8 == 0 && b.rows % groups == 0 && b.rows / groups % 8 == 0, "GEMM: K and N must be multiples of 8");
  Problem g;
  g.M = a.rows; g.N = b.rows / groups; g.K = a.cols;
  g.tiles_m = (g.M + kBM - 1) / kBM;
  PCCL_CHECK(aux_ctas % 2 == 0, "paired GEMM: auxiliary CTAs come in whole clusters of two");
  int grid = ctas > 0 ? ctas : sm_count();
  if (grid > sm_count()) grid = sm_count();
  grid &= ~1;                                             // whole pairs only
  if (grid < aux_ctas + 2) grid = aux_ctas + 2;
  const int64_t forced_bn = Environs::get_int("PCCL_GEMM_TILE_N", 0);
  g.bn = forced_bn >= 32 && forced_bn <= kBN && forced_bn % 32 == 0 ? static_cast<int>(forced_bn)
                                                                      : pick_tile_n(g.M, g.N, (grid - aux_ctas) / 2);
  g.tiles_n = (g.N + g.bn - 1) / g.bn;
  g.trace = g_trace;
  g.error = error_word();
  g.timeout_ns = timeout_ms * 1000000ull;
  const CUtensorMap ta = make_map(a, kBM), tb = make_map(b, g.bn / 2);
  auto kernel = umma_gemm2_kernel<Policy>;
  PCCL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes2));
  const int pair_tiles = (g.tiles_m + 1) / 2 * g.tiles_n;
  if (groups == 1 && grid - aux_ctas > 2 * pair_tiles) grid = 2 * pair_tiles + aux_ctas;
  // Split tail: when the last round keeps at most half of the pairs busy, cut its tiles along K.
  const int pairs = (grid - aux_ctas) / 2, k_blocks = (g.K + kBK - 1) / kBK;
  g.tail_first = g.num_items = pair_tiles;
  g.tail_slices = 1; g.tail_kb = k_blocks; g.tail_ws = nullptr; g.tail_counters = nullptr;
  bool split = false;
  if (Policy::kSplitTail && Environs::get_flag("PCCL_GEMM_SPLIT_TAIL", true) && pair_tiles > pairs && g.bn == kBN) {
    const int tail = pair_tiles % pairs;
    int slices = tail > 0 ? std::min(pairs / tail, k_blocks / 4) : 0;      // at least four k-blocks per slice
    // Measured on B200: the workspace round trip costs about 8 us, half of a K=4096 tile, so two
    // slices do not pay; from three slices on the shorter last round wins.
    static const int min_slices = Environs::get_int("PCCL_GEMM_SPLIT_MIN_SLICES", 3);
    if (tail > 0 && tail <= kTailMaxTiles && slices >= std::max(2, min_slices)) {
      const int per = (k_blocks + slices - 1) / slices;
      slices = (k_blocks + per - 1) / per;
      std::call_once(g_tail_once, [] {
        PCCL_CUDA(cudaMalloc(reinterpret_cast<void**>(&g_tail_ws),
                             static_cast<size_t>(sm_count() / 2 + 1) * 2 * kBM * kBN * sizeof(float)));
        PCCL_CUDA(cudaMalloc(reinterpret_cast<void**>(&g_tail_counters), 2 * kTailMaxTiles * sizeof(uint32_t)));
        PCCL_CUDA(cudaMemset(g_tail_counters, 0, 2 * kTailMaxTiles * sizeof(uint32_t)));
      });
      g.tail_first = pair_tiles - tail;
      g.tail_slices = slices;
      g.tail_kb = per;
      g.num_items = g.tail_first + tail * slices;
      g.tail_ws = g_tail_ws;
      g.tail_counters = g_tail_counters;
      split = true;                                         // slices of a tile wait for one another: co-residency
    }
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads + 32 * Policy::kReducerWarps);
  cfg.dynamicSmemBytes = kSmemBytes2;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = 2; attrs[0].val.clusterDim.y = 1; attrs[0].val.clusterDim.z = 1;
  attrs[1].id = cudaLaunchAttributeCooperative;
  attrs[1].val.cooperative = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = (cooperative || split) && cooperative_launches() ? 2 : 1;
  PCCL_CUDA(cudaLaunchKernelEx(&cfg, kernel, ta, tb, g, params));
}

}  // namespace

uint32_t* error_word() {
  std::call_once(g_error_once, [] {
    PCCL_CUDA(cudaMalloc(reinterpret_cast<void**>(&g_error), sizeof(uint32_t)));
    PCCL_CUDA(cudaMemset(g_error, 0, sizeof(uint32_t)));
  });
  return g_error;
}

void gemm_trace_enable(bool on) {
  if (on && !g_trace) PCCL_CUDA(cudaMalloc(reinterpret_cast<void**>(&g_trace), kTraceCtas * kGemmTraceStamps * sizeof(uint64_t)));
  if (on) PCCL_CUDA(cudaMemset(g_trace, 0, kTraceCtas * kGemmTraceStamps * sizeof(uint64_t)));
  if (!on && g_trace) { cudaFree(g_trace); g_trace = nullptr; }
}

std::vector<uint64_t> gemm_trace_read() {
  std::vector<uint64_t> out;
  if (!g_trace) return out;
  out.resize(kTraceCtas * kGemmTraceStamps);
  PCCL_CUDA(cudaMemcpy(out.data(), g_trace, out.size() * sizeof(uint64_t), cudaMemcpyDeviceToHost));
  return out;
}

uint32_t read_error() {
  uint32_t v = 0;
  PCCL_CUDA(cudaMemcpy(&v, error_word(), sizeof v, cudaMemcpyDeviceToHost));
  return v;
}

void clear_error() {
  PCCL_CUDA(cudaMemset(error_word(), 0, sizeof(uint32_t)));
  // A launch that gave up may have left the split tail's counters mid-count.
  if (g_tail_counters) PCCL_CUDA(cudaMemset(g_tail_counters, 0, 2 * kTailMaxTiles * sizeof(uint32_t)));
}

void gemm_bf16_nt(const MatrixDesc& a, const MatrixDesc& b, void* c, int64_t ldc, cudaStream_t stream, int ctas,
                  uint64_t timeout_ms, int sms_per_tile) {
  PCCL_CHECK(ldc % 8 == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0, "GEMM: C must be 16-byte aligned rows");
  PCCL_CHECK(sms_per_tile >= 0 && sms_per_tile <= 2, "GEMM: sms_per_tile is 0 (default), 1 or 2");
  StorePolicy::Params p{static_cast<__nv_bfloat16*>(c), ldc};
  if (sms_per_tile == 0) sms_per_tile = static_cast<int>(Environs::get_int("PCCL_GEMM_SMS_PER_TILE", 2));
  // A single 128-row block gains nothing from pairing two SMs.
  if (sms_per_tile == 2 && a.rows > kBM) launch_pair<StorePolicy>(a, b, p, ctas, timeout_ms, stream, false);
  else launch<StorePolicy>(a, b, p, ctas, timeout_ms, stream);
}

namespace {
PeerView to_view(const PeerBases& b) {
  PeerView v{};
  for (int r = 0; r < b.world; ++r) v.base[r] = b.base[r];
  v.rank = b.rank;
  v.world = b.world;
  return v;
}
}  // namespace

void gemm_reduce_scatter(const PeerBases& peers, const MatrixDesc& x, const MatrixDesc& w, uint64_t recv_off,
                         uint64_t flags_off, uint32_t* block_counter, void* out, int64_t ldo, uint32_t epoch,
                         cudaStream_t stream, int ctas, uint64_t timeout_ms) {
  PCCL_CHECK(x.rows % peers.world == 0, "GEMM->RS: M must divide by the world size");
  const int rows_per_rank = x.rows / peers.world;
  PCCL_CHECK(rows_per_rank % kBM == 0, "GEMM->RS: rows per rank must be a multiple of " << kBM);
  PCCL_CHECK(w.rows % 8 == 0 && ldo % 8 == 0, "GEMM->RS: N and the output stride must be multiples of 8");
  PCCL_CHECK(epoch >= 1, "GEMM->RS: epoch counts calls from 1");
  ReduceScatterPolicy::Params p{};
  p.peers = to_view(peers);
  p.recv_off = recv_off;
  p.flags_off = flags_off;
  p.block_counter = block_counter;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.rows_per_rank = rows_per_rank;
  p.blocks_per_rank = rows_per_rank / kBM;
  p.epoch = epoch;
  // Pairs of SMs on 256-row blocks when every rank's rows split into whole pairs of blocks.
  if (Environs::get_int("PCCL_GEMM_SMS_PER_TILE", 2) == 2 && p.blocks_per_rank % 2 == 0)
    launch_pair<ReduceScatterPolicy>(x, w, p, ctas, timeout_ms, stream, true);
  else
    launch<ReduceScatterPolicy>(x, w, p, ctas, timeout_ms, stream);
}

void all_gather_gemm(const PeerBases& peers, uint64_t gathered_off, int M, int K, const MatrixDesc& w,
                     uint64_t flags_off, uint32_t* ready, void* out, int64_t ldc, uint32_t epoch,
                     cudaStream_t stream, int copy_ctas, int ctas, uint64_t timeout_ms, bool swiglu) {
  PCCL_CHECK(!swiglu || w.rows % 32 == 0, "AG->GEMM with SwiGLU: gate and up rows come in groups of 16 each");
  PCCL_CHECK(M % peers.world == 0 && (M / peers.world) % kBM == 0,
             "AG->GEMM: rows per rank must be a multiple of " << kBM);
  PCCL_CHECK(epoch >= 1, "AG->GEMM: epoch counts calls from 1");
  AllGatherPolicy::Params p{};
  p.peers = to_view(peers);
  p.gathered_off = gathered_off;
  p.flags_off = flags_off;
  p.ready = ready;
  p.c = static_cast<__nv_bfloat16*>(out);
  p.ldc = ldc;
  p.rows_per_rank = M / peers.world;
  p.blocks_per_rank = p.rows_per_rank / kBM;
  // Copier CTAs: by default the SMs that the GEMM tiles leave idle (at least 16, at most 48).  A block
  // is cut into copiers / 4 parts, so that about four row blocks are in flight at a time and blocks
  // complete in the order the GEMM needs them.
  const int sms = sm_count();
  const int remote_blocks = (peers.world - 1) * p.blocks_per_rank;
  if (peers.world == 1) {
    p.copy_ctas = 0;
    p.copy_parts = 1;
  } else {
    const int tiles = ((M + kBM - 1) / kBM) * ((w.rows + kBN - 1) / kBN);
    // More tiles than SMs: the GEMM runs several waves and the copy must keep ahead of it: 32 SMs with
    // 128 KB in flight each cover the link's bandwidth-delay product twice over.
    int want = copy_ctas > 0 ? copy_ctas : (tiles >= sms ? 32 : std::min(48, std::max(16, sms - tiles)));
    want &= ~1;                                           // whole clusters for the paired kernel
    if (want < 2) want = 2;
    p.copy_parts = std::max(1, want / 4);
    if (remote_blocks * p.copy_parts < want) want = std::max(2, (remote_blocks * p.copy_parts + 1) & ~1);
    p.copy_ctas = want;
  }
  p.epoch = epoch;
  MatrixDesc a{peers.base[peers.rank] + gathered_off, M, K, K};
  int grid = ctas > 0 ? ctas : sms;
  const bool pair = Environs::get_int("PCCL_GEMM_SMS_PER_TILE", 2) == 2 && p.blocks_per_rank % 2 == 0 &&
                    p.copy_ctas % 2 == 0;
  if (swiglu) {
    if (pair) launch_pair<AllGatherSwigluPolicy>(a, w, p, grid, timeout_ms, stream, true, p.copy_ctas);
    else launch<AllGatherSwigluPolicy>(a, w, p, grid, timeout_ms, stream, p.copy_ctas);
  } else {
    if (pair) launch_pair<AllGatherPolicy>(a, w, p, grid, timeout_ms, stream, true, p.copy_ctas);
    else launch<AllGatherPolicy>(a, w, p, grid, timeout_ms, stream, p.copy_ctas);
  }
}

namespace {
// SMs per tile of the expert GEMMs: 2 (SM pairs, the default) or 1; read per call so that tests can flip it.
int moe_sms_per_tile() { return Environs::get_int("PCCL_GEMM_SMS_PER_TILE", 2) == 1 ? 1 : 2; }

MoeShape moe_shape(const PeerBases& peers, const MoeBuffers& buf, int local_experts, bool wait_ready, uint32_t epoch) {
  PCCL_CHECK(buf.cap > 0 && buf.cap % kBM == 0, "MoE: region capacity must be a multiple of " << kBM);
  PCCL_CHECK(local_experts * peers.world <= kMoeMaxRegions,
             "MoE: local experts x world exceeds " << kMoeMaxRegions << " regions");
  PCCL_CHECK(epoch >= 1, "MoE: epoch counts calls from 1");
  MoeShape s{};
  uint8_t* self = peers.base[peers.rank];
  s.counts = reinterpret_cast<const uint32_t*>(self + buf.counts_off);
  s.ready = reinterpret_cast<const uint32_t*>(self + buf.ready_off);
  s.world = peers.world;
  s.local_experts = local_experts;
  s.cap_blocks = buf.cap / kBM;
  s.wait_ready = wait_ready ? 1 : 0;
  s.epoch = epoch;
  return s;
}
}  // namespace

void moe_expert_up(const PeerBases& peers, const MoeBuffers& buf, int hidden, int ffn, int local_experts,
                   const void* w13, void* h, uint32_t epoch, cudaStream_t stream, int ctas, uint64_t timeout_ms) {
  PCCL_CHECK(ffn % 16 == 0 && hidden % 8 == 0, "MoE: ffn must be a multiple of 16, hidden of 8");
  MoeUpPolicy::Params p{};
  p.shape = moe_shape(peers, buf, local_experts, true, epoch);
  p.h = static_cast<__nv_bfloat16*>(h);
  p.ldh = ffn;
  const int rows = local_experts * peers.world * buf.cap;
  MatrixDesc a{peers.base[peers.rank] + buf.recv_off, rows, hidden, hidden};
  MatrixDesc b{w13, local_experts * 2 * ffn, hidden, hidden};
  if (moe_sms_per_tile() == 2) launch_pair<MoeUpPolicy>(a, b, p, ctas, timeout_ms, stream, true, 0, local_experts);
  else launch<MoeUpPolicy>(a, b, p, ctas, timeout_ms, stream, 0, local_experts);
}

void moe_expert_down(const PeerBases& peers, const MoeBuffers& buf, int tokens, int hidden, int ffn,
                     int local_experts, const void* h, const void* w2, void* out, uint32_t* cta_counter,
                     uint32_t epoch, cudaStream_t stream, int ctas, uint64_t timeout_ms) {
  PCCL_CHECK(hidden % 8 == 0 && ffn % 8 == 0, "MoE: hidden and ffn must be multiples of 8");
  MoeDownPolicy::Params p{};
  p.shape = moe_shape(peers, buf, local_experts, false, epoch);
  p.peers = to_view(peers);
  p.meta_off = buf.meta_off;
  p.comb_off = buf.comb_off;
  p.done_off = buf.done_off;
  p.cta_counter = cta_counter;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.tokens = tokens;
  const int rows = local_experts * peers.world * buf.cap;
  MatrixDesc a{h, rows, ffn, ffn};
  MatrixDesc b{w2, local_experts * hidden, ffn, ffn};
  if (moe_sms_per_tile() == 2) launch_pair<MoeDownPolicy>(a, b, p, ctas, timeout_ms, stream, true, 0, local_experts);
  else launch<MoeDownPolicy>(a, b, p, ctas, timeout_ms, stream, 0, local_experts);
}

}  // namespace gemm
}  // namespace pccl
