// libkvskip_b200: C ABI over the sm_100a kernels (see include/kvskip_b200.h).
// Single translation unit: the kernels live in the .cuh files included below.
#include "../../include/kvskip_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <set>
#include <string>
#include <utility>

#include "common.cuh"
#include "decode_exact.cuh"
#include "decode_tc.cuh"
#include "decode_tcq.cuh"
#include "planner.cuh"
#include "vskip.cuh"
#include "vskip_tc.cuh"
#include "pv_tc.cuh"

namespace {

thread_local std::string t_error;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  t_error = buf;
  return code;
}

#define KVB_CUDA(expr)                                                                       \
  do {                                                                                       \
    cudaError_t e_ = (expr);                                                                 \
    if (e_ != cudaSuccess) return fail(KVSKIP_E_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

// Opt a kernel into its dynamic shared-memory size once per (device, kernel).
int ensure_smem(const void* func, int bytes) {
  static std::mutex mu;
  static std::set<std::pair<int, const void*>> done;
  int dev = 0;
  KVB_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  if (done.count({dev, func})) return KVSKIP_OK;
  KVB_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  done.insert({dev, func});
  return KVSKIP_OK;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// 4-D map over a [B,Hkv,T,D] bf16 view (element strides sb, sh, st; D contiguous); one box is
// box_d dims x 64 tokens of one (b, head).  Rows at or beyond T read as zero.
int make_kv_map(CUtensorMap* map, const void* base, int64_t sb, int64_t sh, int64_t st, int B, int Hkv, int T,
                int D, int box_d, CUtensorMapSwizzle swz) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return fail(KVSKIP_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if (reinterpret_cast<uintptr_t>(base) % 16) return fail(KVSKIP_E_ARG, "k / v must be 16-byte aligned");
  if (st % 8 || sh % 8 || sb % 8) return fail(KVSKIP_E_ARG, "k / v strides must be multiples of 8 elements");
  // a size-1 dim may carry any stride (even 0); give the map a valid one
  if (T == 1 && st < D) st = D;
  if (Hkv == 1 && sh <= 0) sh = static_cast<int64_t>(T) * st;
  if (B == 1 && sb <= 0) sb = static_cast<int64_t>(Hkv) * (sh > 0 ? sh : 8);
  if (st <= 0 || sh <= 0 || sb <= 0) return fail(KVSKIP_E_ARG, "k / v strides must be positive");
  const cuuint64_t gdim[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(Hkv),
                              static_cast<cuuint64_t>(B)};
  const cuuint64_t gstr[3] = {static_cast<cuuint64_t>(st) * 2, static_cast<cuuint64_t>(sh) * 2,
                              static_cast<cuuint64_t>(sb) * 2};
  const cuuint32_t box[4] = {static_cast<cuuint32_t>(box_d), KVSKIP_TILE, 1, 1};
  const cuuint32_t est[4] = {1, 1, 1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), gdim, gstr, box, est,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(KVSKIP_E_CUDA, "cuTensorMapEncodeTiled failed (%d) for strides %lld/%lld/%lld dims %d/%d/%d/%d",
                static_cast<int>(r), static_cast<long long>(sb), static_cast<long long>(sh),
                static_cast<long long>(st), B, Hkv, T, D);
  return KVSKIP_OK;
}

int check_common(const kvskip_params* p, int D, int G) {
  if (!p) return fail(KVSKIP_E_ARG, "null parameter block");
  if (G != 4) return fail(KVSKIP_E_ARG, "kvskip: only G = 4 query heads per KV head are instantiated");
  if (D != 64 && D != 128) return fail(KVSKIP_E_ARG, "kvskip: unsupported head dim");
  if (p->B < 1 || p->Hkv < 1 || p->T < 1 || p->Hq != p->Hkv * G) return fail(KVSKIP_E_ARG, "bad B / Hq / Hkv / T");
  if (p->num_splits < 1) return fail(KVSKIP_E_ARG, "num_splits >= 1");
  if (p->B > 65535 || p->Hkv > 65535) return fail(KVSKIP_E_LIMIT, "B and Hkv are grid dims: at most 65535");
  return KVSKIP_OK;
}

template <int D, bool MASKED, bool STATS, bool LOAD_V>
int launch_exact(const kvskip_params& p, cudaStream_t stream) {
  using Cfg = kvb::ExactCfg<D, LOAD_V>;
  auto kernel = kvb::decode_exact_kernel<D, MASKED, STATS, LOAD_V>;
  if (int rc = ensure_smem(reinterpret_cast<const void*>(kernel), Cfg::kSmemBytes)) return rc;
  kvb::TmaMaps maps;
  if (int rc = make_kv_map(&maps.k, p.k, p.k_sb, p.k_sh, p.k_st, p.B, p.Hkv, p.T, D, D, CU_TENSOR_MAP_SWIZZLE_NONE))
    return rc;
  if (LOAD_V) {
    if (int rc = make_kv_map(&maps.v, p.v, p.v_sb, p.v_sh, p.v_st, p.B, p.Hkv, p.T, D, D, CU_TENSOR_MAP_SWIZZLE_NONE))
      return rc;
  } else {
    maps.v = maps.k;
  }
  const dim3 grid(p.num_splits, p.Hkv, p.B);
  kernel<<<grid, kvb::EX_THREADS, Cfg::kSmemBytes, stream>>>(p, maps);
  KVB_CUDA(cudaGetLastError());
  if (LOAD_V && p.num_splits > 1) {
    kvb::merge_kernel<D><<<p.B * p.Hq, D, 0, stream>>>(p.part_acc, p.part_ml, p.num_splits,
                                                        static_cast<int64_t>(p.B) * p.Hq, true, p.out, p.out_f32,
                                                        p.lse);
    KVB_CUDA(cudaGetLastError());
  }
  return KVSKIP_OK;
}

std::atomic<int> g_use_pdl{1};

// Launch that lets the kernel's prologue overlap the tail of the previous kernel on the stream
// (programmatic dependent launch).  Only for kernels that execute griddepcontrol.wait before
// their first read of global memory.
template <typename... KArgs, typename... Args>
cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_use_pdl.load(std::memory_order_relaxed) ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with the CTAs along x grouped into clusters of `cluster` (gridDim.x a multiple of it).
template <typename... KArgs, typename... Args>
cudaError_t launch_overlapped_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, unsigned cluster, size_t smem,
                                      cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_use_pdl.load(std::memory_order_relaxed) ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cluster;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Counters of finished splits for the in-kernel merge: zero at load, put back to zero by the CTA
// that merges.  A region of counters belongs to a (device, stream) pair: launches on one stream run
// one after the other (a dependent launch touches its counters only after griddepcontrol.wait), so
// they can share a region, and launches on different streams never do.  A kernel captured into a
// CUDA graph keeps the region of the stream it was captured on.  Regions are handed out on first
// use and never taken back; a device that has seen more than kMergeRegions streams gets no region
// for the newcomers (the attention kernels then merge with a second launch, plan reports a limit).
constexpr int kMergeRegion = 4096;
constexpr int kMergeRegions = 64;
constexpr int kMaxDevices = 64;
__device__ int g_split_done[kMergeRegion * kMergeRegions];
std::atomic<int> g_half_cta{1};
// Block lists on more CTAs than SMs: 1 = one persistent CTA per SM pulling pieces from a queue
// (decode_tcq.cuh), 0 = one CTA per piece (decode_tc.cuh).  Same bits either way.
std::atomic<int> g_queue{1};
std::atomic<int> g_queue_min_heads{32};   // fewest (batch, kv head) pairs of a launch that takes the queue kernel
std::atomic<int> g_plan_rounds{0};     // 32-block rounds per CTA of `plan` (counter version): 1, 2, 4, 8, or 0 = chosen per launch
std::atomic<int> g_plan_cluster{-1};   // CTAs per head of `plan` on a cluster: 1, 2, 4, 8; -1 = chosen per launch; 0 = counter version
std::atomic<int> g_min_blocks{24};     // shortest piece a block list is cut into when there are more CTAs than SMs
// Polls (of about 100 ns) a kernel spends on a peer's flag before it gives up: about 2 s by default.
// The "spin_limit" option lowers it, so that a missing peer is reported in microseconds (tests of the
// failure path; a host that prefers a fast error over a long wait).
constexpr int kDefaultSpin = 1 << 21;
std::atomic<int> g_xchg_spin{kDefaultSpin};

int split_done_region(int units, cudaStream_t stream, int** out) {
  static std::mutex mu;
  static int* base[kMaxDevices] = {};
  static cudaStream_t owner[kMaxDevices][kMergeRegions];
  static int used[kMaxDevices] = {};
  *out = nullptr;
  if (units > kMergeRegion) return KVSKIP_OK;          // too many (batch, head) pairs: separate merge launch
  int dev = 0;
  KVB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return KVSKIP_OK;
  std::lock_guard<std::mutex> lock(mu);
  if (!base[dev]) {
    void* ptr = nullptr;
    KVB_CUDA(cudaGetSymbolAddress(&ptr, g_split_done));
    base[dev] = static_cast<int*>(ptr);
  }
  int r = 0;
  while (r < used[dev] && owner[dev][r] != stream) ++r;
  if (r == used[dev]) {
    if (used[dev] == kMergeRegions) return KVSKIP_OK;
    owner[dev][used[dev]++] = stream;
  }
  *out = base[dev] + r * kMergeRegion;
  return KVSKIP_OK;
}

// What the _dyn and _paged entry points add to a launch: the length on the device, a page table.
struct DynArgs {
  const int* t_dev = nullptr;
  const int32_t* pages = nullptr;   // [B, max_pages] page of every 64-token block
  int max_pages = 0;
  int num_pages = 0;                // pages in the pool
  kvb::XchgArgs xa{};               // R > 0: cross-GPU exchange inside the kernel (sequence shards)
};

template <int NC, bool MASKED, bool STATS, bool LOAD_V, int D>
int launch_tc_nc(const kvskip_params& p, const kvb::TmaMaps& maps, int* done, int min_blocks, const DynArgs& dyn,
                 cudaStream_t stream) {
  using Cfg = kvb::TcCfg<NC, LOAD_V, D>;
  auto kernel = kvb::decode_tc_kernel<NC, MASKED, STATS, LOAD_V, D>;
  if (int rc = ensure_smem(reinterpret_cast<const void*>(kernel), Cfg::kSmemBytes)) return rc;
  KVB_CUDA(launch_overlapped(kernel, dim3(p.num_splits, p.Hkv, p.B), dim3(Cfg::kThreads), Cfg::kSmemBytes, stream, p,
                             maps, done, min_blocks, dyn.t_dev, dyn.pages, dyn.max_pages, dyn.xa));
  return KVSKIP_OK;
}

template <bool MASKED, bool STATS, bool LOAD_V, int D = 128>
int launch_tc(const kvskip_params& p, const DynArgs& dyn, cudaStream_t stream) {
  kvb::TmaMaps maps;
  // contiguous cache: (D, T, Hkv, B); paged cache: (D, 64, Hkv, pages) over the pool
  const int map_b = dyn.pages ? dyn.num_pages : p.B, map_t = dyn.pages ? KVSKIP_TILE : p.T;
  if (int rc = make_kv_map(&maps.k, p.k, p.k_sb, p.k_sh, p.k_st, map_b, p.Hkv, map_t, D, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  if (LOAD_V) {
    if (int rc = make_kv_map(&maps.v, p.v, p.v_sb, p.v_sh, p.v_st, map_b, p.Hkv, map_t, D, 64, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  } else {
    maps.v = maps.k;
  }
  int sms = 148;
  {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int64_t total = static_cast<int64_t>(p.num_splits) * p.Hkv * p.B;
  int* done = nullptr;
  if (LOAD_V && p.num_splits > 1)
    if (int rc = split_done_region(p.B * p.Hkv, stream, &done)) return rc;
  if (dyn.xa.R > 0 && (!LOAD_V || done == nullptr || 2 * p.B * p.Hkv > sms))
    return fail(KVSKIP_E_ARG,
                "exchange inside the kernel: needs V, num_splits > 1 and at most half as many (batch, kv head) "
                "pairs as SMs (the CTAs that wait for their peers must leave room for the others)");
  // With more CTAs than SMs a short block list is cut into pieces of at least 24 blocks.  A dense
  // launch of four or more waves uses the half-size CTA (two per SM), so that set-up and merge of
  // one overlap the other's streaming; with a block list, where many CTAs leave at once and the
  // rest differ in length, the full-size CTA measured faster.
  const bool multi_wave =
      !MASKED && total >= 4 * static_cast<int64_t>(sms) && g_half_cta.load(std::memory_order_relaxed);
  const int min_blocks = (total > sms) ? g_min_blocks.load(std::memory_order_relaxed) : 1;
  if constexpr (MASKED && LOAD_V && D == 128) {
    // more pieces than SMs: persistent CTAs fed from a queue (the last counter of the stream's
    // region is the queue head)
    // (from 32 heads on: below that the pieces of a launch are fewer than the SMs and a CTA per piece
    // starts sooner than the queue)
    if (total > sms && done != nullptr && dyn.xa.R == 0 && p.B * p.Hkv >= g_queue_min_heads.load(std::memory_order_relaxed) &&
        p.B * p.Hkv <= kvb::TcqCfg::kMaxHeads && g_queue.load(std::memory_order_relaxed)) {
      auto kernel = kvb::decode_tcq_kernel<MASKED, STATS>;
      if (int rc = ensure_smem(reinterpret_cast<const void*>(kernel), kvb::TcqCfg::kSmemBytes)) return rc;
      const int ctas = static_cast<int>(std::min<int64_t>(sms, total));
      KVB_CUDA(launch_overlapped(kernel, dim3(ctas), dim3(kvb::TcqCfg::kThreads), kvb::TcqCfg::kSmemBytes, stream, p,
                                 maps, done, done + (kMergeRegion - 1), min_blocks, dyn.t_dev, dyn.pages,
                                 dyn.max_pages));
      return KVSKIP_OK;
    }
  }
  if (int rc = multi_wave ? launch_tc_nc<3, MASKED, STATS, LOAD_V, D>(p, maps, done, min_blocks, dyn, stream)
                          : launch_tc_nc<6, MASKED, STATS, LOAD_V, D>(p, maps, done, min_blocks, dyn, stream))
    return rc;
  if (LOAD_V && p.num_splits > 1 && done == nullptr) {   // no device counters for this launch: merge as a second kernel
    kvb::tc_merge_kernel<D><<<p.B * p.Hq, D, 0, stream>>>(p.part_acc, p.part_ml, p.num_splits, p.out, p.out_f32, p.lse);
    KVB_CUDA(cudaGetLastError());
  }
  return KVSKIP_OK;
}

template <int D>
int dispatch_tc(const kvskip_params& p, bool masked, bool stats, bool load_v, const DynArgs& dyn, cudaStream_t s) {
  if (!masked && !stats && load_v) return launch_tc<false, false, true, D>(p, dyn, s);
  if (!masked && stats && load_v) return launch_tc<false, true, true, D>(p, dyn, s);
  if (!masked && stats && !load_v) return launch_tc<false, true, false, D>(p, dyn, s);
  if (masked && !stats && load_v) return launch_tc<true, false, true, D>(p, dyn, s);
  if (masked && stats && load_v) return launch_tc<true, true, true, D>(p, dyn, s);
  if (masked && stats && !load_v) return launch_tc<true, true, false, D>(p, dyn, s);
  return fail(KVSKIP_E_ARG, "kvskip: unsupported flag combination (load_v=false needs stats=true)");
}

std::atomic<int> g_decode_path{0};   // 0 auto (tensor-core path where it exists), 1 exact-order, 2 tensor-core

template <int D>
int dispatch_exact(const kvskip_params& p, bool masked, bool stats, bool load_v, cudaStream_t s) {
  if (!masked && !stats && load_v) return launch_exact<D, false, false, true>(p, s);
  if (!masked && stats && load_v) return launch_exact<D, false, true, true>(p, s);
  if (!masked && stats && !load_v) return launch_exact<D, false, true, false>(p, s);
  if (masked && !stats && load_v) return launch_exact<D, true, false, true>(p, s);
  if (masked && stats && load_v) return launch_exact<D, true, true, true>(p, s);
  if (masked && stats && !load_v) return launch_exact<D, true, true, false>(p, s);
  return fail(KVSKIP_E_ARG, "kvskip: unsupported flag combination (load_v=false needs stats=true)");
}

template <int D>
int launch_vskip1_t(const kvskip_params& p, cudaStream_t stream) {
  using Cfg = kvb::Vskip1Cfg<D>;
  auto kernel = kvb::vskip1_kernel<D>;
  if (int rc = ensure_smem(reinterpret_cast<const void*>(kernel), Cfg::kSmemBytes)) return rc;
  kvb::TmaMaps maps;
  if (int rc = make_kv_map(&maps.k, p.k, p.k_sb, p.k_sh, p.k_st, p.B, p.Hkv, p.T, D, D, CU_TENSOR_MAP_SWIZZLE_NONE))
    return rc;
  if (int rc = make_kv_map(&maps.v, p.v, p.v_sb, p.v_sh, p.v_st, p.B, p.Hkv, p.T, D, D, CU_TENSOR_MAP_SWIZZLE_NONE))
    return rc;
  kernel<<<dim3(p.num_splits, p.Hkv, p.B), kvb::EX_THREADS, Cfg::kSmemBytes, stream>>>(p, maps);
  KVB_CUDA(cudaGetLastError());
  if (p.num_splits > 1) {
    kvb::merge_kernel<D><<<p.B * p.Hq, D, 0, stream>>>(p.part_acc, p.part_ml, p.num_splits,
                                                        static_cast<int64_t>(p.B) * p.Hq, true, p.out, p.out_f32,
                                                        p.lse);
    KVB_CUDA(cudaGetLastError());
  }
  return KVSKIP_OK;
}

int launch_vskip1_tc(const kvskip_params& p, const DynArgs& dyn, cudaStream_t stream) {
  auto kernel = kvb::vskip1_tc_kernel;
  if (int rc = ensure_smem(reinterpret_cast<const void*>(kernel), kvb::Vs1TcCfg::kSmemBytes)) return rc;
  kvb::TmaMaps maps;
  const int map_b = dyn.pages ? dyn.num_pages : p.B, map_t = dyn.pages ? KVSKIP_TILE : p.T;
  if (int rc = make_kv_map(&maps.k, p.k, p.k_sb, p.k_sh, p.k_st, map_b, p.Hkv, map_t, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  if (int rc = make_kv_map(&maps.v, p.v, p.v_sb, p.v_sh, p.v_st, map_b, p.Hkv, map_t, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  int* done = nullptr;
  if (p.num_splits > 1)
    if (int rc = split_done_region(p.B * p.Hkv, stream, &done)) return rc;
  KVB_CUDA(launch_overlapped(kernel, dim3(p.num_splits, p.Hkv, p.B), dim3(kvb::TC_THREADS),
                             kvb::Vs1TcCfg::kSmemBytes, stream, p, maps, done, dyn.pages, dyn.max_pages, dyn.t_dev));
  if (p.num_splits > 1 && done == nullptr) {
    kvb::merge_kernel<128><<<p.B * p.Hq, 128, 0, stream>>>(p.part_acc, p.part_ml, p.num_splits,
                                                          static_cast<int64_t>(p.B) * p.Hq, true, p.out, p.out_f32,
                                                          p.lse);
    KVB_CUDA(cudaGetLastError());
  }
  return KVSKIP_OK;
}

int launch_pv_tc(const kvskip_params& p, const int* t_dev, cudaStream_t stream) {
  auto kernel = kvb::pv_tc_kernel;
  if (int rc = ensure_smem(reinterpret_cast<const void*>(kernel), kvb::PvTcCfg::kSmemBytes)) return rc;
  kvb::TmaMaps maps;
  if (int rc = make_kv_map(&maps.v, p.v, p.v_sb, p.v_sh, p.v_st, p.B, p.Hkv, p.T, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  maps.k = maps.v;
  int* done = nullptr;
  if (p.num_splits > 1)
    if (int rc = split_done_region(p.B * p.Hkv, stream, &done)) return rc;
  KVB_CUDA(launch_overlapped(kernel, dim3(p.num_splits, p.Hkv, p.B), dim3(kvb::TC_THREADS), kvb::PvTcCfg::kSmemBytes,
                             stream, p, maps, done, t_dev));
  if (p.num_splits > 1 && done == nullptr) {
    kvb::sum_splits_kernel<128><<<p.B * p.Hq, 128, 0, stream>>>(p);
    KVB_CUDA(cudaGetLastError());
  }
  return KVSKIP_OK;
}

template <int D>
int launch_pv_t(const kvskip_params& p, cudaStream_t stream) {
  using Cfg = kvb::PvCfg<D>;
  auto kernel = kvb::pv_kernel<D>;
  if (int rc = ensure_smem(reinterpret_cast<const void*>(kernel), Cfg::kSmemBytes)) return rc;
  kvb::TmaMaps maps;
  if (int rc = make_kv_map(&maps.v, p.v, p.v_sb, p.v_sh, p.v_st, p.B, p.Hkv, p.T, D, D, CU_TENSOR_MAP_SWIZZLE_NONE))
    return rc;
  maps.k = maps.v;
  kernel<<<dim3(p.num_splits, p.Hkv, p.B), kvb::EX_THREADS, Cfg::kSmemBytes, stream>>>(p, maps);
  KVB_CUDA(cudaGetLastError());
  if (p.num_splits > 1) {
    kvb::sum_splits_kernel<D><<<p.B * p.Hq, D, 0, stream>>>(p);
    KVB_CUDA(cudaGetLastError());
  }
  return KVSKIP_OK;
}

}  // namespace

extern "C" {

int kvskip_version(void) { return 100; }

const char* kvskip_last_error(void) { return t_error.c_str(); }

int kvskip_max_smem_bytes(int D, int stages, int load_v) {
  (void)stages;
  if (D == 128) return load_v ? kvb::ExactCfg<128, true>::kSmemBytes : kvb::ExactCfg<128, false>::kSmemBytes;
  if (D == 64) return load_v ? kvb::ExactCfg<64, true>::kSmemBytes : kvb::ExactCfg<64, false>::kSmemBytes;
  return 0;
}

namespace {
int decode_impl(const kvskip_params* p, int D, int G, int stages, int masked, int stats, int load_v, const DynArgs& dyn,
                void* stream) {
  if (int rc = check_common(p, D, G)) return rc;
  if (dyn.pages) {
    if (dyn.num_pages < 1 || dyn.max_pages < (p->T + KVSKIP_TILE - 1) / KVSKIP_TILE)
      return fail(KVSKIP_E_ARG, "paged cache: the page table needs an entry for every block of the sequence");
    if (p->p_out) return fail(KVSKIP_E_ARG, "paged cache: write_p is not supported");
  }
  if (stages != 2 && stages != 3) return fail(KVSKIP_E_ARG, "kvskip: unsupported head dim / stages");
  if (!load_v && !stats) return fail(KVSKIP_E_ARG, "kvskip: unsupported flag combination (load_v=false needs stats=true)");
  if (masked && (!p->block_idx || !p->block_cnt)) return fail(KVSKIP_E_ARG, "masked mode needs block_idx and block_cnt");
  if (stats && (!p->blk_max || !p->blk_sum)) return fail(KVSKIP_E_ARG, "stats mode needs blk_max and blk_sum");
  if (load_v && !p->out) return fail(KVSKIP_E_ARG, "out is required when load_v");
  if (p->num_splits > 1 && (!p->part_ml || (load_v && !p->part_acc)))
    return fail(KVSKIP_E_ARG, "num_splits > 1 needs part_acc / part_ml scratch");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int path = g_decode_path.load(std::memory_order_relaxed);
  // the tensor-core kernel: D = 128, and D = 64 except with write_p (the fp16 P of the two-pass
  // V-skip is written by the D = 128 instantiation and by the exact-order kernels only)
  if (path != 1 && D == 128) return dispatch_tc<128>(*p, masked, stats, load_v, dyn, s);
  if (path != 1 && D == 64 && !p->p_out) {
    if (dyn.xa.R > 0) return fail(KVSKIP_E_ARG, "the exchange inside the kernel exists for D = 128");
    return dispatch_tc<64>(*p, masked, stats, load_v, dyn, s);
  }
  if (dyn.t_dev || dyn.pages)
    return fail(KVSKIP_E_ARG, "a device-resident length or a paged cache needs the tensor-core path (decode_path != 1)");
  if (path == 2) return fail(KVSKIP_E_ARG, "the tensor-core path does not write P for D = 64");
  return D == 128 ? dispatch_exact<128>(*p, masked, stats, load_v, s) : dispatch_exact<64>(*p, masked, stats, load_v, s);
}
}  // namespace

int kvskip_launch_decode(const kvskip_params* p, int D, int G, int stages, int masked, int stats, int load_v,
                         void* stream) {
  return decode_impl(p, D, G, stages, masked, stats, load_v, DynArgs{}, stream);
}

int kvskip_launch_decode_dyn(const kvskip_params* p, int D, int G, int stages, int masked, int stats, int load_v,
                             const int* t_dev, void* stream) {
  if (!t_dev) return fail(KVSKIP_E_ARG, "t_dev is null");
  DynArgs dyn;
  dyn.t_dev = t_dev;
  return decode_impl(p, D, G, stages, masked, stats, load_v, dyn, stream);
}

int kvskip_launch_decode_xchg(const kvskip_params* p, int D, int G, int stages, int masked, int stats,
                              float* const* peer_bufs, unsigned int* const* peer_flags, int rank, int R,
                              unsigned int seq, void* stream) {
  if (!p || !peer_bufs) return fail(KVSKIP_E_ARG, "decode_xchg: null argument");
  if (R < 1 || R > kvb::XCHG_MAX_RANKS || rank < 0 || rank >= R)
    return fail(KVSKIP_E_LIMIT, "decode_xchg: 1..%d ranks", kvb::XCHG_MAX_RANKS);
  if (seq == 0) return fail(KVSKIP_E_ARG, "decode_xchg: seq >= 1");
  DynArgs dyn;
  for (int r = 0; r < R; ++r) {
    if (!peer_bufs[r] || reinterpret_cast<uintptr_t>(peer_bufs[r]) % 8)
      return fail(KVSKIP_E_ARG, "decode_xchg: null or misaligned peer buffer");
    dyn.xa.peers.buf[r] = peer_bufs[r];
    dyn.xa.peers.flags[r] = peer_flags ? peer_flags[r] : nullptr;
  }
  dyn.xa.rank = rank;
  dyn.xa.R = R;
  dyn.xa.N = static_cast<long long>(p->B) * p->Hq;
  dyn.xa.seq = seq;
  dyn.xa.spin = static_cast<unsigned int>(g_xchg_spin.load(std::memory_order_relaxed));
  if (D != 128 || g_decode_path.load(std::memory_order_relaxed) == 1)
    return fail(KVSKIP_E_ARG, "decode_xchg: tensor-core path only (D = 128, decode_path != 1)");
  return decode_impl(p, D, G, stages, masked, stats, 1, dyn, stream);
}

int kvskip_launch_decode_paged(const kvskip_params* p, int D, int G, int stages, int masked, int stats, int load_v,
                               const int32_t* page_table, int max_pages, int num_pages, const int* t_dev,
                               void* stream) {
  if (!page_table) return fail(KVSKIP_E_ARG, "page_table is null");
  DynArgs dyn;
  dyn.t_dev = t_dev;
  dyn.pages = page_table;
  dyn.max_pages = max_pages;
  dyn.num_pages = num_pages;
  return decode_impl(p, D, G, stages, masked, stats, load_v, dyn, stream);
}

// ---- split-K decode for callers that cannot allocate device memory -------------------------
// The split scratch of this entry point: one array per device that loads the library, held
// until the process exits.  Partials of every (row, split) are fully rewritten by each call, so
// nothing in it has to start at zero; it keeps the last call's contents.
static __device__ __align__(256) float g_noalloc_scratch[KVSKIP_NOALLOC_MAX_FLOATS];

namespace {
// device address of g_noalloc_scratch per device ordinal, looked up once with that device current
// (in host code the array's name is only a handle for the runtime, not a device address)
float* g_noalloc_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mu;

int noalloc_scratch(float** out) {
  int dev = 0;
  KVB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(KVSKIP_E_LIMIT, "device ordinal %d beyond %d", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (!g_noalloc_ptr[dev]) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || !ptr)
      return fail(KVSKIP_E_CUDA, "cudaGetSymbolAddress(g_noalloc_scratch): %s", cudaGetErrorString(e));
    g_noalloc_ptr[dev] = static_cast<float*>(ptr);
  }
  *out = g_noalloc_ptr[dev];
  return KVSKIP_OK;
}
}  // namespace

int kvskip_launch_decode_noalloc(const kvskip_params* p, int D, int G, int stages, int masked, int stats, int load_v,
                                 void* stream) {
  if (int rc = check_common(p, D, G)) return rc;
  kvskip_params q = *p;
  q.part_acc = nullptr;
  q.part_ml = nullptr;
  if (q.num_splits > 1) {
    const int64_t rows = static_cast<int64_t>(q.B) * q.Hq * q.num_splits;
    const int64_t need = rows * (D + 2);
    if (need > static_cast<int64_t>(KVSKIP_NOALLOC_MAX_FLOATS))
      return fail(KVSKIP_E_LIMIT,
                  "kvskip_launch_decode_noalloc: B*Hq*num_splits*(D+2) = %lld floats of split scratch exceed the "
                  "built-in %lld; use fewer splits or kvskip_launch_decode with caller scratch",
                  static_cast<long long>(need), static_cast<long long>(KVSKIP_NOALLOC_MAX_FLOATS));
    float* base = nullptr;
    if (int rc = noalloc_scratch(&base)) return rc;
    q.part_acc = base;                 // [B,Hq,S,D]
    q.part_ml = base + rows * D;       // [B,Hq,S,2]
  }
  return kvskip_launch_decode(&q, D, G, stages, masked, stats, load_v, stream);
}

int kvskip_set_option(const char* name, int value) {
  if (!name) return fail(KVSKIP_E_ARG, "null option name");
  if (!std::strcmp(name, "decode_path")) {
    if (value < 0 || value > 2) return fail(KVSKIP_E_ARG, "decode_path: 0 auto, 1 exact-order, 2 tensor-core");
    g_decode_path.store(value, std::memory_order_relaxed);
    return KVSKIP_OK;
  }
  if (!std::strcmp(name, "half_cta")) {
    g_half_cta.store(value ? 1 : 0, std::memory_order_relaxed);
    return KVSKIP_OK;
  }
  if (!std::strcmp(name, "pdl")) {
    g_use_pdl.store(value ? 1 : 0, std::memory_order_relaxed);
    return KVSKIP_OK;
  }
  if (!std::strcmp(name, "queue")) {
    g_queue.store(value ? 1 : 0, std::memory_order_relaxed);
    return KVSKIP_OK;
  }
  if (!std::strcmp(name, "queue_min_heads")) {
    if (value < 1) return fail(KVSKIP_E_ARG, "queue_min_heads: at least 1");
    g_queue_min_heads.store(value, std::memory_order_relaxed);
    return KVSKIP_OK;
  }
  if (!std::strcmp(name, "min_blocks")) {
    if (value < 1 || value > 4096) return fail(KVSKIP_E_ARG, "min_blocks: 1..4096");
    g_min_blocks.store(value, std::memory_order_relaxed);
    return KVSKIP_OK;
  }
  if (!std::strcmp(name, "plan_cluster")) {
    if (value != -1 && value != 0 && value != 1 && value != 2 && value != 4 && value != 8)
      return fail(KVSKIP_E_ARG, "plan_cluster: 1, 2, 4 or 8 CTAs per head, -1 for the per-launch choice, 0 for the counter version");
    g_plan_cluster.store(value, std::memory_order_relaxed);
    return KVSKIP_OK;
  }
  if (!std::strcmp(name, "plan_rounds")) {
    if (value != 0 && value != 1 && value != 2 && value != 4 && value != 8)
      return fail(KVSKIP_E_ARG, "plan_rounds: 1, 2, 4 or 8, or 0 for the per-launch choice");
    g_plan_rounds.store(value, std::memory_order_relaxed);
    return KVSKIP_OK;
  }
  if (!std::strcmp(name, "spin_limit")) {   // 0 restores the default
    if (value < 0) return fail(KVSKIP_E_ARG, "spin_limit: polls >= 1, or 0 for the default");
    g_xchg_spin.store(value ? value : kDefaultSpin, std::memory_order_relaxed);
    return KVSKIP_OK;
  }
  return fail(KVSKIP_E_ARG, "unknown option %s", name);
}

int kvskip_get_option(const char* name) {
  if (name && !std::strcmp(name, "decode_path")) return g_decode_path.load(std::memory_order_relaxed);
  if (name && !std::strcmp(name, "pdl")) return g_use_pdl.load(std::memory_order_relaxed);
  if (name && !std::strcmp(name, "half_cta")) return g_half_cta.load(std::memory_order_relaxed);
  if (name && !std::strcmp(name, "spin_limit")) return g_xchg_spin.load(std::memory_order_relaxed);
  if (name && !std::strcmp(name, "queue")) return g_queue.load(std::memory_order_relaxed);
  if (name && !std::strcmp(name, "min_blocks")) return g_min_blocks.load(std::memory_order_relaxed);
  if (name && !std::strcmp(name, "queue_min_heads")) return g_queue_min_heads.load(std::memory_order_relaxed);
  if (name && !std::strcmp(name, "plan_rounds")) return g_plan_rounds.load(std::memory_order_relaxed);
  if (name && !std::strcmp(name, "plan_cluster")) return g_plan_cluster.load(std::memory_order_relaxed);
  return fail(KVSKIP_E_ARG, "unknown option");
}

int kvskip_launch_vskip1(const kvskip_params* p, int D, int G, void* stream) {
  if (int rc = check_common(p, D, G)) return rc;
  if (!p->out || !p->lse) return fail(KVSKIP_E_ARG, "out and lse are required");
  if (p->num_splits > 1 && (!p->part_ml || !p->part_acc)) return fail(KVSKIP_E_ARG, "num_splits > 1 needs scratch");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (D == 128 && g_decode_path.load(std::memory_order_relaxed) != 1) return launch_vskip1_tc(*p, DynArgs{}, s);
  return D == 128 ? launch_vskip1_t<128>(*p, s) : launch_vskip1_t<64>(*p, s);
}

int kvskip_launch_vskip1_dyn(const kvskip_params* p, int D, int G, const int* t_dev, void* stream) {
  if (int rc = check_common(p, D, G)) return rc;
  if (!t_dev) return fail(KVSKIP_E_ARG, "t_dev is null");
  if (!p->out || !p->lse) return fail(KVSKIP_E_ARG, "out and lse are required");
  if (p->num_splits > 1 && (!p->part_ml || !p->part_acc)) return fail(KVSKIP_E_ARG, "num_splits > 1 needs scratch");
  if (D != 128 || g_decode_path.load(std::memory_order_relaxed) == 1)
    return fail(KVSKIP_E_ARG, "a device-resident length needs the tensor-core path (D = 128, decode_path != 1)");
  DynArgs dyn;
  dyn.t_dev = t_dev;
  return launch_vskip1_tc(*p, dyn, static_cast<cudaStream_t>(stream));
}

int kvskip_launch_vskip1_paged(const kvskip_params* p, int D, int G, const int32_t* page_table, int max_pages,
                               int num_pages, void* stream) {
  if (int rc = check_common(p, D, G)) return rc;
  if (!p->out || !p->lse) return fail(KVSKIP_E_ARG, "out and lse are required");
  if (p->num_splits > 1 && (!p->part_ml || !p->part_acc)) return fail(KVSKIP_E_ARG, "num_splits > 1 needs scratch");
  if (!page_table || num_pages < 1 || max_pages < (p->T + KVSKIP_TILE - 1) / KVSKIP_TILE)
    return fail(KVSKIP_E_ARG, "paged cache: the page table needs an entry for every block of the sequence");
  if (D != 128 || g_decode_path.load(std::memory_order_relaxed) == 1)
    return fail(KVSKIP_E_ARG, "a paged cache needs the tensor-core path (D = 128, decode_path != 1)");
  DynArgs dyn;
  dyn.pages = page_table;
  dyn.max_pages = max_pages;
  dyn.num_pages = num_pages;
  return launch_vskip1_tc(*p, dyn, static_cast<cudaStream_t>(stream));
}

namespace {
int pv_impl(const kvskip_params* p, int D, int G, const int* t_dev, void* stream) {
  if (int rc = check_common(p, D, G)) return rc;
  if (!p->p_in || !p->blk_scale || !p->block_idx || !p->block_cnt || !p->out)
    return fail(KVSKIP_E_ARG, "pv needs p_in, blk_scale, block_idx, block_cnt, out");
  if (p->num_splits > 1 && !p->part_acc) return fail(KVSKIP_E_ARG, "num_splits > 1 needs part_acc scratch");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (D == 128 && g_decode_path.load(std::memory_order_relaxed) != 1) return launch_pv_tc(*p, t_dev, s);
  if (t_dev) return fail(KVSKIP_E_ARG, "a device-resident length needs the tensor-core path (D = 128, decode_path != 1)");
  return D == 128 ? launch_pv_t<128>(*p, s) : launch_pv_t<64>(*p, s);
}
}  // namespace

int kvskip_launch_pv(const kvskip_params* p, int D, int G, void* stream) { return pv_impl(p, D, G, nullptr, stream); }

int kvskip_launch_pv_dyn(const kvskip_params* p, int D, int G, const int* t_dev, void* stream) {
  if (!t_dev) return fail(KVSKIP_E_ARG, "t_dev is null");
  return pv_impl(p, D, G, t_dev, stream);
}

namespace {
int plan_impl(const kvskip_plan_params* p, const DynArgs& dyn, void* stream) {
  if (!p) return fail(KVSKIP_E_ARG, "null parameter block");
  if (p->Hq != 4 * p->Hkv) return fail(KVSKIP_E_ARG, "planner kernels: D = 128, G = 4");
  const int nb = (p->T + KVSKIP_TILE - 1) / KVSKIP_TILE;
  if (nb > p->NBC) return fail(KVSKIP_E_ARG, "block capacity exceeded");
  if (((p->flags == nullptr)) || !p->csum || !p->keep || !p->block_idx || !p->block_cnt || !p->trig || !p->cs_now)
    return fail(KVSKIP_E_ARG, "plan: missing state tensor");
  if (p->B > 65535 || p->Hkv > 65535) return fail(KVSKIP_E_LIMIT, "B and Hkv are grid dims: at most 65535");
  int sms = 148;
  {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  // The cluster version: the CTAs of a head hand their results to the first one through its shared
  // memory (17 bytes per block of the head).  CTAs per head: as many as keep the launch at about
  // four CTAs per SM, and no more than the head has 32-block rounds.
  int cluster = g_plan_cluster.load(std::memory_order_relaxed);
  const int64_t heads = static_cast<int64_t>(p->B) * p->Hkv;
  const int csmem = (17 * nb + 15) & ~15;
  if (cluster != 0 && csmem <= 200 * 1024) {
    if (cluster < 0) {
      cluster = 8;
      while (cluster > 1 && heads * cluster > 4 * static_cast<int64_t>(sms)) cluster /= 2;
    }
    while (cluster > 1 && cluster > (nb + kvb::PL_CHUNK - 1) / kvb::PL_CHUNK) cluster /= 2;
    if (csmem > 40 * 1024)
      if (int rc = ensure_smem(reinterpret_cast<const void*>(kvb::plan_cluster_kernel), 200 * 1024)) return rc;
    KVB_CUDA(launch_overlapped_cluster(kvb::plan_cluster_kernel, dim3(cluster, p->Hkv, p->B), dim3(kvb::PL_THREADS),
                                       static_cast<unsigned>(cluster), csmem, static_cast<cudaStream_t>(stream), *p,
                                       dyn.t_dev, dyn.pages, dyn.max_pages, dyn.num_pages));
    return KVSKIP_OK;
  }
  int* done = nullptr;
  if (int rc = split_done_region(p->B * p->Hkv, static_cast<cudaStream_t>(stream), &done)) return rc;
  if (!done)
    return fail(KVSKIP_E_LIMIT, "plan: more than %d (batch, kv head) pairs per call, or more than %d streams used on this device",
                kMergeRegion, kMergeRegions);
  // A CTA computes the centroid scores of 32 * rounds blocks.  With one round a long context at a
  // large batch is a grid of thousands of short CTAs whose start-up rate bounds the kernel; the
  // rounds double until the grid is down to about four CTAs per SM.
  int rounds = g_plan_rounds.load(std::memory_order_relaxed);
  if (rounds == 0) {
    const int64_t ctas = static_cast<int64_t>((nb + kvb::PL_CHUNK - 1) / kvb::PL_CHUNK) * p->Hkv * p->B;
    rounds = 1;
    while (rounds < 8 && ctas / rounds > 4 * static_cast<int64_t>(sms)) rounds *= 2;
  }
  const int chunk = kvb::PL_CHUNK * rounds;
  const int chunks = (nb + chunk - 1) / chunk;
  const int smem = (nb + 15) & ~15;   // attended flags of one head
  if (smem > 200 * 1024) return fail(KVSKIP_E_LIMIT, "plan: more than %d blocks", 200 * 1024);
  auto launch = [&](auto kernel) -> int {
    if (smem > 40 * 1024)
      if (int rc = ensure_smem(reinterpret_cast<const void*>(kernel), 200 * 1024)) return rc;
    KVB_CUDA(launch_overlapped(kernel, dim3(chunks, p->Hkv, p->B), dim3(kvb::PL_THREADS), smem,
                               static_cast<cudaStream_t>(stream), *p, done, dyn.t_dev, dyn.pages, dyn.max_pages,
                               dyn.num_pages));
    return KVSKIP_OK;
  };
  switch (rounds) {
    case 1: return launch(kvb::plan_kernel<1>);
    case 2: return launch(kvb::plan_kernel<2>);
    case 4: return launch(kvb::plan_kernel<4>);
    default: return launch(kvb::plan_kernel<8>);
  }
}
}  // namespace

int kvskip_launch_plan(const kvskip_plan_params* p, void* stream) { return plan_impl(p, DynArgs{}, stream); }

int kvskip_launch_plan_dyn(const kvskip_plan_params* p, const int* t_dev, void* stream) {
  if (!t_dev) return fail(KVSKIP_E_ARG, "t_dev is null");
  DynArgs dyn;
  dyn.t_dev = t_dev;
  return plan_impl(p, dyn, stream);
}

int kvskip_launch_plan_paged(const kvskip_plan_params* p, const int32_t* page_table, int max_pages, int num_pages,
                             const int* t_dev, void* stream) {
  if (!page_table) return fail(KVSKIP_E_ARG, "page_table is null");
  if (p && (num_pages < 1 || max_pages < (p->T + KVSKIP_TILE - 1) / KVSKIP_TILE))
    return fail(KVSKIP_E_ARG, "paged cache: the page table needs an entry for every block of the sequence");
  DynArgs dyn;
  dyn.t_dev = t_dev;
  dyn.pages = page_table;
  dyn.max_pages = max_pages;
  dyn.num_pages = num_pages;
  return plan_impl(p, dyn, stream);
}

namespace {
int update_impl(const kvskip_update_params* p, const int* t_dev, void* stream) {
  if (!p) return fail(KVSKIP_E_ARG, "null parameter block");
  if (p->Hq != 4 * p->Hkv) return fail(KVSKIP_E_ARG, "planner kernels: D = 128, G = 4");
  const int nb = (p->T + KVSKIP_TILE - 1) / KVSKIP_TILE;
  if (nb > p->NBC) return fail(KVSKIP_E_ARG, "block capacity exceeded");
  if (p->calib && (!p->flags || !p->est)) return fail(KVSKIP_E_ARG, "calibration needs flags and est");
  if (p->aix && !p->idx) return fail(KVSKIP_E_ARG, "aix needs idx");
  const int smem = 2 * kvb::PL_G * nb * static_cast<int>(sizeof(float)) + 2 * nb;
  if (smem > 220 * 1024) return fail(KVSKIP_E_LIMIT, "update: more than %d blocks", 220 * 1024 / 33);
  if (smem > 48 * 1024)
    if (int rc = ensure_smem(reinterpret_cast<const void*>(kvb::update_kernel), 220 * 1024)) return rc;
  KVB_CUDA(launch_overlapped(kvb::update_kernel, dim3(p->Hkv, p->B), dim3(kvb::PL_THREADS), smem,
                             static_cast<cudaStream_t>(stream), *p, t_dev));
  return KVSKIP_OK;
}
}  // namespace

int kvskip_launch_update(const kvskip_update_params* p, void* stream) { return update_impl(p, nullptr, stream); }

int kvskip_launch_update_dyn(const kvskip_update_params* p, const int* t_dev, void* stream) {
  if (!t_dev) return fail(KVSKIP_E_ARG, "t_dev is null");
  return update_impl(p, t_dev, stream);
}

int kvskip_launch_read(const void* x, int64_t bytes, uint32_t* out, int blocks, void* stream) {
  if (!x || !out || bytes % 16 || blocks < 1) return fail(KVSKIP_E_ARG, "read: x, out, bytes %% 16 == 0, blocks >= 1");
  kvb::read_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const uint4*>(x),
                                                                          bytes / 16, out);
  KVB_CUDA(cudaGetLastError());
  return KVSKIP_OK;
}

int kvskip_launch_read_bulk(const void* x, int64_t bytes, uint32_t* out, int blocks, void* stream) {
  if (!x || !out || blocks < 1 || bytes < kvb::RB_PIECE || reinterpret_cast<uintptr_t>(x) % 16)
    return fail(KVSKIP_E_ARG, "read_bulk: x 16-byte aligned, at least %d bytes, blocks >= 1", kvb::RB_PIECE);
  if (int rc = ensure_smem(reinterpret_cast<const void*>(kvb::read_bulk_kernel), kvb::RB_SMEM)) return rc;
  kvb::read_bulk_kernel<<<blocks, 64, kvb::RB_SMEM, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned char*>(x), bytes / kvb::RB_PIECE, out);
  KVB_CUDA(cudaGetLastError());
  return KVSKIP_OK;
}

int kvskip_launch_merge(const float* part_acc, const float* part_ml, int R, int64_t N, int D, uint16_t* out,
                        float* out_f32, float* lse, void* stream) {
  if (!part_acc || !part_ml || R < 1 || N < 1) return fail(KVSKIP_E_ARG, "merge: bad arguments");
  if (N > 2147483647LL) return fail(KVSKIP_E_LIMIT, "merge: too many rows");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (D == 128)
    kvb::merge_kernel<128><<<static_cast<unsigned>(N), 128, 0, s>>>(part_acc, part_ml, R, N, false, out, out_f32, lse);
  else if (D == 64)
    kvb::merge_kernel<64><<<static_cast<unsigned>(N), 64, 0, s>>>(part_acc, part_ml, R, N, false, out, out_f32, lse);
  else
    return fail(KVSKIP_E_ARG, "kvskip: unsupported head dim");
  KVB_CUDA(cudaGetLastError());
  return KVSKIP_OK;
}

int kvskip_launch_pack_partial(const float* out_f32, const float* lse, float* packed, int64_t N, int D, void* stream) {
  if (!out_f32 || !lse || !packed || N < 1 || N > 2147483647LL) return fail(KVSKIP_E_ARG, "pack_partial: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (D == 128)
    kvb::pack_partial_kernel<128><<<static_cast<unsigned>(N), 128, 0, s>>>(out_f32, lse, packed);
  else if (D == 64)
    kvb::pack_partial_kernel<64><<<static_cast<unsigned>(N), 64, 0, s>>>(out_f32, lse, packed);
  else
    return fail(KVSKIP_E_ARG, "kvskip: unsupported head dim");
  KVB_CUDA(cudaGetLastError());
  return KVSKIP_OK;
}

int kvskip_launch_merge_packed(const float* parts, int R, int64_t N, int D, uint16_t* out, float* out_f32, float* lse,
                               void* stream) {
  if (!parts || R < 1 || N < 1 || N > 2147483647LL) return fail(KVSKIP_E_ARG, "merge_packed: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (D == 128)
    kvb::merge_packed_kernel<128><<<static_cast<unsigned>(N), 128, 0, s>>>(parts, R, N, out, out_f32, lse);
  else if (D == 64)
    kvb::merge_packed_kernel<64><<<static_cast<unsigned>(N), 64, 0, s>>>(parts, R, N, out, out_f32, lse);
  else
    return fail(KVSKIP_E_ARG, "kvskip: unsupported head dim");
  KVB_CUDA(cudaGetLastError());
  return KVSKIP_OK;
}

int kvskip_launch_exchange_merge(const float* out_f32, const float* lse, float* const* peer_bufs,
                                 unsigned int* const* peer_flags, int rank, int R, int64_t N, int D, unsigned int seq,
                                 uint16_t* out, float* res_f32, float* res_lse, void* stream) {
  if (!out_f32 || !lse || !peer_bufs) return fail(KVSKIP_E_ARG, "exchange_merge: null argument");
  if (R < 1 || R > kvb::XCHG_MAX_RANKS || rank < 0 || rank >= R)
    return fail(KVSKIP_E_LIMIT, "exchange_merge: 1..%d ranks", kvb::XCHG_MAX_RANKS);
  if (N < 1 || N > 2147483647LL || seq == 0) return fail(KVSKIP_E_ARG, "exchange_merge: N >= 1, seq >= 1");
  kvb::XchgPeers peers{};
  for (int r = 0; r < R; ++r) {
    if (!peer_bufs[r] || reinterpret_cast<uintptr_t>(peer_bufs[r]) % 8)
      return fail(KVSKIP_E_ARG, "exchange_merge: null or misaligned peer buffer");
    peers.buf[r] = peer_bufs[r];
    peers.flags[r] = peer_flags ? peer_flags[r] : nullptr;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (D != 128 && D != 64) return fail(KVSKIP_E_ARG, "kvskip: unsupported head dim");
  {
    // One waiting CTA per row: every CTA of the grid must be resident at once, or a CTA that waits
    // for a peer's row could keep that peer's CTA for another row of this rank off the GPU.
    int dev = 0, sms = 0, per_sm = 0;
    KVB_CUDA(cudaGetDevice(&dev));
    KVB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (D == 128)
      KVB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kvb::exchange_merge_kernel<128>, 128, 0));
    else
      KVB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kvb::exchange_merge_kernel<64>, 64, 0));
    if (N > static_cast<int64_t>(per_sm) * sms)
      return fail(KVSKIP_E_LIMIT, "exchange_merge: %lld rows exceed the %d CTAs this GPU keeps resident at once",
                  static_cast<long long>(N), per_sm * sms);
  }
  if (D == 128)
    kvb::exchange_merge_kernel<128><<<static_cast<unsigned>(N), 128, 0, s>>>(
        out_f32, lse, peers, rank, R, N, seq, static_cast<unsigned int>(g_xchg_spin.load(std::memory_order_relaxed)), out,
        res_f32, res_lse);
  else if (D == 64)
    kvb::exchange_merge_kernel<64><<<static_cast<unsigned>(N), 64, 0, s>>>(
        out_f32, lse, peers, rank, R, N, seq, static_cast<unsigned int>(g_xchg_spin.load(std::memory_order_relaxed)), out,
        res_f32, res_lse);
  else
    return fail(KVSKIP_E_ARG, "kvskip: unsupported head dim");
  KVB_CUDA(cudaGetLastError());
  return KVSKIP_OK;
}

namespace {
int index_blocks_impl(const int64_t* ids, int64_t ids_stride, int n, int T, const int* t_dev, uint8_t* out, int NBC,
                      void* stream) {
  if (!ids || !out || n < 1 || T < 1) return fail(KVSKIP_E_ARG, "index_blocks: bad arguments");
  if ((T + KVSKIP_TILE - 1) / KVSKIP_TILE > NBC) return fail(KVSKIP_E_ARG, "block capacity exceeded");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  KVB_CUDA(cudaMemsetAsync(out, 0, static_cast<size_t>(n) * NBC, s));
  kvb::index_blocks_kernel<<<dim3((T + 255) / 256, n), 256, 0, s>>>(ids, ids_stride, T, out, NBC, t_dev);
  KVB_CUDA(cudaGetLastError());
  return KVSKIP_OK;
}
}  // namespace

int kvskip_launch_index_blocks(const int64_t* ids, int64_t ids_stride, int n, int T, uint8_t* out, int NBC,
                               void* stream) {
  return index_blocks_impl(ids, ids_stride, n, T, nullptr, out, NBC, stream);
}

int kvskip_launch_index_blocks_dyn(const int64_t* ids, int64_t ids_stride, int n, int T_bound, const int* t_dev,
                                   uint8_t* out, int NBC, void* stream) {
  if (!t_dev) return fail(KVSKIP_E_ARG, "t_dev is null");
  return index_blocks_impl(ids, ids_stride, n, T_bound, t_dev, out, NBC, stream);
}

int kvskip_launch_append(uint16_t* k, uint16_t* v, int64_t sb, int64_t sh, int64_t st, const uint16_t* k_new,
                         const uint16_t* v_new, int B, int Hkv, int D, int T, const int* t_dev,
                         const int32_t* page_table, int max_pages, int num_pages, void* stream) {
  if (!k || !v || !k_new || !v_new || B < 1 || Hkv < 1 || T < 1) return fail(KVSKIP_E_ARG, "append: bad arguments");
  if (D % 8 || D < 8 || D > 1024) return fail(KVSKIP_E_ARG, "append: D must be a multiple of 8, at most 1024");
  if ((sb | sh | st) % 8 || (reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                             reinterpret_cast<uintptr_t>(k_new) | reinterpret_cast<uintptr_t>(v_new)) % 16)
    return fail(KVSKIP_E_ARG, "append: 16-byte aligned rows (strides multiples of 8 elements)");
  if (B > 65535) return fail(KVSKIP_E_LIMIT, "B is a grid dim: at most 65535");
  if (page_table && (num_pages < 1 || max_pages < (T + KVSKIP_TILE - 1) / KVSKIP_TILE))
    return fail(KVSKIP_E_ARG, "paged cache: the page table needs an entry for every block of the sequence");
  kvb::append_kernel<<<dim3(Hkv, B), D / 8, 0, static_cast<cudaStream_t>(stream)>>>(
      k, v, sb, sh, st, k_new, v_new, D, T, t_dev, page_table, max_pages, num_pages);
  KVB_CUDA(cudaGetLastError());
  return KVSKIP_OK;
}

namespace {
int select_impl(const float* blk_max, const float* blk_sum, int B, int Hkv, int nb, int rule, float value, int local,
                uint8_t* keep, int32_t* block_idx, int32_t* block_cnt, float* weight, const int* t_dev, int T_bound,
                void* stream) {
  if (!blk_max || !blk_sum || !keep || !block_idx || !block_cnt || !weight || B < 1 || Hkv < 1 || nb < 1)
    return fail(KVSKIP_E_ARG, "select: bad arguments");
  if (rule != 0 && rule != 1) return fail(KVSKIP_E_ARG, "select: rule 0 (top-p) or 1 (tau)");
  if (B > 65535) return fail(KVSKIP_E_LIMIT, "B is a grid dim: at most 65535");
  const int smem = 2 * kvb::PL_G * nb * static_cast<int>(sizeof(float)) + nb;
  if (smem > 220 * 1024) return fail(KVSKIP_E_LIMIT, "select: more than %d blocks", 220 * 1024 / 33);
  if (smem > 48 * 1024)
    if (int rc = ensure_smem(reinterpret_cast<const void*>(kvb::select_kernel), 220 * 1024)) return rc;
  KVB_CUDA(launch_overlapped(kvb::select_kernel, dim3(Hkv, B), dim3(kvb::PL_THREADS), smem,
                             static_cast<cudaStream_t>(stream), blk_max, blk_sum, nb, Hkv, rule, value, local, keep,
                             block_idx, block_cnt, weight, t_dev, T_bound));
  return KVSKIP_OK;
}
}  // namespace

int kvskip_launch_select(const float* blk_max, const float* blk_sum, int B, int Hkv, int nb, int rule, float value,
                         int local, uint8_t* keep, int32_t* block_idx, int32_t* block_cnt, float* weight,
                         void* stream) {
  return select_impl(blk_max, blk_sum, B, Hkv, nb, rule, value, local, keep, block_idx, block_cnt, weight, nullptr, 0,
                     stream);
}

int kvskip_launch_select_dyn(const float* blk_max, const float* blk_sum, int B, int Hkv, int T_bound, const int* t_dev,
                             int rule, float value, int local, uint8_t* keep, int32_t* block_idx, int32_t* block_cnt,
                             float* weight, void* stream) {
  if (!t_dev || T_bound < 1) return fail(KVSKIP_E_ARG, "select: t_dev and T_bound >= 1");
  return select_impl(blk_max, blk_sum, B, Hkv, (T_bound + KVSKIP_TILE - 1) / KVSKIP_TILE, rule, value, local, keep,
                     block_idx, block_cnt, weight, t_dev, T_bound, stream);
}

int kvskip_launch_advance(int* t_dev, int delta, void* stream) {
  if (!t_dev) return fail(KVSKIP_E_ARG, "t_dev is null");
  kvb::advance_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(t_dev, delta);
  KVB_CUDA(cudaGetLastError());
  return KVSKIP_OK;
}

#ifdef KVB_TIMELINE
// development builds only: the per-CTA stamps of the last queue-kernel launch (see decode_tcq.cuh)
int kvskip_debug_timeline(unsigned long long* dst, int n) {
  KVB_CUDA(cudaDeviceSynchronize());
  KVB_CUDA(cudaMemcpyFromSymbol(dst, kvb::g_timeline, sizeof(unsigned long long) * std::min(n, 256 * 16)));
  return KVSKIP_OK;
}
#endif

int kvskip_device_status(void* stream, unsigned int* status) {
  if (!status) return fail(KVSKIP_E_ARG, "null status pointer");
  KVB_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  KVB_CUDA(cudaMemcpyFromSymbol(status, kvb::g_status, sizeof(unsigned int)));
  if (*status) {   // a kernel gave up mid-way: wait for everything on the device, then clear the word and the
                   // split counters the kernel may have left behind (on every stream's region)
    KVB_CUDA(cudaDeviceSynchronize());
    const unsigned int zero = 0;
    KVB_CUDA(cudaMemcpyToSymbol(kvb::g_status, &zero, sizeof(zero)));
    void* ptr = nullptr;
    KVB_CUDA(cudaGetSymbolAddress(&ptr, g_split_done));
    KVB_CUDA(cudaMemset(ptr, 0, sizeof(int) * kMergeRegion * kMergeRegions));
  }
  return KVSKIP_OK;
}

}  // extern "C"
