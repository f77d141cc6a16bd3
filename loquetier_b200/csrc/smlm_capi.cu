// C ABI of the SMLM path: argument checks, kernel selection and launches.
// Declarations and the reference interfaces they stand in for: include/smlm_b200.h.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <mutex>
#include <utility>
#include <vector>

#include "../../include/smlm_b200.h"
#include "../../include/smlm_b200_kv.h"
#include "paged_kv.cuh"
#include "paged_prefill.cuh"
#include "rms_norm.cuh"
#include "smlm_fused.cuh"
#include "smlm_fused_tc.cuh"
#include "smlm_merge.cuh"
#include "smlm_plan.cuh"
#include "smlm_wgrad.cuh"
#include "smlm_wgrad_tc.cuh"

namespace {

using namespace smlm;

constexpr int kNumSMs = 148;


// ---- tensor maps ------------------------------------------------------------
// cuTensorMapEncodeTiled is a host-only driver routine; it is looked up through the
// runtime on first use so that the library itself does not link against libcuda.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      p = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Row-major [rows, cols] matrix of 16-bit elements, boxes of [box_rows, 64] elements
// (128 bytes wide) stored with the 128-byte swizzle; out-of-range parts read as zero.
// Encoding a map is a driver call of about a microsecond, and a module forward encodes several per
// launch for tensors that mostly stay where they are (activations of a captured graph, pre-allocated
// buffers of a serving loop), so the most recent encodings are kept in a small direct-mapped table.
// A map depends only on (address, shape, box, type) - not on the device or the contents - so an
// entry can never go stale.
struct MapKey {
  const void* base;
  int rows, cols, box_rows, dtype;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows && dtype == o.dtype;
  }
};
constexpr int kMapCacheSlots = 256;
struct MapCacheEntry {
  MapKey key;
  CUtensorMap map;
  bool valid;
};
std::mutex g_map_mutex;
MapCacheEntry g_map_cache[kMapCacheSlots];

bool make_map_2d(CUtensorMap* m, const void* base, int rows, int cols, int box_rows, int dtype) {
  const MapKey key = {base, rows, cols, box_rows, dtype};
  const uintptr_t h = (reinterpret_cast<uintptr_t>(base) >> 8) * 0x9E3779B97F4A7C15ull +
                      static_cast<uintptr_t>(cols) * 31u + static_cast<uintptr_t>(rows) * 7u + box_rows + dtype;
  MapCacheEntry& e = g_map_cache[(h >> 20) % kMapCacheSlots];
  {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    if (e.valid && e.key == key) {
      *m = e.map;
      return true;
    }
  }
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return false;
  const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  if (fn(m, dtype == SMLM_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
         const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  std::lock_guard<std::mutex> lock(g_map_mutex);
  e.key = key;
  e.map = *m;
  e.valid = true;
  return true;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Rows per piece for a batch of T rows.  The plan builder and every launch derive it from T alone,
// so they always agree.  64 everywhere: cutting 8192 rows into 56-row pieces would give each of the
// 148 SMs one piece of a uniform batch, but with ragged segments the remainders spill into a second
// wave and the launch got slower (measured), so the height stays at the maximum.
inline int piece_rows_for(int T) {
  (void)T;
  return kBM;
}

inline int max_pieces_of(int T, int nseg) { return T / piece_rows_for(T) + nseg; }
// Rows per piece of the tall list (the tcgen05 kernel's tiles).  Always the full 128: cutting a
// batch that needs a little more than a whole number of waves of 148 CTAs at 120 rows instead made
// the launch 1.5x slower (measured), because every piece then ends in rows that leave the kernel's
// 16-row tensor stores for plain stores, and a short tail piece costs as much as a full one.
inline int tall_rows_for(int T, int nseg) {
  (void)T;
  (void)nseg;
  return 2 * kBM;
}
inline int max_tall_pieces_of(int T, int nseg) { return T / tall_rows_for(T, nseg) + nseg; }

// The opt-in to more than 48 KB of dynamic shared memory is a property of (kernel, device): it is
// set when a kernel is first launched on a device, or with more shared memory than before, and
// remembered - not repeated per launch.
constexpr int kMaxDevices = 64;
std::mutex g_attr_mutex;
std::vector<std::pair<const void*, int>> g_attr_done[kMaxDevices];

bool ensure_dynamic_smem(const void* kern, int smem_bytes) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return false;
  }
  {
    std::lock_guard<std::mutex> lock(g_attr_mutex);
    for (const auto& k : g_attr_done[dev])
      if (k.first == kern && k.second >= smem_bytes) return true;
  }
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  std::lock_guard<std::mutex> lock(g_attr_mutex);
  for (auto& k : g_attr_done[dev])
    if (k.first == kern) {
      k.second = std::max(k.second, smem_bytes);
      return true;
    }
  g_attr_done[dev].emplace_back(kern, smem_bytes);
  return true;
}

template <typename Kern, typename... Args>
int launch(Kern kern, dim3 grid, int threads, int cluster_x, int smem_bytes, cudaStream_t stream,
           const Args&... args) {
  if (grid.x == 0 || grid.y == 0) return SMLM_OK;
  // the limit without the opt-in is 48 KB for dynamic and static shared memory TOGETHER, hence the margin
  if (smem_bytes > 40 * 1024 && !ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes))
    return SMLM_ERR_CUDA;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(threads, 1, 1);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // every kernel of the library calls pdl_wait() before it touches memory that an earlier kernel
  // of the stream may have written, so it may be scheduled while its predecessor drains
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  if (cudaLaunchKernelEx(&cfg, kern, args...) != cudaSuccess) {
    cudaGetLastError();
    return SMLM_ERR_CUDA;
  }
  return SMLM_OK;
}

// ---- fused shrink + expand ----------------------------------------------------

template <typename T, int R16, bool RM>
int launch_fused(const FusedArgs& a, const FusedMapsN& tm, int ctas, bool grouped, cudaStream_t stream) {
  const dim3 grid(ctas, 1, 1);
  return grouped ? launch(fused_kernel<T, R16, RM, true>, grid, kFusedThreads, a.ksplit, FusedSmem<R16, RM>::kTotal,
                          stream, a, tm)
                 : launch(fused_kernel<T, R16, RM, false>, grid, kFusedThreads, a.ksplit,
                          FusedSmem<R16, RM>::kTotal, stream, a, tm);
}

template <typename T, bool RM>
int dispatch_fused_r(const FusedArgs& a, const FusedMapsN& tm, int ctas, bool grouped, cudaStream_t stream) {
  const int r16 = (a.R + 15) / 16;
  if (r16 <= 1) return launch_fused<T, 1, RM>(a, tm, ctas, grouped, stream);
  if (r16 <= 2) return launch_fused<T, 2, RM>(a, tm, ctas, grouped, stream);
  if (r16 <= 4) return launch_fused<T, 4, RM>(a, tm, ctas, grouped, stream);
  return launch_fused<T, 8, RM>(a, tm, ctas, grouped, stream);
}

// ---- the tcgen05 variant for ranks above 32 ----------------------------------
// 0: chosen by shape, 1: wherever the kernel applies, -1: never
std::atomic<int> g_tensor_core_mode{0};
// 0: the cluster split of the fused kernel is chosen by the cost model; 1..4: forced
std::atomic<int> g_cluster_split{0};

template <typename T, int R16, bool RM>
int launch_tc(const TcArgs& a, const TcMaps& tm, int max_tall, cudaStream_t stream) {
  return launch(fused_tc_kernel<T, R16, RM>, dim3(max_tall, 1, 1), kTcThreads, 1, TcSmem<R16>::kTotal, stream, a, tm);
}

template <typename T, bool RM>
int dispatch_tc(const TcArgs& a, const TcMaps& tm, int max_tall, cudaStream_t stream) {
  if (a.R <= 64) return launch_tc<T, 4, RM>(a, tm, max_tall, stream);
  return launch_tc<T, 8, RM>(a, tm, max_tall, stream);
}

// The 128-row MMA tile pays off when segments are long enough to fill it and the batch has
// enough of them for every SM; short ragged segments stay on the 64-row mma.sync kernel.
inline bool use_tensor_core_kernel(int T, int nseg, int R, int mode) {
  (void)mode;   // the tcgen05 kernel serves both products and either half alone
  if (R <= 32) return false;
  const int m = g_tensor_core_mode.load(std::memory_order_relaxed);
  if (m < 0) return false;
  if (m > 0) return true;
  return T >= 128 * 96 && T / std::max(nseg, 1) >= 96;
}

// One job of a fused launch: OUT[T, N2] (+)= s2 * round(s1 * IN[T, K1] . W1) . W2 per segment, MID[T, R] written.
struct FusedJobDesc {
  void* out;
  void* mid;
  const void* in;
  const void* const* w1_table;
  const void* const* w2_table;
  int K1, N2, accumulate;
};

// Runs njobs jobs that share the plan, the adapter ids, the rank and the scale.  The jobs must not
// depend on one another (none reads what another writes).  Up to kFusedMaxJobs of them share one
// launch; the tcgen05 variant is launched once per job.
int run_fused(const FusedJobDesc* jobs, int njobs, const int32_t* ids, const float* scale, void* plan, int n_table,
              int T, int nseg, int R, int dtype, int row_major, int scale_mid, int independent, int mode,
              int grouped, cudaStream_t stream) {
  if (use_tensor_core_kernel(T, nseg, R, mode)) {
    const int mt = max_tall_pieces_of(T, nseg);
    for (int j = 0; j < njobs; ++j) {
      const FusedJobDesc& d = jobs[j];
      TcArgs t;
      t.out = d.out; t.mid = d.mid; t.w1_table = d.w1_table; t.w2_table = d.w2_table; t.ids = ids; t.scale = scale;
      t.plan = static_cast<int*>(plan);
      t.n_table = n_table; t.K1 = d.K1; t.R = R; t.N2 = d.N2; t.scale_mid = scale_mid; t.accumulate = d.accumulate;
      t.independent = (independent || j > 0) ? 1 : 0;
      t.mode = mode;
      TcMaps m;
      // one half alone has only one of the two large tensors: the other map is never used, any valid one will do
      const void* in_t = mode == kFusedExpandOnly ? d.out : d.in;
      const void* out_t = mode == kFusedShrinkOnly ? d.in : d.out;
      const int in_cols = mode == kFusedExpandOnly ? d.N2 : d.K1, out_cols = mode == kFusedShrinkOnly ? d.K1 : d.N2;
      if (!make_map_2d(&m.in16, in_t, T, in_cols, 16, dtype) || !make_map_2d(&m.out16, out_t, T, out_cols, 16, dtype))
        return SMLM_ERR_CUDA;
      int rc;
      if (dtype == SMLM_F16)
        rc = row_major ? dispatch_tc<__half, true>(t, m, mt, stream) : dispatch_tc<__half, false>(t, m, mt, stream);
      else
        rc = row_major ? dispatch_tc<__nv_bfloat16, true>(t, m, mt, stream)
                       : dispatch_tc<__nv_bfloat16, false>(t, m, mt, stream);
      if (rc != SMLM_OK) return rc;
    }
    return SMLM_OK;
  }
  const int mp = max_pieces_of(T, nseg);
  const int r16b = (R + 15) / 16;
  const int r16 = r16b > 4 ? 8 : (r16b > 2 ? 4 : r16b);
  const int kc = 64 * fused_chunks(r16);
  // pieces the plan is expected to hold: its capacity, except that a grouped plan turns the short
  // segments of an adapter into one gather piece, so no more than one piece per adapter comes from them
  const int est_pieces = grouped ? std::min(mp, T / piece_rows_for(T) + std::min(nseg, n_table)) : mp;
  const double stage_kb = 64.0 * kc * 2 / 1024.0 * 1.28, slab_kb = 64.0 * fused_slab(r16) * 2 / 1024.0;
  const int slots = kNumSMs * fused_ctas_per_sm(r16);
  for (int j0 = 0; j0 < njobs; j0 += kFusedMaxJobs) {
    const int nj = std::min(kFusedMaxJobs, njobs - j0);
    // A piece can be split over the KS CTAs of a cluster; pick the KS that minimises the estimated
    // time of the launch in microseconds (constants fitted to device-side timelines on B200): per
    // CTA a set-up, a read phase that is bound either by the latency of its ring stages or by what
    // one SM can ingest, the reduce across the cluster, and a write phase bound the same way.  One
    // job: waves of CTAs x time per CTA.  Several jobs: their CTAs differ in length, so the launch
    // takes the summed CTA time over the CTA slots, and never less than its longest CTA.
    int ks = 1;
    double best = 1e30;
    for (int k = 1; k <= 4; ++k) {
      bool fits = true;
      double sum = 0.0, longest = 0.0;
      const int ctas = std::max(est_pieces, 1) * k * nj;
      const double load = std::max(1.0, std::min<double>(ctas, slots) / kNumSMs);  // CTAs sharing one SM
      for (int j = 0; j < nj; ++j) {
        const FusedJobDesc& d = jobs[j0 + j];
        const int ksteps = (d.K1 + kc - 1) / kc, nslabs = (d.N2 + fused_slab(r16) - 1) / fused_slab(r16);
        if (k > 1 && ((mode != kFusedExpandOnly && ksteps < k) || (mode != kFusedShrinkOnly && nslabs < k)))
          fits = false;
        const int nk = (ksteps + k - 1) / k, ns = (nslabs + k - 1) / k;
        const double ph1 = mode == kFusedExpandOnly ? 0.0 : std::max(2.5 + 0.9 * nk, load * nk * stage_kb / 35.0);
        const double ph3 = mode == kFusedShrinkOnly ? 0.0 : std::max(1.0 + 1.2 * ns, load * ns * slab_kb / 33.0);
        const double ph2 = (k > 1 && mode != kFusedExpandOnly) ? 1.0 * k : 0.6;
        const double t = 2.0 + ph1 + ph2 + ph3;
        sum += t * std::max(est_pieces, 1) * k;
        longest = std::max(longest, t);
      }
      if (!fits) break;
      const int waves = (ctas + slots - 1) / slots;
      const double cost = nj == 1 ? waves * longest : std::max(longest, sum / std::min(ctas, slots));
      if (cost < best - 1e-9) {
        best = cost;
        ks = k;
      }
    }
    // Several jobs with at least a piece per SM between them: no split.  Such a launch is bound by
    // bandwidth as a whole, not by the length of its longest CTA, and un-split its CTAs are few enough
    // to become resident at once, so that an independent launch behind it can move in beside them
    // from the start (measured on the benchmark step: dV/dX of seven projections alone takes 87 us
    // split in two and 101 us un-split, but the step is 11 us shorter un-split, because the forward
    // launched behind it no longer waits for a second wave of CTAs).
    if (nj > 1 && static_cast<long long>(std::max(est_pieces, 1)) * nj >= kNumSMs) ks = 1;
    {
      const int forced = g_cluster_split.load(std::memory_order_relaxed);
      if (forced > 0) ks = forced;
    }
    FusedArgs a;
    FusedMapsN tm;
    a.ids = ids; a.scale = scale; a.plan = static_cast<int*>(plan);
    a.n_table = n_table; a.R = R; a.ksplit = ks; a.scale_mid = scale_mid;
    // groups: runs of jobs with the same K1 + N2 (the caller sorted the jobs by it)
    a.ngroups = 0;
    for (int j = 0; j < nj; ++j) {
      const FusedJobDesc& d = jobs[j0 + j];
      if (j == 0 || static_cast<long long>(d.K1) + d.N2 !=
                        static_cast<long long>(jobs[j0 + j - 1].K1) + jobs[j0 + j - 1].N2) {
        a.grp_job_begin[a.ngroups] = j;
        a.grp_cta_begin[a.ngroups] = j * mp * ks;
        ++a.ngroups;
      }
    }
    for (int g = a.ngroups; g <= kFusedMaxJobs; ++g) {
      a.grp_job_begin[g] = nj;
      a.grp_cta_begin[g] = nj * mp * ks;
    }
    a.independent = (independent || j0 > 0) ? 1 : 0;
    a.mode = mode;
    for (int j = 0; j < kFusedMaxJobs; ++j) {
      const FusedJobDesc& d = jobs[j0 + std::min(j, nj - 1)];  // unused slots repeat the last job
      // a half-only launch has no IN (expand only) or no OUT (shrink only): describe the tensor it does
      // have in the unused slots, they are never dereferenced
      const void* in_t = mode == kFusedExpandOnly ? d.out : d.in;
      const int in_cols = mode == kFusedExpandOnly ? d.N2 : d.K1;
      void* out_t = mode == kFusedShrinkOnly ? const_cast<void*>(d.in) : d.out;
      const int out_cols = mode == kFusedShrinkOnly ? d.K1 : d.N2;
      FusedJob& fj = a.job[j];
      fj.in = in_t; fj.out = d.out; fj.mid = d.mid; fj.w1_table = d.w1_table; fj.w2_table = d.w2_table;
      fj.K1 = d.K1; fj.N2 = d.N2; fj.accumulate = d.accumulate; fj.pad_ = 0;
      if (j >= nj) {
        tm.m[j] = tm.m[nj - 1];
        continue;
      }
      if (!make_map_2d(&tm.m[j].in8, in_t, T, in_cols, 8, dtype) ||
          !make_map_2d(&tm.m[j].in16, in_t, T, in_cols, 16, dtype) ||
          !make_map_2d(&tm.m[j].out, out_t, T, out_cols, 16, dtype) ||
          !make_map_2d(&tm.m[j].out8, out_t, T, out_cols, 8, dtype))
        return SMLM_ERR_CUDA;
    }
    const bool g = grouped != 0;
    const int ctas = mp * ks * nj;
    int rc;
    if (dtype == SMLM_F16)
      rc = row_major ? dispatch_fused_r<__half, true>(a, tm, ctas, g, stream)
                     : dispatch_fused_r<__half, false>(a, tm, ctas, g, stream);
    else
      rc = row_major ? dispatch_fused_r<__nv_bfloat16, true>(a, tm, ctas, g, stream)
                     : dispatch_fused_r<__nv_bfloat16, false>(a, tm, ctas, g, stream);
    if (rc != SMLM_OK) return rc;
  }
  return SMLM_OK;
}

// ---- wgrad ------------------------------------------------------------------

template <typename T, int RT>
int launch_wgrad(const WgradArgs& a, const WgradMaps& tm, int groups, cudaStream_t stream) {
  return launch(wgrad_kernel<T, RT>, dim3(groups, a.slabs_total, 1), kWgThreads, 1, WgradSmem<RT>::kTotal, stream, a,
                tm);
}

struct WgradJobDesc {
  void* const* g_table;
  const void* p;
  const void* q;
  int H;
  int transposed;
  int use_scale;
};

inline int wgrad_rt(int R) {
  const int rtb = (R + 15) / 16;
  return rtb > 4 ? 8 : (rtb > 2 ? 4 : rtb);
}

// How a batch of T token rows in npart partitions is cut for the jobs' column counts.
struct WgradShape {
  int slab, slabs_total, group, groups;
  size_t ticket_bytes, scratch_bytes;
};

// The tcgen05 variant serves every rank above 32 unless it is switched off, and the lower ranks
// (padded to 32) when it is forced on.
inline bool wgrad_uses_tensor_cores(int R) {
  const int m = g_tensor_core_mode.load(std::memory_order_relaxed);
  return R > 32 ? m >= 0 : m > 0;
}

WgradShape wgrad_shape(int T, int npart, int R, const int* h, int nh, bool tc) {
  WgradShape s;
  const int rt = tc ? std::max(2, wgrad_rt(R)) : wgrad_rt(R);  // the tcgen05 kernel pads ranks below 32
  s.slab = tc ? wg_tc_slab(rt) : 4 * wgrad_cols_per_warp(rt);
  s.slabs_total = 0;
  for (int i = 0; i < nh; ++i)
    if (h[i] > 0) s.slabs_total += (h[i] + s.slab - 1) / s.slab;
  const int mp = std::max(1, max_pieces_of(T, npart));
  // CTAs that run side by side: one per SM for the tcgen05 kernel, two for the other.  The group
  // size (pieces per CTA) that minimises  rounds of CTAs x (pieces per CTA + a fixed cost for set-up
  // and closing runs, worth about two pieces of the tcgen05 kernel's 512-column slabs and four of the
  // other's 256-column ones); a launch with fewer CTAs than slots takes one round.
  const long long slots = tc ? kNumSMs : 2 * kNumSMs;
  const int fixed = tc ? 2 : 4;
  long long best = -1, g = 1;
  for (int c = 1; c <= kWgMaxGroup; ++c) {
    const long long ctas = static_cast<long long>((mp + c - 1) / c) * s.slabs_total;
    const long long cost = ((ctas + slots - 1) / slots) * (c + fixed);
    if (best < 0 || cost < best) {
      best = cost;
      g = c;
    }
  }
  s.group = static_cast<int>(g);
  s.groups = (mp + s.group - 1) / s.group;
  s.ticket_bytes = (static_cast<size_t>(npart) * s.slabs_total * 4 * sizeof(int) + 255) / 256 * 256;
  s.scratch_bytes = static_cast<size_t>(s.groups) * 2 * s.slabs_total * (rt * 16) * s.slab * sizeof(float);
  return s;
}

// One launch for up to kWgMaxJobs jobs.
int run_wgrad(const WgradJobDesc* jobs, int njobs, const int32_t* part_indptr, const float* scale,
              const int32_t* ids, int n_table, void* plan, void* workspace, size_t workspace_bytes, int npart, int T,
              int R, int dtype, int accumulate, int grad_fp32, int independent, bool tc, cudaStream_t stream) {
  if (njobs < 1 || njobs > kWgMaxJobs) return SMLM_ERR_INVALID_ARGUMENT;
  WgradArgs a;
  WgradMaps tm;
  const int rt = tc ? std::max(2, wgrad_rt(R)) : wgrad_rt(R);
  int hs[kWgMaxJobs];
  for (int j = 0; j < njobs; ++j) hs[j] = jobs[j].H;
  const WgradShape sh = wgrad_shape(T, npart, R, hs, njobs, tc);
  if (workspace == nullptr || workspace_bytes < sh.ticket_bytes + sh.scratch_bytes) return SMLM_ERR_WORKSPACE;
  if (!aligned16(workspace)) return SMLM_ERR_MISALIGNED;
  WgradTcMaps tcm = {};
  int slab_at = 0;
  for (int j = 0; j < kWgMaxJobs; ++j) {
    WgradJob& w = a.job[j];
    if (j >= njobs) {
      w.g_table = nullptr; w.p = nullptr; w.H = 0; w.transposed = 0; w.use_scale = 0; w.slab_begin = slab_at;
      tm.q[j] = tm.q[0];
      tcm.p[j] = tcm.p[0];
      continue;
    }
    if (tc && !make_map_2d(&tcm.p[j], jobs[j].p, T, R, 16, dtype)) return SMLM_ERR_CUDA;
    w.g_table = jobs[j].g_table; w.p = jobs[j].p; w.H = jobs[j].H; w.transposed = jobs[j].transposed;
    w.use_scale = jobs[j].use_scale; w.slab_begin = slab_at;
    slab_at += (jobs[j].H + sh.slab - 1) / sh.slab;
    if (!make_map_2d(&tm.q[j], jobs[j].q, T, jobs[j].H, 16, dtype)) return SMLM_ERR_CUDA;
  }
  a.njobs = njobs; a.slabs_total = sh.slabs_total;
  a.part_indptr = part_indptr; a.scale = scale; a.ids = ids; a.n_table = n_table;
  a.plan = static_cast<int*>(plan);
  a.tickets = static_cast<int*>(workspace);
  a.scratch = reinterpret_cast<float*>(static_cast<char*>(workspace) + sh.ticket_bytes);
  a.npart = npart; a.T = T; a.R = R; a.group = sh.group; a.accumulate = accumulate; a.out_fp32 = grad_fp32;
  a.independent = independent;
  if (tc) {
    for (int j = 0; j < kWgMaxJobs; ++j) tcm.q[j] = tm.q[j];
    const dim3 grid(sh.groups, sh.slabs_total, 1);
    if (dtype == SMLM_F16) {
      if (rt <= 2) return launch(wgrad_tc_kernel<__half, 2>, grid, kWgTcThreads, 1, WgradTcSmem<2>::kTotal, stream, a, tcm);
      return rt <= 4 ? launch(wgrad_tc_kernel<__half, 4>, grid, kWgTcThreads, 1, WgradTcSmem<4>::kTotal, stream, a, tcm)
                     : launch(wgrad_tc_kernel<__half, 8>, grid, kWgTcThreads, 1, WgradTcSmem<8>::kTotal, stream, a, tcm);
    }
    if (rt <= 2)
      return launch(wgrad_tc_kernel<__nv_bfloat16, 2>, grid, kWgTcThreads, 1, WgradTcSmem<2>::kTotal, stream, a, tcm);
    return rt <= 4 ? launch(wgrad_tc_kernel<__nv_bfloat16, 4>, grid, kWgTcThreads, 1, WgradTcSmem<4>::kTotal, stream,
                            a, tcm)
                   : launch(wgrad_tc_kernel<__nv_bfloat16, 8>, grid, kWgTcThreads, 1, WgradTcSmem<8>::kTotal, stream,
                            a, tcm);
  }
  if (dtype == SMLM_F16) {
    if (rt == 1) return launch_wgrad<__half, 1>(a, tm, sh.groups, stream);
    if (rt == 2) return launch_wgrad<__half, 2>(a, tm, sh.groups, stream);
    if (rt == 4) return launch_wgrad<__half, 4>(a, tm, sh.groups, stream);
    return launch_wgrad<__half, 8>(a, tm, sh.groups, stream);
  }
  if (rt == 1) return launch_wgrad<__nv_bfloat16, 1>(a, tm, sh.groups, stream);
  if (rt == 2) return launch_wgrad<__nv_bfloat16, 2>(a, tm, sh.groups, stream);
  if (rt == 4) return launch_wgrad<__nv_bfloat16, 4>(a, tm, sh.groups, stream);
  return launch_wgrad<__nv_bfloat16, 8>(a, tm, sh.groups, stream);
}

// Workspace that serves either kernel variant, so that a buffer sized before a change of the
// tensor-core mode stays valid.
size_t wgrad_workspace_need(int T, int npart, int R, const int* h, int nh) {
  const WgradShape a = wgrad_shape(T, npart, R, h, nh, false);
  const WgradShape b = wgrad_shape(T, npart, R, h, nh, true);
  return std::max(a.ticket_bytes + a.scratch_bytes, b.ticket_bytes + b.scratch_bytes);
}

// The head of a workspace that holds the tickets, for either kernel variant (the larger of the two).
size_t wgrad_ticket_need(int T, int npart, int R, const int* h, int nh) {
  const WgradShape a = wgrad_shape(T, npart, R, h, nh, false);
  const WgradShape b = wgrad_shape(T, npart, R, h, nh, true);
  return std::max(a.ticket_bytes, b.ticket_bytes);
}

// ---- built-in scratch for callers that cannot allocate ------------------------------
// Some hosts of this library run where device allocation is off the table: inside a
// latency-critical serving loop that has pre-carved all of its memory, in a plugin that
// is handed buffers but owns no allocator, or under a framework whose memory pool must
// not be bypassed.  For them the weight-gradient kernel's workspace lives in this fixed
// array in the library's own device image.  Every GPU that loads the library carries the
// array (kStaticWgradBytes) until the process exits.
constexpr size_t kStaticWgradBytes = SMLM_STATIC_WGRAD_BYTES;
static __device__ __align__(256) unsigned char g_wgrad_static_scratch[kStaticWgradBytes];

std::mutex g_static_mutex;
void* g_static_scratch_ptr[kMaxDevices] = {};

// The array's name is only a host-side handle; kernels need its device address, which is
// looked up once per device (with that device current) and remembered.
int static_scratch_of_current_device(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return SMLM_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_wgrad_static_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return SMLM_ERR_CUDA;
    }
    g_static_scratch_ptr[dev] = p;
  }
  *out = g_static_scratch_ptr[dev];
  return SMLM_OK;
}

// ---- RMSNorm ---------------------------------------------------------------------
// Kernel variant for rows of n8 16-byte chunks: threads per CTA and chunks per thread (0: two-pass).
struct RmsShape { int threads, vpt; };
inline RmsShape rms_shape(int n8) {
  if (n8 <= 256) return {256, 1};
  if (n8 <= 512) return {256, 2};
  if (n8 <= 1024) return {512, 2};
  if (n8 <= 2048) return {1024, 2};
  return {1024, 0};
}
// persistent CTAs: about 2048 threads per SM in the forward, 512 in the backward (which holds two rows
// of x, two of gO and its share of dW in registers)
inline int rms_fwd_grid(int rows, int cols) {
  return std::max(1, std::min(rows, kNumSMs * (2048 / rms_shape(cols / 8).threads)));
}
inline int rms_bwd_grid(int rows, int cols) {
  return std::max(1, std::min(rows, kNumSMs * std::max(1, 512 / rms_shape(cols / 8).threads)));
}

template <typename T, int VPT, int NT>
int launch_rms_fwd_v(void* out, float* rms_out, const void* x, const void* w, int rows, int cols, float eps,
                     cudaStream_t stream) {
  return launch(rms_norm_fwd_kernel<T, VPT, NT>, dim3(rms_fwd_grid(rows, cols), 1, 1), NT, 1, 0, stream,
                static_cast<uint4*>(out), rms_out, static_cast<const uint4*>(x), static_cast<const uint4*>(w), rows,
                cols / 8, 1.0f / static_cast<float>(cols), eps);
}

template <typename T>
int launch_rms_fwd(void* out, float* rms_out, const void* x, const void* w, int rows, int cols, float eps,
                   cudaStream_t stream) {
  const RmsShape sh = rms_shape(cols / 8);
  if (sh.vpt == 0) return launch_rms_fwd_v<T, 0, 1024>(out, rms_out, x, w, rows, cols, eps, stream);
  if (sh.threads == 1024) return launch_rms_fwd_v<T, 2, 1024>(out, rms_out, x, w, rows, cols, eps, stream);
  if (sh.threads == 512) return launch_rms_fwd_v<T, 2, 512>(out, rms_out, x, w, rows, cols, eps, stream);
  if (sh.vpt == 2) return launch_rms_fwd_v<T, 2, 256>(out, rms_out, x, w, rows, cols, eps, stream);
  return launch_rms_fwd_v<T, 1, 256>(out, rms_out, x, w, rows, cols, eps, stream);
}

template <typename T, int VPT, int NT>
int launch_rms_bwd_v(void* dx, const void* go, const void* x, const void* w, const float* rms, float* partial,
                     int rows, int cols, int grid, cudaStream_t stream) {
  return launch(rms_norm_bwd_kernel<T, VPT, NT>, dim3(grid, 1, 1), NT, 1, 0, stream, static_cast<uint4*>(dx),
                partial, static_cast<const uint4*>(go), static_cast<const uint4*>(x), static_cast<const uint4*>(w),
                rms, rows, cols / 8, 1.0f / static_cast<float>(cols));
}

template <typename T>
int launch_rms_bwd(void* dx, void* dw, const void* go, const void* x, const void* w, const float* rms,
                   float* partial, int rows, int cols, int dw_fp32, cudaStream_t stream) {
  const RmsShape sh = rms_shape(cols / 8);
  const int g = rms_bwd_grid(rows, cols);
  int rc;
  if (sh.vpt == 0) rc = launch_rms_bwd_v<T, 0, 1024>(dx, go, x, w, rms, partial, rows, cols, g, stream);
  else if (sh.threads == 1024) rc = launch_rms_bwd_v<T, 2, 1024>(dx, go, x, w, rms, partial, rows, cols, g, stream);
  else if (sh.threads == 512) rc = launch_rms_bwd_v<T, 2, 512>(dx, go, x, w, rms, partial, rows, cols, g, stream);
  else if (sh.vpt == 2) rc = launch_rms_bwd_v<T, 2, 256>(dx, go, x, w, rms, partial, rows, cols, g, stream);
  else rc = launch_rms_bwd_v<T, 1, 256>(dx, go, x, w, rms, partial, rows, cols, g, stream);
  if (rc != SMLM_OK) return rc;
  return launch(rms_norm_dw_kernel<T>, dim3((cols + 31) / 32, 1, 1), kRmsThreads, 1, 0, stream, dw,
                static_cast<const float*>(partial), g, cols, dw_fp32);
}

// ---- paged key-value cache ----------------------------------------------------------
// Page ranges a (request, kv head) is cut into, so that small batches still fill the machine.  The
// sequence lengths live on the device, so the choice depends on the batch shape only.
inline int decode_splits(int batch, int num_kv_heads) {
  const int ctas = std::max(1, batch * num_kv_heads);
  return std::max(1, std::min(kPdMaxSplits, (3 * kNumSMs + ctas - 1) / ctas));
}

inline size_t decode_ticket_bytes(int batch, int num_kv_heads) {
  return (static_cast<size_t>(batch) * num_kv_heads * sizeof(int) + 255) / 256 * 256;
}

template <typename T, int G>
int launch_decode(const PdArgs& a, cudaStream_t stream) {
  return launch(paged_decode_kernel<T, G>, dim3(a.batch * a.num_kv_heads * a.splits, 1, 1), kPdWarps * 32, 1, kPdSmem,
                stream, a);
}

template <typename T>
int dispatch_decode(const PdArgs& a, int group, cudaStream_t stream) {
  switch (group) {
    case 1: return launch_decode<T, 1>(a, stream);
    case 2: return launch_decode<T, 2>(a, stream);
    case 4: return launch_decode<T, 4>(a, stream);
    case 8: return launch_decode<T, 8>(a, stream);
    default: return SMLM_ERR_NO_KERNEL;
  }
}

template <typename T>
int dispatch_prefill(const PfArgs& a, const CUtensorMap& kvmap, int group, cudaStream_t stream) {
  int rc = launch(prefill_gather_kernel<T>, dim3(a.total_pages, 1, 1), 128, 1, 0, stream, a);
  if (rc != SMLM_OK) return rc;
  // query tiles: sum over requests of ceil(len / positions per tile) <= total_q / positions per tile + batch
  const int ppt = kPfRows / group;
  const int slots = (a.total_q / ppt + a.batch) * a.num_kv_heads;
  const dim3 grid(slots, 1, 1);
  switch (group) {
    case 1: return launch(paged_prefill_kernel<T, 1>, grid, kPfThreads, 1, kPfSmem, stream, a, kvmap);
    case 2: return launch(paged_prefill_kernel<T, 2>, grid, kPfThreads, 1, kPfSmem, stream, a, kvmap);
    case 4: return launch(paged_prefill_kernel<T, 4>, grid, kPfThreads, 1, kPfSmem, stream, a, kvmap);
    case 8: return launch(paged_prefill_kernel<T, 8>, grid, kPfThreads, 1, kPfSmem, stream, a, kvmap);
    default: return SMLM_ERR_NO_KERNEL;
  }
}

inline bool kv_shape_ok(int head_dim, int page_size) {
  return head_dim == kPdDim && (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64);
}

int run_append(const void* const* kv_ptrs, const int32_t* kv_indptr, const int32_t* last_page_offset, const void* k,
               const void* v, const int32_t* append_indptr, int* err, int batch, int total_pages, int max_tokens,
               int num_layers, int layer_idx, int num_kv_heads, int head_dim, int page_size, int dtype,
               cudaStream_t stream) {
  if (batch < 0 || total_pages < 0 || num_layers <= 0 || layer_idx < 0 || layer_idx >= num_layers || num_kv_heads <= 0)
    return SMLM_ERR_INVALID_ARGUMENT;
  if (dtype != SMLM_F16 && dtype != SMLM_BF16) return SMLM_ERR_DTYPE;
  if (!kv_shape_ok(head_dim, page_size)) return SMLM_ERR_NO_KERNEL;
  if (batch == 0) return SMLM_OK;
  if (kv_ptrs == nullptr || kv_indptr == nullptr || last_page_offset == nullptr || k == nullptr || v == nullptr)
    return SMLM_ERR_INVALID_ARGUMENT;
  if (!aligned16(k) || !aligned16(v)) return SMLM_ERR_MISALIGNED;
  AppendArgs a;
  a.kv_ptrs = kv_ptrs; a.kv_indptr = kv_indptr; a.last_page_offset = last_page_offset; a.k = k; a.v = v;
  a.append_indptr = append_indptr; a.err = err;
  a.batch = batch; a.num_kv_heads = num_kv_heads; a.num_layers = num_layers; a.layer_idx = layer_idx;
  a.page_size = page_size; a.total_pages = total_pages;
  // token chunks per (request, head): enough CTAs to fill the machine when few requests bring long runs
  const int rows = batch * num_kv_heads;
  int chunks = 1;
  if (append_indptr != nullptr) {
    const int per = std::max(1, (max_tokens + 31) / 32);   // a CTA moves 8 rows x 4 tokens per step
    chunks = std::max(1, std::min(per, (16 * kNumSMs + rows - 1) / rows));
  }
  const dim3 grid(rows, chunks, 1);
  return dtype == SMLM_F16 ? launch(append_kv_kernel<__half>, grid, 128, 1, 0, stream, a)
                           : launch(append_kv_kernel<__nv_bfloat16>, grid, 128, 1, 0, stream, a);
}

inline bool projs_ok(const smlm_b200_proj* projs, int nproj) {
  return projs != nullptr && nproj >= 1 && nproj <= SMLM_MAX_PROJ;
}
inline bool small_dim_ok(int v) { return v >= 8 && v <= 128 && (v % 8) == 0; }
inline bool large_dim_ok(int v) { return v >= 8 && (v % 8) == 0; }

}  // namespace

extern "C" {

int smlm_b200_version(void) { return 1; }

int smlm_b200_piece_rows(int T) { return T < 0 ? 0 : piece_rows_for(T); }

const char* smlm_b200_status_string(int status) {
  switch (status) {
    case SMLM_OK: return "ok";
    case SMLM_ERR_INVALID_ARGUMENT: return "invalid argument";
    case SMLM_ERR_DTYPE: return "unsupported dtype (fp16 and bf16 only)";
    case SMLM_ERR_NO_KERNEL: return "No suitable kernel.";
    case SMLM_ERR_MISALIGNED: return "pointer not 16-byte aligned";
    case SMLM_ERR_WORKSPACE: return "plan buffer too small";
    case SMLM_ERR_CUDA: return "CUDA launch failed";
    case SMLM_ERR_BAD_INDPTR: return "segment index pointer is not monotone within [0, T]";
    case SMLM_ERR_BAD_POINTER: return "adapter pointer is null or not 16-byte aligned";
    case SMLM_ERR_BAD_INDEX: return "adapter index outside the table";
    case SMLM_ERR_TIMEOUT: return "a bounded wait inside a kernel ran out";
    case SMLM_ERR_GROUPED_PLAN:
      return "a weight-gradient call was handed a grouped plan; build an ordinary plan for it";
    case SMLM_ERR_STATIC_LIMIT:
      return "problem too large for the library's built-in 16 MiB scratch; use the entry point that takes a "
             "workspace";
    default: return "unknown status";
  }
}

size_t smlm_b200_tmp_size(int num_problems) {
  // three pointer arrays, three int64 leading dimensions and one 3-int problem size per segment
  return num_problems > 0 ? static_cast<size_t>(3 * 8 + 3 * 8 + 12) * static_cast<size_t>(num_problems) : 0;
}

size_t smlm_b200_plan_bytes(int T, int nseg) {
  if (T < 0 || nseg < 0) return 0;
  // two piece lists, then the row index array of a grouped plan (one int per token row)
  return sizeof(int) * kPlanHeaderInts + sizeof(Piece) * static_cast<size_t>(max_pieces_of(T, nseg) + 1) +
         sizeof(int) * kPlanHeaderInts + sizeof(Piece) * static_cast<size_t>(max_tall_pieces_of(T, nseg) + 1) +
         sizeof(int) * (static_cast<size_t>(T) + 4);
}

int smlm_b200_plan(void* plan, size_t plan_bytes, const int32_t* seg_indptr, int nseg, int T, void* stream) {
  return smlm_b200_plan_grouped(plan, plan_bytes, seg_indptr, nullptr, nseg, 0, T, stream);
}

namespace {
int fill_plan_job(PlanJob* j, void* plan, size_t plan_bytes, const int32_t* seg_indptr, const int32_t* seg_ids,
                  int nseg, int n_table, int T) {
  if (plan == nullptr || seg_indptr == nullptr || nseg < 0 || T < 0 || n_table < 0) return SMLM_ERR_INVALID_ARGUMENT;
  if (!aligned16(plan)) return SMLM_ERR_MISALIGNED;
  if (plan_bytes < smlm_b200_plan_bytes(T, nseg)) return SMLM_ERR_WORKSPACE;
  // tables beyond what the builder can count in shared memory get an ordinary plan
  if (seg_ids == nullptr || n_table == 0 || n_table > kGatherMaxTable) {
    seg_ids = nullptr;
    n_table = 0;
  }
  j->plan = static_cast<int*>(plan); j->indptr = seg_indptr; j->ids = seg_ids; j->nseg = nseg; j->T = T;
  j->max_pieces = max_pieces_of(T, nseg); j->bm = piece_rows_for(T);
  j->max_pieces2 = max_tall_pieces_of(T, nseg); j->bm2 = tall_rows_for(T, nseg); j->n_table = n_table;
  return SMLM_OK;
}
}  // namespace

int smlm_b200_plan_grouped(void* plan, size_t plan_bytes, const int32_t* seg_indptr, const int32_t* seg_ids,
                           int nseg, int n_table, int T, void* stream) {
  PlanJobs jobs = {};
  const int rc = fill_plan_job(&jobs.job[0], plan, plan_bytes, seg_indptr, seg_ids, nseg, n_table, T);
  if (rc != SMLM_OK) return rc;
  plan_pieces_kernel<<<1, kPlanThreads, 0, static_cast<cudaStream_t>(stream)>>>(jobs);
  if (cudaGetLastError() != cudaSuccess) return SMLM_ERR_CUDA;
  return SMLM_OK;
}

int smlm_b200_plan_pair(void* plan_a, size_t plan_a_bytes, const int32_t* indptr_a, const int32_t* ids_a, int nseg_a,
                        int n_table_a, int T_a, void* plan_b, size_t plan_b_bytes, const int32_t* indptr_b,
                        int nseg_b, int T_b, void* stream) {
  PlanJobs jobs = {};
  int rc = fill_plan_job(&jobs.job[0], plan_a, plan_a_bytes, indptr_a, ids_a, nseg_a, n_table_a, T_a);
  if (rc != SMLM_OK) return rc;
  rc = fill_plan_job(&jobs.job[1], plan_b, plan_b_bytes, indptr_b, nullptr, nseg_b, 0, T_b);
  if (rc != SMLM_OK) return rc;
  plan_pieces_kernel<<<2, kPlanThreads, 0, static_cast<cudaStream_t>(stream)>>>(jobs);
  if (cudaGetLastError() != cudaSuccess) return SMLM_ERR_CUDA;
  return SMLM_OK;
}

int smlm_b200_merge_segments(const int32_t* req_ids, const int32_t* req_len, int n, int32_t* seg_ids,
                             int32_t* seg_len, int32_t* seg_indptr, int32_t* nseg_out, void* stream) {
  if (n < 0) return SMLM_ERR_INVALID_ARGUMENT;
  if (seg_indptr == nullptr || nseg_out == nullptr) return SMLM_ERR_INVALID_ARGUMENT;
  if (n > 0 && (req_ids == nullptr || req_len == nullptr || seg_ids == nullptr || seg_len == nullptr))
    return SMLM_ERR_INVALID_ARGUMENT;
  merge_segments_kernel<<<1, kMergeThreads, 0, static_cast<cudaStream_t>(stream)>>>(req_ids, req_len, n, seg_ids,
                                                                                  seg_len, seg_indptr, nseg_out);
  if (cudaGetLastError() != cudaSuccess) return SMLM_ERR_CUDA;
  return SMLM_OK;
}

int smlm_b200_group_ids_from_pointers(const void* const* w_table, int nseg, int32_t* ids_out, void* stream) {
  if (nseg < 0) return SMLM_ERR_INVALID_ARGUMENT;
  if (nseg == 0) return SMLM_OK;
  if (w_table == nullptr || ids_out == nullptr) return SMLM_ERR_INVALID_ARGUMENT;
  return launch(pointer_groups_kernel, dim3((nseg + kGroupThreads - 1) / kGroupThreads, 1, 1), kGroupThreads, 1, 0,
                static_cast<cudaStream_t>(stream), w_table, nseg, ids_out);
}

int smlm_b200_plan_status(const void* plan, int* n_pieces, void* stream) {
  if (plan == nullptr) return SMLM_ERR_INVALID_ARGUMENT;
  int hdr[kPlanHeaderInts] = {0, 0, 0, 0};
  if (cudaMemcpyAsync(hdr, plan, sizeof(hdr), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)) !=
          cudaSuccess ||
      cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess) {
    cudaGetLastError();
    return SMLM_ERR_CUDA;
  }
  if (n_pieces != nullptr) *n_pieces = hdr[0];
  if (hdr[1] & kErrBadIndptr) return SMLM_ERR_BAD_INDPTR;
  if (hdr[1] & kErrBadIndex) return SMLM_ERR_BAD_INDEX;
  if (hdr[1] & kErrBadPointer) return SMLM_ERR_BAD_POINTER;
  if (hdr[1] & kErrTimeout) return SMLM_ERR_TIMEOUT;
  if (hdr[1] & kErrGrouped) return SMLM_ERR_GROUPED_PLAN;
  return SMLM_OK;
}

int smlm_b200_gemm(void* y, const void* x, const void* const* w_table, const int32_t* seg_ids,
                   const float* seg_scale, void* plan, int n_table, int T, int nseg, int d_in, int d_out,
                   int dtype, int is_row_major, int accumulate, int grouped, void* stream) {
  if (T < 0 || nseg < 0 || n_table < 0) return SMLM_ERR_INVALID_ARGUMENT;
  if (dtype != SMLM_F16 && dtype != SMLM_BF16) return SMLM_ERR_DTYPE;
  if (T == 0 || nseg == 0) return SMLM_OK;
  if (y == nullptr || x == nullptr || w_table == nullptr || plan == nullptr) return SMLM_ERR_INVALID_ARGUMENT;
  if (!aligned16(y) || !aligned16(x) || !aligned16(plan)) return SMLM_ERR_MISALIGNED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (d_in >= d_out) {
    // shrink: the small dimension is the output width; y plays the part of MID
    if (!small_dim_ok(d_out) || !large_dim_ok(d_in)) return SMLM_ERR_NO_KERNEL;
    if (accumulate) return SMLM_ERR_NO_KERNEL;
    const FusedJobDesc job = {nullptr, y, x, w_table, nullptr, d_in, 64, 0};
    return run_fused(&job, 1, seg_ids, seg_scale, plan, n_table, T, nseg, d_out, dtype, is_row_major, 1, 0,
                     kFusedShrinkOnly, grouped, st);
  }
  // expand: the small dimension is the input width; x plays the part of MID
  if (!small_dim_ok(d_in) || !large_dim_ok(d_out)) return SMLM_ERR_NO_KERNEL;
  const FusedJobDesc job = {y, const_cast<void*>(x), nullptr, nullptr, w_table, 64, d_out, accumulate};
  return run_fused(&job, 1, seg_ids, seg_scale, plan, n_table, T, nseg, d_in, dtype, is_row_major, 0, 0,
                   kFusedExpandOnly, grouped, st);
}

int smlm_b200_set_cluster_split(int split) {
  const int v = split < 0 ? 0 : (split > 4 ? 4 : split);
  return g_cluster_split.exchange(v, std::memory_order_relaxed);
}

int smlm_b200_set_tensor_core_mode(int mode) {
  const int m = mode > 0 ? 1 : (mode < 0 ? -1 : 0);
  return g_tensor_core_mode.exchange(m, std::memory_order_relaxed);
}

int smlm_b200_fwd(void* y, const void* x, void* v, const void* const* wa_table, const void* const* wb_table,
                  const int32_t* seg_ids, const float* seg_scale, void* plan, int n_table, int T, int nseg,
                  int h_in, int h_out, int rank, int dtype, int is_row_major, int accumulate, int independent,
                  int grouped, void* stream) {
  if (T < 0 || nseg < 0 || n_table < 0) return SMLM_ERR_INVALID_ARGUMENT;
  if (dtype != SMLM_F16 && dtype != SMLM_BF16) return SMLM_ERR_DTYPE;
  if (T == 0 || nseg == 0) return SMLM_OK;
  if (y == nullptr || x == nullptr || v == nullptr || wa_table == nullptr || wb_table == nullptr ||
      plan == nullptr)
    return SMLM_ERR_INVALID_ARGUMENT;
  if (!aligned16(y) || !aligned16(x) || !aligned16(v) || !aligned16(plan)) return SMLM_ERR_MISALIGNED;
  if (!small_dim_ok(rank) || !large_dim_ok(h_in) || !large_dim_ok(h_out)) return SMLM_ERR_NO_KERNEL;
  const FusedJobDesc job = {y, v, x, wa_table, wb_table, h_in, h_out, accumulate};
  return run_fused(&job, 1, seg_ids, seg_scale, plan, n_table, T, nseg, rank, dtype, is_row_major, /*scale_mid=*/0,
                   independent != 0, kFusedBoth, grouped, static_cast<cudaStream_t>(stream));
}

size_t smlm_b200_wgrad_workspace_bytes(int T, int npart, int rank, int h0, int h1) {
  if (T < 0 || npart < 0 || rank <= 0 || h0 <= 0 || h1 < 0) return 0;
  // enough for either kernel, so that a buffer sized before a change of the tensor-core mode stays valid
  const int hs[2] = {h0, h1};
  return wgrad_workspace_need(T, npart, rank, hs, 2);
}

size_t smlm_b200_wgrad_ticket_bytes(int T, int npart, int rank, int h0, int h1) {
  if (T < 0 || npart < 0 || rank <= 0 || h0 <= 0 || h1 < 0) return 0;
  const int hs[2] = {h0, h1};
  return wgrad_ticket_need(T, npart, rank, hs, 2);
}

int smlm_b200_wgrad(void* const* g_table, const void* p, const void* q, const int32_t* part_indptr,
                    const float* part_scale, void* plan, void* workspace, size_t workspace_bytes, int npart, int T,
                    int rank, int h, int dtype, int transposed, int accumulate, int grad_fp32, void* stream) {
  if (T < 0 || npart < 0) return SMLM_ERR_INVALID_ARGUMENT;
  if (dtype != SMLM_F16 && dtype != SMLM_BF16) return SMLM_ERR_DTYPE;
  if (npart == 0 || T == 0) return SMLM_OK;
  if (g_table == nullptr || p == nullptr || q == nullptr || part_indptr == nullptr || plan == nullptr)
    return SMLM_ERR_INVALID_ARGUMENT;
  if (!aligned16(p) || !aligned16(q) || !aligned16(plan)) return SMLM_ERR_MISALIGNED;
  if (!small_dim_ok(rank) || !large_dim_ok(h)) return SMLM_ERR_NO_KERNEL;
  const WgradJobDesc job = {g_table, p, q, h, transposed, part_scale != nullptr};
  return run_wgrad(&job, 1, part_indptr, part_scale, nullptr, 0, plan, workspace, workspace_bytes, npart, T,
                   rank, dtype, accumulate, grad_fp32, 0, wgrad_uses_tensor_cores(rank),
                   static_cast<cudaStream_t>(stream));
}

int smlm_b200_wgrad_static(void* const* g_table, const void* p, const void* q, const int32_t* part_indptr,
                           const float* part_scale, void* plan, int npart, int T, int rank, int h, int dtype,
                           int transposed, int accumulate, int grad_fp32, void* stream) {
  if (T < 0 || npart < 0) return SMLM_ERR_INVALID_ARGUMENT;
  if (dtype != SMLM_F16 && dtype != SMLM_BF16) return SMLM_ERR_DTYPE;
  if (npart == 0 || T == 0) return SMLM_OK;
  if (g_table == nullptr || p == nullptr || q == nullptr || part_indptr == nullptr || plan == nullptr)
    return SMLM_ERR_INVALID_ARGUMENT;
  if (!aligned16(p) || !aligned16(q) || !aligned16(plan)) return SMLM_ERR_MISALIGNED;
  if (!small_dim_ok(rank) || !large_dim_ok(h)) return SMLM_ERR_NO_KERNEL;
  // the kernel variant is chosen once, here: the size check, the ticket range that is cleared and the
  // launch all follow this one reading of the process-wide mode
  const bool tc = wgrad_uses_tensor_cores(rank);
  const WgradShape sh = wgrad_shape(T, npart, rank, &h, 1, tc);
  if (sh.ticket_bytes + sh.scratch_bytes > kStaticWgradBytes) return SMLM_ERR_STATIC_LIMIT;
  void* scratch = nullptr;
  const int rc = static_scratch_of_current_device(&scratch);
  if (rc != SMLM_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the array keeps whatever the previous call left; only the tickets have to start at zero
  if (cudaMemsetAsync(scratch, 0, sh.ticket_bytes, st) != cudaSuccess) {
    cudaGetLastError();
    return SMLM_ERR_CUDA;
  }
  const WgradJobDesc job = {g_table, p, q, h, transposed, part_scale != nullptr};
  return run_wgrad(&job, 1, part_indptr, part_scale, nullptr, 0, plan, scratch, kStaticWgradBytes, npart, T,
                   rank, dtype, accumulate, grad_fp32, 0, tc, st);
}

int smlm_b200_wgrad_pair(void* const* dA_table, void* const* dB_table, const void* dv, const void* x,
                         const void* v, const void* go, const int32_t* part_indptr, const int32_t* part_ids,
                         const float* part_scale, void* plan, void* workspace, size_t workspace_bytes, int n_table,
                         int npart, int T, int h_in, int h_out, int rank, int dtype, int is_row_major,
                         int accumulate, int grad_fp32, int independent, void* stream) {
  if (T < 0 || npart < 0 || n_table < 0) return SMLM_ERR_INVALID_ARGUMENT;
  if (dtype != SMLM_F16 && dtype != SMLM_BF16) return SMLM_ERR_DTYPE;
  if (npart == 0 || T == 0) return SMLM_OK;
  if (dA_table == nullptr || dB_table == nullptr || dv == nullptr || x == nullptr || v == nullptr ||
      go == nullptr || part_indptr == nullptr || plan == nullptr)
    return SMLM_ERR_INVALID_ARGUMENT;
  if (!aligned16(dv) || !aligned16(x) || !aligned16(v) || !aligned16(go) || !aligned16(plan))
    return SMLM_ERR_MISALIGNED;
  if (!small_dim_ok(rank) || !large_dim_ok(h_in) || !large_dim_ok(h_out)) return SMLM_ERR_NO_KERNEL;
  const WgradJobDesc jobs[2] = {{dB_table, v, go, h_out, is_row_major ? 0 : 1, part_scale != nullptr},
                                {dA_table, dv, x, h_in, is_row_major ? 1 : 0, 0}};
  return run_wgrad(jobs, 2, part_indptr, part_scale, part_ids, n_table, plan, workspace, workspace_bytes, npart, T,
                   rank, dtype, accumulate, grad_fp32, independent != 0, wgrad_uses_tensor_cores(rank),
                   static_cast<cudaStream_t>(stream));
}

int smlm_b200_bwd_dx(void* dx, void* dv, const void* go, const void* const* wa_table, const void* const* wb_table,
                     const int32_t* part_ids, const float* part_scale, void* plan, int n_table, int T, int npart,
                     int h_in, int h_out, int rank, int dtype, int is_row_major, int independent, int grouped,
                     void* stream) {
  if (T < 0 || npart < 0 || n_table < 0) return SMLM_ERR_INVALID_ARGUMENT;
  if (dtype != SMLM_F16 && dtype != SMLM_BF16) return SMLM_ERR_DTYPE;
  if (T == 0 || npart == 0) return SMLM_OK;
  if (dx == nullptr || dv == nullptr || go == nullptr || wa_table == nullptr || wb_table == nullptr ||
      plan == nullptr)
    return SMLM_ERR_INVALID_ARGUMENT;
  if (!aligned16(dx) || !aligned16(dv) || !aligned16(go) || !aligned16(plan)) return SMLM_ERR_MISALIGNED;
  if (!small_dim_ok(rank) || !large_dim_ok(h_in) || !large_dim_ok(h_out)) return SMLM_ERR_NO_KERNEL;
  // dV = scale * gO . B : B is [h_out, r] (r contiguous) in the PEFT layout, i.e. a row-major
  // [K = h_out][N = r] operand; the math layout B [r, h_out] is the column-major one.  The layout
  // flag therefore flips for both products of this launch (dX = dV . A likewise).
  const FusedJobDesc job = {dx, dv, go, wb_table, wa_table, h_out, h_in, 0};
  return run_fused(&job, 1, part_ids, part_scale, plan, n_table, T, npart, rank, dtype, !is_row_major,
                   /*scale_mid=*/1, independent != 0, kFusedBoth, grouped, static_cast<cudaStream_t>(stream));
}

int smlm_b200_bwd(void* dx, void* const* dA_table, void* const* dB_table, void* dv, const void* go,
                  const void* x, const void* v, const void* const* wa_table, const void* const* wb_table,
                  const int32_t* part_ids, const float* part_scale, const int32_t* part_indptr, void* plan,
                  void* workspace, size_t workspace_bytes, int n_table, int T, int npart, int h_in, int h_out,
                  int rank, int dtype, int is_row_major, int accumulate_grads, int grad_fp32, void* stream) {
  if (T == 0 || npart == 0) return (T < 0 || npart < 0) ? SMLM_ERR_INVALID_ARGUMENT : SMLM_OK;
  if (dA_table == nullptr || dB_table == nullptr || x == nullptr || v == nullptr || part_indptr == nullptr)
    return SMLM_ERR_INVALID_ARGUMENT;
  const int rc = smlm_b200_bwd_dx(dx, dv, go, wa_table, wb_table, part_ids, part_scale, plan, n_table, T, npart,
                                  h_in, h_out, rank, dtype, is_row_major, 0, 0, stream);
  if (rc != SMLM_OK) return rc;
  // dB = scale * gO^T . V ([h_out, r] in the PEFT layout: transposed store) and
  // dA = dV^T . X ([r, h_in] in the PEFT layout; dV already carries the scale), in one launch
  return smlm_b200_wgrad_pair(dA_table, dB_table, dv, x, v, go, part_indptr, part_ids, part_scale, plan, workspace,
                              workspace_bytes, n_table, npart, T, h_in, h_out, rank, dtype, is_row_major,
                              accumulate_grads, grad_fp32, 0, stream);
}

// ---- several projections per launch ---------------------------------------------------

int smlm_b200_fwd_multi(const smlm_b200_proj* projs, int nproj, const int32_t* seg_ids, const float* seg_scale,
                        void* plan, int n_table, int T, int nseg, int rank, int dtype, int is_row_major,
                        int accumulate, int independent, int grouped, void* stream) {
  if (T < 0 || nseg < 0 || n_table < 0 || !projs_ok(projs, nproj)) return SMLM_ERR_INVALID_ARGUMENT;
  if (dtype != SMLM_F16 && dtype != SMLM_BF16) return SMLM_ERR_DTYPE;
  if (T == 0 || nseg == 0) return SMLM_OK;
  if (plan == nullptr || !aligned16(plan)) return plan == nullptr ? SMLM_ERR_INVALID_ARGUMENT : SMLM_ERR_MISALIGNED;
  if (!small_dim_ok(rank)) return SMLM_ERR_NO_KERNEL;
  FusedJobDesc jobs[SMLM_MAX_PROJ];
  for (int j = 0; j < nproj; ++j) {
    const smlm_b200_proj& p = projs[j];
    if (p.y == nullptr || p.x == nullptr || p.v == nullptr || p.wa_table == nullptr || p.wb_table == nullptr)
      return SMLM_ERR_INVALID_ARGUMENT;
    if (!aligned16(p.y) || !aligned16(p.x) || !aligned16(p.v)) return SMLM_ERR_MISALIGNED;
    if (!large_dim_ok(p.h_in) || !large_dim_ok(p.h_out)) return SMLM_ERR_NO_KERNEL;
    jobs[j] = {p.y, p.v, p.x, p.wa_table, p.wb_table, p.h_in, p.h_out, accumulate};
  }
  // the longest jobs first, so that the launch ends on its shortest CTAs
  std::stable_sort(jobs, jobs + nproj, [](const FusedJobDesc& a, const FusedJobDesc& b) {
    return static_cast<long long>(a.K1) + a.N2 > static_cast<long long>(b.K1) + b.N2;
  });
  return run_fused(jobs, nproj, seg_ids, seg_scale, plan, n_table, T, nseg, rank, dtype, is_row_major, 0,
                   independent != 0, kFusedBoth, grouped, static_cast<cudaStream_t>(stream));
}

int smlm_b200_bwd_dx_multi(const smlm_b200_proj* projs, int nproj, const int32_t* part_ids, const float* part_scale,
                           void* plan, int n_table, int T, int npart, int rank, int dtype, int is_row_major,
                           int independent, void* stream) {
  if (T < 0 || npart < 0 || n_table < 0 || !projs_ok(projs, nproj)) return SMLM_ERR_INVALID_ARGUMENT;
  if (dtype != SMLM_F16 && dtype != SMLM_BF16) return SMLM_ERR_DTYPE;
  if (T == 0 || npart == 0) return SMLM_OK;
  if (plan == nullptr || !aligned16(plan)) return plan == nullptr ? SMLM_ERR_INVALID_ARGUMENT : SMLM_ERR_MISALIGNED;
  if (!small_dim_ok(rank)) return SMLM_ERR_NO_KERNEL;
  FusedJobDesc jobs[SMLM_MAX_PROJ];
  for (int j = 0; j < nproj; ++j) {
    const smlm_b200_proj& p = projs[j];
    if (p.dx == nullptr || p.dv == nullptr || p.go == nullptr || p.wa_table == nullptr || p.wb_table == nullptr)
      return SMLM_ERR_INVALID_ARGUMENT;
    if (!aligned16(p.dx) || !aligned16(p.dv) || !aligned16(p.go)) return SMLM_ERR_MISALIGNED;
    if (!large_dim_ok(p.h_in) || !large_dim_ok(p.h_out)) return SMLM_ERR_NO_KERNEL;
    jobs[j] = {p.dx, p.dv, p.go, p.wb_table, p.wa_table, p.h_out, p.h_in, 0};
  }
  std::stable_sort(jobs, jobs + nproj, [](const FusedJobDesc& a, const FusedJobDesc& b) {
    return static_cast<long long>(a.K1) + a.N2 > static_cast<long long>(b.K1) + b.N2;
  });
  // the layout flag flips for both products of the backward, as in smlm_b200_bwd_dx
  return run_fused(jobs, nproj, part_ids, part_scale, plan, n_table, T, npart, rank, dtype, !is_row_major, 1,
                   independent != 0, kFusedBoth, 0, static_cast<cudaStream_t>(stream));
}

size_t smlm_b200_wgrad_multi_workspace_bytes(const smlm_b200_proj* projs, int nproj, int T, int npart, int rank) {
  if (T < 0 || npart < 0 || rank <= 0 || !projs_ok(projs, nproj)) return 0;
  int hs[2 * SMLM_MAX_PROJ];
  for (int j = 0; j < nproj; ++j) {
    hs[2 * j] = projs[j].h_out;
    hs[2 * j + 1] = projs[j].h_in;
  }
  return wgrad_workspace_need(T, npart, rank, hs, 2 * nproj);
}

size_t smlm_b200_wgrad_multi_ticket_bytes(const smlm_b200_proj* projs, int nproj, int T, int npart, int rank) {
  if (T < 0 || npart < 0 || rank <= 0 || !projs_ok(projs, nproj)) return 0;
  int hs[2 * SMLM_MAX_PROJ];
  for (int j = 0; j < nproj; ++j) {
    hs[2 * j] = projs[j].h_out;
    hs[2 * j + 1] = projs[j].h_in;
  }
  return wgrad_ticket_need(T, npart, rank, hs, 2 * nproj);
}

int smlm_b200_wgrad_select_multi(const smlm_b200_proj* projs, int nproj, int which, const int32_t* part_indptr,
                                 const int32_t* part_ids, const float* part_scale, void* plan, void* workspace,
                                 size_t workspace_bytes, int n_table, int npart, int T, int rank, int dtype,
                                 int is_row_major, int accumulate, int grad_fp32, int independent, void* stream) {
  if (T < 0 || npart < 0 || n_table < 0 || !projs_ok(projs, nproj) || (which & 3) == 0 || (which & ~3) != 0)
    return SMLM_ERR_INVALID_ARGUMENT;
  if (dtype != SMLM_F16 && dtype != SMLM_BF16) return SMLM_ERR_DTYPE;
  if (npart == 0 || T == 0) return SMLM_OK;
  if (part_indptr == nullptr || plan == nullptr) return SMLM_ERR_INVALID_ARGUMENT;
  if (!aligned16(plan)) return SMLM_ERR_MISALIGNED;
  if (!small_dim_ok(rank)) return SMLM_ERR_NO_KERNEL;
  WgradJobDesc jobs[2 * SMLM_MAX_PROJ];
  int nj = 0;
  for (int j = 0; j < nproj; ++j) {
    const smlm_b200_proj& p = projs[j];
    if (!large_dim_ok(p.h_in) || !large_dim_ok(p.h_out)) return SMLM_ERR_NO_KERNEL;
    if (which & SMLM_WGRAD_DB) {
      if (p.dB_table == nullptr || p.v == nullptr || p.go == nullptr) return SMLM_ERR_INVALID_ARGUMENT;
      if (!aligned16(p.v) || !aligned16(p.go)) return SMLM_ERR_MISALIGNED;
      jobs[nj++] = {p.dB_table, p.v, p.go, p.h_out, is_row_major ? 0 : 1, part_scale != nullptr};
    }
    if (which & SMLM_WGRAD_DA) {
      if (p.dA_table == nullptr || p.dv == nullptr || p.x == nullptr) return SMLM_ERR_INVALID_ARGUMENT;
      if (!aligned16(p.dv) || !aligned16(p.x)) return SMLM_ERR_MISALIGNED;
      jobs[nj++] = {p.dA_table, p.dv, p.x, p.h_in, is_row_major ? 1 : 0, 0};
    }
  }
  return run_wgrad(jobs, nj, part_indptr, part_scale, part_ids, n_table, plan, workspace, workspace_bytes, npart, T,
                   rank, dtype, accumulate, grad_fp32, independent != 0, wgrad_uses_tensor_cores(rank),
                   static_cast<cudaStream_t>(stream));
}

int smlm_b200_wgrad_pair_multi(const smlm_b200_proj* projs, int nproj, const int32_t* part_indptr,
                               const int32_t* part_ids, const float* part_scale, void* plan, void* workspace,
                               size_t workspace_bytes, int n_table, int npart, int T, int rank, int dtype,
                               int is_row_major, int accumulate, int grad_fp32, int independent, void* stream) {
  return smlm_b200_wgrad_select_multi(projs, nproj, SMLM_WGRAD_DB | SMLM_WGRAD_DA, part_indptr, part_ids, part_scale,
                                      plan, workspace, workspace_bytes, n_table, npart, T, rank, dtype, is_row_major,
                                      accumulate, grad_fp32, independent, stream);
}

// ---- paged key-value cache ------------------------------------------------------------------

size_t smlm_b200_batch_decode_workspace_bytes(int batch_size, int num_qo_heads, int num_kv_heads) {
  if (batch_size <= 0 || num_qo_heads <= 0 || num_kv_heads <= 0) return 0;
  return decode_ticket_bytes(batch_size, num_kv_heads) +
         static_cast<size_t>(batch_size) * num_qo_heads * decode_splits(batch_size, num_kv_heads) * kPdRec *
             sizeof(float);
}

size_t smlm_b200_batch_decode_ticket_bytes(int batch_size, int num_kv_heads) {
  if (batch_size <= 0 || num_kv_heads <= 0) return 0;
  return decode_ticket_bytes(batch_size, num_kv_heads);
}

int smlm_b200_batch_decode(void* o, const void* q, const void* const* kv_ptrs, const int32_t* kv_indptr,
                           const int32_t* last_page_offset, void* workspace, size_t workspace_bytes, int* status_word,
                           int batch_size, int total_pages, int num_qo_heads, int num_kv_heads, int head_dim,
                           int num_layers, int layer_idx, int page_size, float rope_theta, int dtype, void* stream) {
  if (batch_size < 0 || total_pages < 0 || num_qo_heads <= 0 || num_kv_heads <= 0 || num_layers <= 0 ||
      layer_idx < 0 || layer_idx >= num_layers || !(rope_theta > 0.f))
    return SMLM_ERR_INVALID_ARGUMENT;
  if (dtype != SMLM_F16 && dtype != SMLM_BF16) return SMLM_ERR_DTYPE;
  // the reference's "No suitable kernel." (loquetier_ops.cc:157-159): head_dim, page size, group size
  if (num_qo_heads % num_kv_heads != 0 || !kv_shape_ok(head_dim, page_size)) return SMLM_ERR_NO_KERNEL;
  const int group = num_qo_heads / num_kv_heads;
  if (group != 1 && group != 2 && group != 4 && group != 8) return SMLM_ERR_NO_KERNEL;
  if (batch_size == 0) return SMLM_OK;
  if (o == nullptr || q == nullptr || kv_ptrs == nullptr || kv_indptr == nullptr || last_page_offset == nullptr)
    return SMLM_ERR_INVALID_ARGUMENT;
  if (!aligned16(o) || !aligned16(q)) return SMLM_ERR_MISALIGNED;
  PdArgs a;
  a.splits = decode_splits(batch_size, num_kv_heads);
  if (a.splits > 1) {
    if (workspace == nullptr || workspace_bytes < smlm_b200_batch_decode_workspace_bytes(batch_size, num_qo_heads,
                                                                                          num_kv_heads))
      return SMLM_ERR_WORKSPACE;
    if (!aligned16(workspace)) return SMLM_ERR_MISALIGNED;
  }
  a.o = o; a.q = q; a.kv_ptrs = kv_ptrs; a.kv_indptr = kv_indptr; a.last_page_offset = last_page_offset;
  a.err = status_word;
  a.tickets = static_cast<int*>(workspace);
  a.partial = workspace == nullptr ? nullptr
                                   : reinterpret_cast<float*>(static_cast<char*>(workspace) +
                                                              decode_ticket_bytes(batch_size, num_kv_heads));
  a.batch = batch_size; a.num_kv_heads = num_kv_heads; a.num_layers = num_layers; a.layer_idx = layer_idx;
  a.page_size = page_size; a.total_pages = total_pages;
  a.log2_theta = std::log2(rope_theta);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == SMLM_F16 ? dispatch_decode<__half>(a, group, st) : dispatch_decode<__nv_bfloat16>(a, group, st);
}

size_t smlm_b200_batch_prefill_workspace_bytes(int total_pages, int page_size, int num_kv_heads) {
  if (total_pages <= 0 || page_size <= 0 || num_kv_heads <= 0) return 0;
  return static_cast<size_t>(total_pages) * page_size * 2 * num_kv_heads * kPdDim * 2;
}

int smlm_b200_batch_prefill(void* o, const void* q, const int32_t* qo_indptr, const void* const* kv_ptrs,
                            const int32_t* kv_indptr, const int32_t* last_page_offset, void* workspace,
                            size_t workspace_bytes, int* status_word, int batch_size, int total_q, int total_pages, int num_qo_heads, int num_kv_heads,
                            int head_dim, int num_layers, int layer_idx, int page_size, float rope_theta, int dtype,
                            void* stream) {
  if (batch_size < 0 || total_q < 0 || total_pages < 0 || num_qo_heads <= 0 || num_kv_heads <= 0 || num_layers <= 0 ||
      layer_idx < 0 || layer_idx >= num_layers || !(rope_theta > 0.f))
    return SMLM_ERR_INVALID_ARGUMENT;
  if (dtype != SMLM_F16 && dtype != SMLM_BF16) return SMLM_ERR_DTYPE;
  if (num_qo_heads % num_kv_heads != 0 || !kv_shape_ok(head_dim, page_size)) return SMLM_ERR_NO_KERNEL;
  const int group = num_qo_heads / num_kv_heads;
  if (group != 1 && group != 2 && group != 4 && group != 8) return SMLM_ERR_NO_KERNEL;
  if (batch_size == 0 || total_q == 0) return SMLM_OK;
  if (o == nullptr || q == nullptr || qo_indptr == nullptr || kv_ptrs == nullptr || kv_indptr == nullptr ||
      last_page_offset == nullptr)
    return SMLM_ERR_INVALID_ARGUMENT;
  if (!aligned16(o) || !aligned16(q)) return SMLM_ERR_MISALIGNED;
  if (total_pages == 0) return SMLM_ERR_INVALID_ARGUMENT;   // queries without a single page of keys
  if (workspace == nullptr ||
      workspace_bytes < smlm_b200_batch_prefill_workspace_bytes(total_pages, page_size, num_kv_heads))
    return SMLM_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(workspace) & 127) != 0) return SMLM_ERR_MISALIGNED;
  if (static_cast<long long>(total_pages) * page_size > 0x7fffffffLL) return SMLM_ERR_INVALID_ARGUMENT;
  CUtensorMap kvmap;
  if (!make_map_2d(&kvmap, workspace, total_pages * page_size, 2 * num_kv_heads * kPdDim, kPfKeys, dtype))
    return SMLM_ERR_CUDA;
  PfArgs a;
  a.scratch = workspace;
  a.o = o; a.q = q; a.qo_indptr = qo_indptr; a.kv_ptrs = kv_ptrs; a.kv_indptr = kv_indptr;
  a.last_page_offset = last_page_offset; a.err = status_word;
  a.batch = batch_size; a.num_kv_heads = num_kv_heads; a.num_layers = num_layers; a.layer_idx = layer_idx;
  a.page_size = page_size; a.total_pages = total_pages; a.total_q = total_q;
  a.log2_theta = std::log2(rope_theta);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == SMLM_F16 ? dispatch_prefill<__half>(a, kvmap, group, st)
                           : dispatch_prefill<__nv_bfloat16>(a, kvmap, group, st);
}

int smlm_b200_append_kv(const void* const* kv_ptrs, const int32_t* kv_indptr, const int32_t* last_page_offset,
                        const void* k, const void* v, int* status_word, int batch_size, int total_pages,
                        int num_layers, int layer_idx, int num_kv_heads, int head_dim, int page_size, int dtype,
                        void* stream) {
  return run_append(kv_ptrs, kv_indptr, last_page_offset, k, v, nullptr, status_word, batch_size, total_pages, 1,
                    num_layers, layer_idx, num_kv_heads, head_dim, page_size, dtype, static_cast<cudaStream_t>(stream));
}

int smlm_b200_init_kv(const void* const* kv_ptrs, const int32_t* kv_indptr, const int32_t* last_page_offset,
                      const void* k, const void* v, const int32_t* seqlen_indptr, int* status_word, int batch_size,
                      int total_pages, int total_tokens, int num_layers, int layer_idx, int num_kv_heads, int head_dim,
                      int page_size, int dtype, void* stream) {
  if (seqlen_indptr == nullptr || total_tokens < 0) return SMLM_ERR_INVALID_ARGUMENT;
  return run_append(kv_ptrs, kv_indptr, last_page_offset, k, v, seqlen_indptr, status_word, batch_size, total_pages,
                    total_tokens, num_layers, layer_idx, num_kv_heads, head_dim, page_size, dtype,
                    static_cast<cudaStream_t>(stream));
}

int smlm_b200_rms_norm(void* out, float* rms_out, const void* x, const void* w, int rows, int cols, float eps,
                       int dtype, void* stream) {
  if (rows < 0 || cols <= 0) return SMLM_ERR_INVALID_ARGUMENT;
  if (dtype != SMLM_F16 && dtype != SMLM_BF16) return SMLM_ERR_DTYPE;
  if (cols % 8 != 0) return SMLM_ERR_NO_KERNEL;  // the reference's only refusal (rms_norm_cutlass.cu:163-165)
  if (rows == 0) return SMLM_OK;
  if (out == nullptr || rms_out == nullptr || x == nullptr || w == nullptr) return SMLM_ERR_INVALID_ARGUMENT;
  if (!aligned16(out) || !aligned16(x) || !aligned16(w) || (reinterpret_cast<uintptr_t>(rms_out) & 3) != 0)
    return SMLM_ERR_MISALIGNED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == SMLM_F16 ? launch_rms_fwd<__half>(out, rms_out, x, w, rows, cols, eps, st)
                           : launch_rms_fwd<__nv_bfloat16>(out, rms_out, x, w, rows, cols, eps, st);
}

size_t smlm_b200_rms_norm_bwd_workspace_bytes(int rows, int cols) {
  if (rows <= 0 || cols <= 0 || cols % 8 != 0) return 0;
  return static_cast<size_t>(rms_bwd_grid(rows, cols)) * cols * sizeof(float);
}

int smlm_b200_rms_norm_bwd(void* dx, void* dw, const void* go, const void* x, const void* w, const float* rms,
                           void* workspace, size_t workspace_bytes, int rows, int cols, int dtype, int dw_fp32,
                           void* stream) {
  if (rows < 0 || cols <= 0) return SMLM_ERR_INVALID_ARGUMENT;
  if (dtype != SMLM_F16 && dtype != SMLM_BF16) return SMLM_ERR_DTYPE;
  if (cols % 8 != 0) return SMLM_ERR_NO_KERNEL;
  if (dx == nullptr || dw == nullptr || go == nullptr || x == nullptr || w == nullptr || rms == nullptr)
    return SMLM_ERR_INVALID_ARGUMENT;
  if (!aligned16(dx) || !aligned16(go) || !aligned16(x) || !aligned16(w) || !aligned16(workspace))
    return SMLM_ERR_MISALIGNED;
  if (rows == 0) return SMLM_ERR_INVALID_ARGUMENT;  // a sum over no rows: the caller zeroes dW itself
  if (workspace == nullptr || workspace_bytes < smlm_b200_rms_norm_bwd_workspace_bytes(rows, cols))
    return SMLM_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* partial = static_cast<float*>(workspace);
  return dtype == SMLM_F16
             ? launch_rms_bwd<__half>(dx, dw, go, x, w, rms, partial, rows, cols, dw_fp32, st)
             : launch_rms_bwd<__nv_bfloat16>(dx, dw, go, x, w, rms, partial, rows, cols, dw_fp32, st);
}

}  // extern "C"
