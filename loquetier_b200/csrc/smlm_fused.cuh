// Fused segmented LoRA product  OUT[rows, N2] (+)= s2 * round(s1 * IN[rows, K1] . W1_seg) . W2_seg
// for every piece (<= 64 rows of one segment): a shrink through the rank-R
// bottleneck followed at once by the expand, in one kernel, with the rank-R
// intermediate MID also written out in the storage type.
//
//   forward : IN = x,  W1 = A, W2 = B, MID = v,  OUT = y   (the two operator calls of
//             add_lora.forward, src/loquetier_src/kernel_utils.py:114-120, plus the
//             scale and add of MixedLoraLinear.forward, models/mixed_lora.py:214-217)
//   backward: IN = gO, W1 = B, W2 = A, MID = dV, OUT = dX  (kernel_utils.py:142-143)
//
// A gather piece (Piece::pad = 1, from a grouped plan) holds rows of short segments that share an
// adapter but not a place in the batch: each row's slice of a ring stage arrives as one untiled bulk copy
// (1 KB; one tensor copy per row and 64-column chunk moved 128 bytes at a time and ran at a fraction of
// the speed) into rows padded by 16 bytes, which keeps ldmatrix free of bank conflicts without a
// swizzle; MID and OUT rows go out through the row index; everything between is the same.  This is the decode (BGMV-style) case with the adapter's panels streamed once.
//
// The same kernel also runs either half alone (FusedArgs::mode), which is one call of the
// reference operator smlm_forward_cutlass: shrink only (MID is the result) or expand only
// (MID is the input).
//
// It replaces two launches of the reference's grouped GEMM
// (kernel_src/csrc/smlm_forward/smlm_forward_cutlass.cuh:82-171) and keeps its
// numerics: fp32 accumulation, MID rounded to the storage type before the second
// product.
//
// One CTA per SM; one cluster of KS CTAs owns one piece.
// Phase 1 - the HBM-bound read.  Every CTA streams its slice of the K1 columns of IN
//   through a ring of large shared-memory stages fed by a producer warp with TMA.
//   A stage holds 64 rows x (64*CH) columns, fetched as [16 rows x 64 columns] tiled
//   tensor copies (128-byte swizzle) issued row block by row block, so that each
//   row's consecutive 128-byte chunks - up to 1 KB - are requested together and DRAM
//   pages are used whole; the W1 panel slice arrives as untiled bulk copies from its
//   raw pointer.  Eight consumer warps run ldmatrix + mma.sync m16n8k16.
// Phase 2.  The CTAs of the cluster add their partial sums through distributed
//   shared memory in a fixed order (deterministic; no global scratch, no atomics);
//   every CTA ends up with the whole MID tile.
// Phase 3 - the HBM-bound write.  Every CTA expands MID against its slice of the N2
//   columns, one slab at a time (W2 slab double-buffered with 16-byte cp.async).  A warp
//   owns 64-column groups of the slab and walks down the piece's row blocks with the W2
//   fragments of its group held in registers (ranks up to 32), so a 16 x 64 block costs
//   eight MMAs, the conversion and four stmatrix; the blocks go to TMA as tensor stores -
//   or tensor reduce-adds when accumulating into OUT.  A scale that is a power of two is
//   folded into the MID operand (exact), which removes the multiply from this phase.
//
// One launch can serve several jobs - the same segment plan, adapter ids, rank and scale
// applied to different tensors, e.g. the q/k/v or gate/up projections of one layer, or all
// LoRA targets of a benchmark step: the grid is the jobs' grids laid end to end, so that
// short launches do not each pay their own set-up and drain.
#pragma once
#include <cooperative_groups.h>
#include <cuda.h>

#include <type_traits>

#include "smlm_common.cuh"

namespace smlm {

namespace cg = cooperative_groups;

constexpr int kFusedConsumers = 8;                           // consumer warps
constexpr int kFusedThreads = (kFusedConsumers + 1) * 32;    // + one producer warp
constexpr int kFusedCThreads = kFusedConsumers * 32;

#ifndef SMLM_FUSED_CH
#define SMLM_FUSED_CH 8
#endif
// 64-column chunks of IN per ring stage; high ranks trade width for panel space
// Rank <= 16 is sized so that two CTAs fit on one SM: an independent successor launch can then
// move in and read while this launch is still writing.
constexpr int fused_chunks(int r16) { return r16 >= 8 ? 2 : (r16 == 4 ? 4 : (r16 == 2 ? SMLM_FUSED_CH : 4)); }
constexpr int fused_stages(int) { return 2; }
constexpr int fused_slab(int r16) { return r16 >= 8 ? 128 : (r16 == 4 ? 256 : (r16 == 2 ? 1024 : 512)); }
constexpr int fused_ctas_per_sm(int r16) { return r16 == 1 ? 2 : 1; }

struct FusedMaps {
  CUtensorMap in8;    // IN boxes of 8 rows x 64 columns (pieces of at most 8 rows)
  CUtensorMap in16;   // IN boxes of 16 rows x 64 columns
  CUtensorMap out;    // OUT boxes of 16 rows x 64 columns
  CUtensorMap out8;   // OUT boxes of 8 rows x 64 columns (last block of a piece of 8k rows)
};

template <int R16, bool RM>
struct FusedSmem {
  static constexpr int NT = R16 * 2;            // n-tiles of 8 in the shrink
  static constexpr int KP = R16 * 16;           // padded rank
  static constexpr int CH = fused_chunks(R16);
  static constexpr int KC = 64 * CH;            // K1 columns per ring stage
  static constexpr int WPad = KC * 2 + 16;      // bytes between W1 rows in shared memory ([R][K1] layout)
  static constexpr int XPad = KC * 2 + 16;      // bytes between the rows of a gather piece in a ring stage
  static_assert(kGatherRows * XPad <= kBM * KC * 2, "a gather piece must fit the stage's IN region");
  static constexpr int kStages = fused_stages(R16);
  static constexpr int kXBytes = kBM * KC * 2;  // 4 row blocks x CH column chunks of [16][64]
  static constexpr int kW1Raw = RM ? KC * KP * 2 : KP * WPad;
  static constexpr int kW1Bytes = (kW1Raw + 1023) / 1024 * 1024;
  static constexpr int kStage = kXBytes + kW1Bytes;
  static constexpr int kRing = kStages * kStage;
  // phase 3 lives in the space of the ring: two W2 slabs, then per warp two 16 x 128 staging blocks
  static constexpr int SLAB = fused_slab(R16);
  static constexpr int kW2Slab = SLAB * KP * 2;
  static constexpr int kOutOff = 2 * kW2Slab;
  static constexpr int kStageOut = kFusedConsumers * 2 * 4096;
  static constexpr int kPhase3 = kOutOff + kStageOut;
  static constexpr int kUnion = kRing > kPhase3 ? kRing : kPhase3;
  static constexpr int kRedOff = kUnion;
  static constexpr int kRed = kFusedConsumers * 16 * KP * 4;   // one 16 x KP fp32 block per consumer warp
  static constexpr int kMidOff = kRedOff + kRed;
  static constexpr int kMid = kBM * KP * 2;
  static constexpr int kRowOff = kMidOff + kMid;                  // int[kBM]: token rows of a gather piece
  static constexpr int kBarOff = kRowOff + kBM * 4;
  static constexpr int kTotal = kBarOff + 2 * kStages * 8 + 1024;  // + alignment slack
  static_assert(kTotal <= (fused_ctas_per_sm(R16) == 2 ? 113 : 227) * 1024, "shared memory budget");
  static_assert(kW2Slab % 1024 == 0 && kStage % 1024 == 0, "swizzled tiles need 1024-byte alignment");
};

constexpr int kFusedMaxJobs = 8;   // jobs one launch can serve

// What differs between the jobs of one launch: the tensors and the two large dimensions.
struct FusedJob {
  const void* in;               // [T, K1] (gather pieces read it through this pointer, the others through TMA)
  void* out;                    // [T, N2]
  void* mid;                    // [T, R]
  const void* const* w1_table;  // shrink panels
  const void* const* w2_table;  // expand panels
  int K1, N2;
  int accumulate;               // OUT += instead of OUT =
  int pad_;
};

struct FusedArgs {
  FusedJob job[kFusedMaxJobs];
  const int32_t* ids;           // per-segment adapter index, or null: tables are per segment
  const float* scale;           // per adapter (ids != null) or per segment, or null
  int* plan;
  int n_table;
  int R;
  int ksplit;
  // The grid is cut into groups of jobs of the same size; inside a group the jobs' pieces alternate
  // (cluster c of a group of n jobs serves job c % n, piece c / n), so that CTAs resident side by
  // side belong to different jobs - a projection that mostly writes next to one that mostly reads -
  // and both directions of HBM stay busy.  Groups are ordered longest job first, so that the launch
  // ends on its shortest CTAs.
  int ngroups;
  int grp_cta_begin[kFusedMaxJobs + 1];   // first CTA of every group (and the end of the grid)
  int grp_job_begin[kFusedMaxJobs + 1];   // first job of every group (and the number of jobs)
  int scale_mid;                // 1: the scale multiplies MID (backward); 0: it multiplies OUT (forward)
  int independent;              // 1: see smlm_b200_fwd in include/smlm_b200.h
  int mode;                     // kFusedBoth, or one half only (one reference operator call):
                                // kFusedShrinkOnly: MID = s * IN . W1, nothing else;
                                // kFusedExpandOnly: OUT (+)= s * MID . W2 with MID read, not written
};

struct FusedMapsN {
  FusedMaps m[kFusedMaxJobs];
};


__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

template <typename T, int R16, bool RM, bool GATHER>
__global__ void __launch_bounds__(kFusedThreads, fused_ctas_per_sm(R16)) fused_kernel(
    const __grid_constant__ FusedArgs a, const __grid_constant__ FusedMapsN tmn) {
  extern __shared__ unsigned char smem_raw[];
  using SM = FusedSmem<R16, RM>;
  constexpr int NT = SM::NT;
  constexpr int KP = SM::KP;
  constexpr int S = SM::kStages;
  constexpr int CH = SM::CH;
  constexpr int KC = SM::KC;
  constexpr int WPad = SM::WPad;
  constexpr int SLAB = SM::SLAB;
  constexpr int XC = R16 * 2;  // 16-byte chunks per MID row
  constexpr int NW = kFusedConsumers;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int KS = a.ksplit;
  // the grid is the groups' grids laid end to end; a cluster never straddles two pieces
  int grp = 0;
  for (int i = 1; i < a.ngroups; ++i)
    if (static_cast<int>(blockIdx.x) >= a.grp_cta_begin[i]) grp = i;
  const int local = blockIdx.x - a.grp_cta_begin[grp];
  const int gjobs = a.grp_job_begin[grp + 1] - a.grp_job_begin[grp];
  const int cl = local / KS;
  const int z = local - cl * KS;
  const int jidx = a.grp_job_begin[grp] + cl % gjobs;
  const int piece_idx = cl / gjobs;
  const FusedJob& jb = a.job[jidx];
  const FusedMaps& tm = tmn.m[jidx];

  // A launch that depends on its predecessor waits for it here.  An independent one starts at
  // once - it overlaps its read phase with the predecessor's write phase - and waits just before
  // it exits instead, so that completion still happens in stream order.
  if (!a.independent) pdl_wait();
  pdl_trigger();  // the next launch of the stream may be scheduled as soon as there is room
  const int count = a.plan[0];
  const Piece pc = reinterpret_cast<const Piece*>(a.plan + kPlanHeaderInts)[piece_idx];
  if (piece_idx >= count) {  // the whole cluster leaves together
    if (a.independent) pdl_wait();
    return;
  }
  const int nrows = pc.nrows;
  const int K1 = jb.K1, R = a.R, N2 = jb.N2;
  int* err = a.plan + 1;
  // GATHER is a compile-time switch because the extra paths cost the ordinary launch about 3 %: only
  // launches whose caller announces a grouped plan run the instantiation that knows gather pieces
  const bool gather = GATHER && pc.pad != 0;
  if (!GATHER && pc.pad != 0) {  // a grouped plan handed to a launch that was not told so: refuse the piece
    if (tid == 0) atomicOr(a.plan + 1, kErrGrouped);
    if (a.independent) pdl_wait();
    return;
  }
  // rows of a gather piece; its adapter index sits in the piece itself
  const int* rowidx = gather ? plan_row_index(a.plan) + pc.row0 : nullptr;
  if (gather && a.ids == nullptr && tid == 0) atomicOr(err, kErrBadIndex);  // grouped plans need the adapter table

  const int mode = a.mode;
  const T* w1 = nullptr;
  const T* w2 = nullptr;
  float sc = 1.0f;
  if (!gather) {
    if (mode != kFusedExpandOnly) w1 = static_cast<const T*>(adapter_ptr(jb.w1_table, a.ids, a.n_table, pc.seg, err));
    if (mode != kFusedShrinkOnly) w2 = static_cast<const T*>(adapter_ptr(jb.w2_table, a.ids, a.n_table, pc.seg, err));
    sc = adapter_scale(a.scale, a.ids, a.n_table, pc.seg);
  } else if (a.ids != nullptr && pc.seg >= 0 && pc.seg < a.n_table) {
    if (mode != kFusedExpandOnly) w1 = static_cast<const T*>(adapter_ptr(jb.w1_table, nullptr, a.n_table, pc.seg, err));
    if (mode != kFusedShrinkOnly) w2 = static_cast<const T*>(adapter_ptr(jb.w2_table, nullptr, a.n_table, pc.seg, err));
    sc = a.scale != nullptr ? a.scale[pc.seg] : 1.0f;
  }
  const bool w_ok = (w1 != nullptr || mode == kFusedExpandOnly) && (w2 != nullptr || mode == kFusedShrinkOnly) &&
                    !(gather && a.ids == nullptr);
  const float sc_mid = (a.scale_mid || mode == kFusedShrinkOnly) ? sc : 1.0f;
  const float sc_out = (a.scale_mid || mode == kFusedShrinkOnly) ? 1.0f : sc;
  // A scale of 2, 4, ... 256 multiplies the MID operand of the second product instead of every output
  // element: scaling by a power of two is exact in the storage type (bf16 has the exponent range of
  // fp32, so nothing overflows that would not overflow in OUT as well; fp16 could, and is left alone),
  // hence the result is bit-identical and the write phase saves one multiply per element.  MID as
  // written to global memory never carries this factor.
  const bool fold = std::is_same<T, __nv_bfloat16>::value && sc_out >= 2.0f && sc_out <= 256.0f &&
                    (__float_as_uint(sc_out) & 0x007fffffu) == 0u;
  const float sc_w = fold ? 1.0f : sc_out;

  const int ksteps = (K1 + KC - 1) / KC;
  const int per = (ksteps + KS - 1) / KS;
  const int kbeg = z * per;
  const int nk = (w_ok && mode != kFusedExpandOnly) ? max(0, min(ksteps, kbeg + per) - kbeg) : 0;
  // CTAs walk their K slice from different starting points so that, at any moment, the machine as
  // a whole reads many different column bands of IN (and all DRAM channels) instead of one
  const int krot = nk > 0 ? (piece_idx * 5) % nk : 0;

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* smem = smem_raw + (base - raw);
  const uint32_t full0 = base + SM::kBarOff;
  const uint32_t empty0 = full0 + S * 8;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < S; ++s) {
      mbar_init(full0 + s * 8, 1);
      mbar_init(empty0 + s * 8, NW);
    }
    fence_mbar_init();
  }
  // token rows of the piece, looked up once (a gather piece's rows come from the plan's row index)
  int* const rowsm = reinterpret_cast<int*>(smem + SM::kRowOff);
  if (tid < kBM) rowsm[tid] = gather ? (tid < nrows ? rowidx[tid] : 0) : pc.row0 + tid;
  if (gather && (K1 & 15) != 0 && tid < nrows) {
    // the last 16-column step of a row reaches 8 columns past K1, which a bulk copy does not fill:
    // clear them in every stage (W1 holds zeros there, but zero times a non-finite leftover is not zero)
    const int tail = (K1 % KC) * 2;
    for (int s = 0; s < S; ++s)
      *reinterpret_cast<uint4*>(smem + s * SM::kStage + tid * SM::XPad + tail) = make_uint4(0, 0, 0, 0);
    fence_proxy_async();
  }
  if ((K1 % 64) != 0) {
    // the last 64-column chunk is only partly overwritten by the panel copies: start from zeros so
    // that the columns past K1 (which IN supplies as zeros) never meet a non-finite leftover
    for (int s = 0; s < S; ++s) {
      uint4* wz = reinterpret_cast<uint4*>(smem + s * SM::kStage + SM::kXBytes);
      for (int i = tid; i < SM::kW1Bytes / 16; i += kFusedThreads) wz[i] = make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async();
  }
  __syncthreads();

  // consumer warp roles: WM row blocks of 16, WK ways along K (phase 1) or along N2 (phase 3)
  const int WM = nrows <= 16 ? 1 : (nrows <= 32 ? 2 : 4);
  const int WK = NW / WM;
  const int wm = warp % WM;
  const int wk = warp / WM;
  bool dead = false;

  // ======================= phase 1: shrink over this CTA's K1 slice =======================
  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

  if (warp == NW) {
    // rows are fetched in blocks of 16, the last block with the 8-row box when that covers it:
    // nothing beyond the piece's rows (rounded up to 8) is read
    const int nblk = (nrows + 15) >> 4;
    const bool last8 = ((nrows - 1) & 15) < 8;
    const uint32_t rowbytes = static_cast<uint32_t>(nblk * 16 - (last8 ? 8 : 0)) * 128u;  // per 64-column chunk
    for (int it = 0; it < nk; ++it) {
      const int slot = it % S;
      const int kstep = kbeg + (it + krot < nk ? it + krot : it + krot - nk);
      const int k0 = kstep * KC;
      const uint32_t xs = base + slot * SM::kStage;
      const uint32_t ws = xs + SM::kXBytes;
      const uint32_t fb = full0 + slot * 8;
      if (it >= S) mbar_wait(empty0 + slot * 8, ((it / S) - 1) & 1, err, dead);
      const int kcols = min(KC, K1 - k0);
      const int nch = (kcols + 63) >> 6;
      const uint32_t wbytes = static_cast<uint32_t>(kcols) * R * 2;
      if (gather && (kcols & 15) != 0 && it >= S) {
        // the slot held a full step before: the 8 columns past kcols that the last 16-column step
        // reads carry that step's data, not the zeros written before the loop.  The consumers have
        // released the slot (the wait above) and see these stores through the barrier's release.
        for (int r = lane; r < nrows; r += 32)
          *reinterpret_cast<uint4*>(smem + slot * SM::kStage + r * SM::XPad + kcols * 2) = make_uint4(0, 0, 0, 0);
        __syncwarp();
      }
      if (lane == 0)
        mbar_expect_tx(fb, (gather ? static_cast<uint32_t>(nrows) * kcols * 2 : rowbytes * nch) + wbytes);
      __syncwarp();
      if constexpr (!RM) {
        for (int n = lane; n < R; n += 32)
          bulk_load(ws + n * WPad, w1 + static_cast<size_t>(n) * K1 + k0, kcols * 2, fb);
      } else {
        if (lane == 0) bulk_load(ws, w1 + static_cast<size_t>(k0) * R, wbytes, fb);
      }
      if (!gather) {
        for (int i = lane; i < nblk * nch; i += 32) {
          const int b = i / nch, c = i - b * nch;
          tma_load_2d(xs + (b * CH + c) * 2048, (last8 && b == nblk - 1) ? &tm.in8 : &tm.in16, k0 + c * 64,
                      pc.row0 + b * 16, fb);
        }
      } else {
        // one bulk copy per row: its kcols columns of this K step, into rows XPad bytes apart
        const T* in = static_cast<const T*>(jb.in);
        for (int r = lane; r < nrows; r += 32)
          bulk_load(xs + r * SM::XPad, in + static_cast<size_t>(rowidx[r]) * K1 + k0, kcols * 2, fb);
      }
    }
  } else {
    const bool active = (wm * 16 < nrows);
    // the loop exists twice, once per stage layout, so that the common one carries no test per step
    auto consume = [&](auto gathered) {
      constexpr bool G = decltype(gathered)::value;
      for (int it = 0; it < nk; ++it) {
        const int slot = it % S;
        const uint32_t xs = base + slot * SM::kStage;
        const uint32_t ws = xs + SM::kXBytes;
        mbar_wait(full0 + slot * 8, (it / S) & 1, err, dead);
        if (active) {
          const int kstep = kbeg + (it + krot < nk ? it + krot : it + krot - nk);
          const int kmax = (min(KC, K1 - kstep * KC) + 15) >> 4;
          for (int kk = wk; kk < kmax; kk += WK) {
            uint32_t af[4];
            {
              const int m = lane >> 3;
              const int r = (m & 1) * 8 + (lane & 7);
              const int c = (kk & 3) * 2 + (m >> 1);
              if constexpr (!G) ldsm_x4(af, xs + (wm * CH + (kk >> 2)) * 2048 + r * 128 + ((c ^ (r & 7)) << 4));
              else ldsm_x4(af, xs + (wm * 16 + r) * SM::XPad + kk * 32 + (m >> 1) * 16);
            }
#pragma unroll
            for (int j = 0; j < NT; j += 2) {
              uint32_t bf[4];
              const int m = lane >> 3;
              if constexpr (!RM) {
                const int n = (j + (m >> 1)) * 8 + (lane & 7);
                ldsm_x4(bf, ws + n * WPad + ((kk * 2 + (m & 1)) << 4));
              } else {
                // panel stored [K1][R] with rows of R elements, exactly as in global memory
                const int k = kk * 16 + (m & 1) * 8 + (lane & 7);
                ldsm_x4_t(bf, ws + k * (R * 2) + ((j + (m >> 1)) << 4));
              }
              mma16816<T>(acc[j], af, bf[0], bf[1]);
              mma16816<T>(acc[j + 1], af, bf[2], bf[3]);
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + slot * 8);
      }
    };
    if (gather) consume(std::true_type{});
    else consume(std::false_type{});
  }

  // ======================= phase 2: reduce the K1 slices, build MID =======================
  float* red = reinterpret_cast<float*>(smem + SM::kRedOff);  // [warp][16][KP]
  if (warp < NW) {
    const int g = lane >> 2, t = lane & 3;
    float* my = red + warp * 16 * KP;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      *reinterpret_cast<float2*>(my + g * KP + j * 8 + 2 * t) = make_float2(acc[j][0], acc[j][1]);
      *reinterpret_cast<float2*>(my + (g + 8) * KP + j * 8 + 2 * t) = make_float2(acc[j][2], acc[j][3]);
    }
  }
  cg::cluster_group cluster = cg::this_cluster();
  const bool reduce_cluster = KS > 1 && mode != kFusedExpandOnly;
  if (reduce_cluster) {
    cluster_arrive();
    cluster_wait();
  } else {
    __syncthreads();
  }

  const uint32_t mids = base + SM::kMidOff;  // MID tile [64][KP] in the storage type, swizzled rows
  {
    const int load_rows = min(kBM, ((nrows + 15) >> 4) << 4);
    T* const mbase = static_cast<T*>(jb.mid);
    constexpr int HP = KP / 2;
    for (int e = tid; e < load_rows * HP; e += kFusedThreads) {
      const int r = e / HP;
      const int n = (e - r * HP) * 2;
      const int fm = r >> 4, r16 = r & 15;
      const bool inside = r < nrows && n < R && w_ok;
      T* mrow = inside ? mbase + static_cast<size_t>(rowsm[r]) * R + n : mbase;
      uint32_t packed = 0;
      if (mode == kFusedExpandOnly) {
        if (inside) packed = *reinterpret_cast<const uint32_t*>(mrow);
      } else {
        float2 s = make_float2(0.f, 0.f);
        if (inside) {
          for (int cz = 0; cz < KS; ++cz) {
            const float* rr = KS > 1 ? cluster.map_shared_rank(red, cz) : red;
            for (int q = 0; q < WK; ++q) {
              const float2 p = *reinterpret_cast<const float2*>(rr + ((q * WM + fm) * 16 + r16) * KP + n);
              s.x += p.x;
              s.y += p.y;
            }
          }
        }
        packed = pack2<T>(s.x * sc_mid, s.y * sc_mid);
        if (z == 0 && inside) *reinterpret_cast<uint32_t*>(mrow) = packed;
      }
      if (fold) {
        const float2 f = unpack2<T>(packed);
        packed = pack2<T>(f.x * sc_out, f.y * sc_out);
      }
      const int c = n >> 3;
      asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(mids + r * (XC * 16) + (swz<XC>(r, c) << 4) + (n & 7) * 2),
                   "r"(packed));
    }
  }
  // done reading the peers' partial sums; the matching wait sits at the very end, so that no CTA
  // leaves (and frees its shared memory) while a peer may still be reading it
  if (reduce_cluster) cluster_arrive();
  __syncthreads();  // MID is complete; the ring is free for phase 3

  // ======================= phase 3: expand over this CTA's N2 slice =======================
  const int nslabs = (N2 + SLAB - 1) / SLAB;
  const int sper = (nslabs + KS - 1) / KS;
  const int sbeg = z * sper;
  const int ns = (w_ok && mode != kFusedShrinkOnly) ? max(0, min(nslabs, sbeg + sper) - sbeg) : 0;

  if (warp < NW && ns > 0) {
    const uint32_t wslab0 = base;  // two slabs in the space the ring occupied
    const int kchunks = R >> 3;
    const int ctid = tid;          // consumer threads are 0 .. kFusedCThreads-1

    auto load_slab = [&](int buf, int slab) {
      const int n0 = slab * SLAB;
      const int ncols = min(SLAB, N2 - n0);
      const uint32_t ws = wslab0 + buf * SM::kW2Slab;
      if constexpr (!RM) {
        // W2 stored [N2][R]: the slab is one contiguous block of global memory
        for (int i = ctid; i < ncols * XC; i += kFusedCThreads) {
          const int n = i / XC, c = i - n * XC;
          const bool ok = c < kchunks;
          const T* src = ok ? (w2 + static_cast<size_t>(n0 + n) * R + c * 8) : w2;
          cp_async16(ws + n * (XC * 16) + (swz<XC>(n, c) << 4), src, ok);
        }
      } else {
        // W2 stored [R][N2]: KP rows of SLAB/8 chunks
        constexpr int CPR = SLAB / 8;
        const int cvalid = ncols >> 3;
        for (int i = ctid; i < KP * CPR; i += kFusedCThreads) {
          const int k = i / CPR, c = i - k * CPR;
          if (c >= cvalid) continue;
          const bool ok = k < R;
          const T* src = ok ? (w2 + static_cast<size_t>(k) * N2 + n0 + c * 8) : w2;
          cp_async16(ws + k * (SLAB * 2) + (((c & ~7) | ((c ^ k) & 7)) << 4), src, ok);
        }
      }
    };

    // same idea for the write phase: start at a different slab per piece
    const int srot = (piece_idx * 3) % ns;
    auto slab_of = [&](int si) { return sbeg + (si + srot < ns ? si + srot : si + srot - ns); };
    load_slab(0, slab_of(0));
    cp_async_commit();

    // A warp owns 64-column groups of the slab (group = warp, warp + 8, ...) and walks down the
    // piece's row blocks of 16.  Up to rank 32 the W2 fragments of a group are fetched once and
    // serve all row blocks.
    constexpr bool kHold = R16 <= 2;
    const int nblk = (nrows + 15) >> 4;
    auto load_a = [&](uint32_t (&dst)[R16][4], int rb) {
#pragma unroll
      for (int kk = 0; kk < R16; ++kk) {
        const int m = lane >> 3;
        const int r = rb * 16 + (m & 1) * 8 + (lane & 7);
        const int c = kk * 2 + (m >> 1);
        ldsm_x4(dst[kk], mids + r * (XC * 16) + (swz<XC>(r, c) << 4));
      }
    };
    // per warp four staging blocks of 16 x 64 (2 KB): the tensor stores in flight
    const uint32_t ostage = base + SM::kOutOff + warp * 8192;
    T* const obase = static_cast<T*>(jb.out);
    const int accumulate = jb.accumulate;
    int oslot = 0;

    for (int si = 0; si < ns; ++si) {
      const int slab = slab_of(si);
      const int n0 = slab * SLAB;
      const int ncols = min(SLAB, N2 - n0);
      if (si + 1 < ns) load_slab((si + 1) & 1, slab_of(si + 1));
      cp_async_commit();
      cp_async_wait<1>();
      named_bar_sync(1, kFusedCThreads);  // slab si has landed for all consumer warps
      const uint32_t ws = wslab0 + (si & 1) * SM::kW2Slab;
      const int ngroups = (ncols + 63) >> 6;
      for (int grp = warp; grp < ngroups; grp += NW) {
        // W2 fragments of this group: bfr[kk][jj] covers n-tiles 2jj, 2jj+1 at k step kk
        auto load_b = [&](uint32_t (&dst)[4], int kk, int jj) {
          const int m = lane >> 3;
          if constexpr (!RM) {
            const int n = grp * 64 + (2 * jj + (m >> 1)) * 8 + (lane & 7);
            const int c = kk * 2 + (m & 1);
            ldsm_x4(dst, ws + n * (XC * 16) + (swz<XC>(n, c) << 4));
          } else {
            const int k = kk * 16 + (m & 1) * 8 + (lane & 7);
            const int c = grp * 8 + 2 * jj + (m >> 1);
            ldsm_x4_t(dst, ws + k * (SLAB * 2) + (((c & ~7) | ((c ^ k) & 7)) << 4));
          }
        };
        uint32_t bfr[kHold ? R16 : 1][4][4];
        if constexpr (kHold) {
#pragma unroll
          for (int kk = 0; kk < R16; ++kk)
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) load_b(bfr[kk][jj], kk, jj);
        }
#pragma unroll
        for (int rb = 0; rb < 4; ++rb) {
          if (rb >= nblk) break;
          float o[8][4];
          uint32_t af[R16][4];   // the row block's MID fragments: one ldmatrix per k step and 16 x 64 block
          load_a(af, rb);
#pragma unroll
          for (int kk = 0; kk < R16; ++kk)
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              if constexpr (!kHold) load_b(bfr[0][jj], kk, jj);
              const uint32_t (&b4)[4] = bfr[kHold ? kk : 0][jj];
              if (kk == 0) {
                mma16816_z<T>(o[2 * jj], af[kk], b4[0], b4[1]);
                mma16816_z<T>(o[2 * jj + 1], af[kk], b4[2], b4[3]);
              } else {
                mma16816<T>(o[2 * jj], af[kk], b4[0], b4[1]);
                mma16816<T>(o[2 * jj + 1], af[kk], b4[2], b4[3]);
              }
            }
          if (sc_w != 1.0f) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              o[j][0] *= sc_w; o[j][1] *= sc_w; o[j][2] *= sc_w; o[j][3] *= sc_w;
            }
          }
          if (lane == 0) bulk_wait_read<3>();  // the staging block about to be reused has been read
          __syncwarp();
          const uint32_t os = ostage + oslot * 2048;
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            const int m = lane >> 3;
            const int r = (m & 1) * 8 + (lane & 7);
            const int c = j + (m >> 1);
            stsm_x4(os + r * 128 + ((c ^ (r & 7)) << 4), pack2<T>(o[j][0], o[j][1]), pack2<T>(o[j][2], o[j][3]),
                    pack2<T>(o[j + 1][0], o[j + 1][1]), pack2<T>(o[j + 1][2], o[j + 1][3]));
          }
          const int rows_here = min(16, nrows - rb * 16);
          if (!gather && (rows_here == 16 || rows_here == 8)) {
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              const CUtensorMap* omap = rows_here == 8 ? &tm.out8 : &tm.out;
              if (accumulate) tma_reduce_add_2d<T>(omap, n0 + grp * 64, pc.row0 + rb * 16, os);
              else tma_store_2d(omap, n0 + grp * 64, pc.row0 + rb * 16, os);
              bulk_commit();
            }
            oslot = (oslot + 1) & 3;
          } else {
            // ragged tail of the piece, or a gather piece: plain 16-byte stores of the rows that exist
            __syncwarp();
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int i = q * 32 + lane;
              const int r = i >> 3, c = i & 7;
              const int col = grp * 64 + c * 8;
              if (r < rows_here && col < ncols) {
                uint4 v;
                asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                             : "r"(os + r * 128 + ((c ^ (r & 7)) << 4)));
                uint4* dst = reinterpret_cast<uint4*>(obase + static_cast<size_t>(rowsm[rb * 16 + r]) * N2 + n0 + col);
                if (accumulate) {
                  const uint4 old = *dst;
                  const uint32_t* ov = reinterpret_cast<const uint32_t*>(&old);
                  uint32_t* nv = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 p = unpack2<T>(ov[e]);
                    const float2 n2 = unpack2<T>(nv[e]);
                    nv[e] = pack2<T>(p.x + n2.x, p.y + n2.y);
                  }
                }
                *dst = v;
              }
            }
            __syncwarp();
          }
        }
      }
      named_bar_sync(1, kFusedCThreads);  // everyone is done with slab si before it is refilled
    }
    if (lane == 0) bulk_wait<0>();  // shared memory must outlive the tensor stores that read it
    __syncwarp();
  }
  if (reduce_cluster) cluster_wait();
  if (a.independent) pdl_wait();
}

}  // namespace smlm
