// Fused segmented LoRA product for ranks 33..128 on the 5th-generation tensor cores:
//   OUT[rows, N2] (+)= s2 * round(s1 * IN[rows, K1] . W1_seg) . W2_seg ,  MID written,
// the same operation as fused_kernel (smlm_fused.cuh; forward x -> v -> y of
// src/loquetier_src/kernel_utils.py:114-120 and backward gO -> dV -> dX of :142-143), for the
// ranks at which mma.sync can no longer keep up with HBM (rank 64 needs several hundred
// TFLOP/s to stay memory-bound).
//
// One CTA owns one tall piece: up to 128 rows of one segment, the M of one tcgen05.mma.
// Both contractions run as  tcgen05.mma.cta_group::1.kind::f16  issued by a single thread, with
// operands read from shared memory through matrix descriptors and fp32 accumulators in tensor
// memory (TMEM): acc1 [128 x KP] for the shrink, two [128 x 128] buffers for the expand.
//
// Warp roles (12 warps):
//   warp 0   TMA producer of IN: tiled tensor copies of [16 rows x 64 columns] boxes with the
//            128-byte swizzle, which is exactly the K-major SWIZZLE_128B operand layout;
//            in phase 3 it loads the W2 slabs together with warps 6 and 7.
//   warp 1   allocates TMEM, issues every MMA, signals completion with tcgen05.commit.
//   warps 2-5 load the W1 panel slices (16-byte cp.async into the swizzled operand layout,
//            completion counted on the stage's mbarrier) and run both epilogues: TMEM ->
//            registers (tcgen05.ld) -> storage type -> shared -> global (TMA tensor stores).
//   warps 8-11 share the second epilogue with them: of every 128-column group, warps 2-5 drain the
//            first 64 columns and warps 8-11 the second (measured: the drain, not the stores, bounds
//            the write phase - 0.8 us per group with four warps).
//
// Every wait is a bounded mbarrier wait; on a timeout the kernel records kErrTimeout, stops
// issuing work, still frees its TMEM and returns.
#pragma once
#include <cuda.h>

#include "smlm_common.cuh"

namespace smlm {

constexpr int kTcW2Warps = 3;   // warps that load W2 slabs: warp 0, 6, 7 and the last ones
constexpr int kTcThreads = 384 + (kTcW2Warps - 3) * 32;
constexpr int kTcRows = 128;   // rows of a tall piece = M of the MMA
constexpr int kTcNG = 128;     // OUT columns per MMA group of phase 3
constexpr int kTcW2Bufs = 4;   // W2 slabs in flight
// staging blocks per epilogue warp = tensor stores it keeps in flight
constexpr int tc_out_bufs(int r16) { return r16 >= 8 ? 2 : 4; }

constexpr int tc_chunks(int r16) { return r16 >= 8 ? 2 : 4; }  // 64-column chunks of IN per stage

template <int R16>
struct TcSmem {
  static constexpr int KP = R16 * 16;              // padded rank: 64 or 128
  static constexpr int NB = KP / 64;               // 64-wide rank blocks
  static constexpr int CH = tc_chunks(R16);
  static constexpr int KC = 64 * CH;               // K1 columns per ring stage
  static constexpr int kXBytes = CH * kTcRows * 128;          // CH chunks of [128 rows][128 B]
  static constexpr int kW1Bytes = KC * KP * 2;                // either layout
  static constexpr int kStage = kXBytes + kW1Bytes;
  static constexpr int kStages = 2;
  static constexpr int kRing = kStages * kStage;
  // phase 3 lives in the space of the ring: kTcW2Bufs W2 slabs [kTcNG x KP], then per epilogue warp
  // OB staging blocks of [32 rows][128 B]
  static constexpr int kW2Slab = kTcNG * KP * 2;
  static constexpr int kOutOff = kTcW2Bufs * kW2Slab;
  static constexpr int OB = tc_out_bufs(R16);
  static constexpr int kStageOut = 8 * OB * 4096;
  static constexpr int kPhase3 = kOutOff + kStageOut;
  static constexpr int kUnion = kRing > kPhase3 ? kRing : kPhase3;
  static constexpr int kMidOff = kUnion;                      // MID operand: NB blocks of [128 rows][128 B]
  static constexpr int kMid = NB * kTcRows * 128;
  static constexpr int kBarOff = kMidOff + kMid;
  static constexpr int kNumBars = 2 * kStages + 2 + 2 * kTcW2Bufs + 4;
  static constexpr int kTotal = kBarOff + kNumBars * 8 + 16 + 1024;
  static constexpr int kTmemCols = 512;                       // acc1 (KP) + 2 x 128, rounded up to a power of two
  static_assert(kTotal <= 227 * 1024, "shared memory budget");
};

struct TcArgs {
  void* out;                    // [T, N2]
  void* mid;                    // [T, R]
  const void* const* w1_table;
  const void* const* w2_table;
  const int32_t* ids;
  const float* scale;
  int* plan;                    // plan buffer: first header (error word), the tall list follows the first list
  int n_table;
  int K1, R, N2;
  int scale_mid;
  int accumulate;
  int independent;
  int mode;                     // kFusedBoth, kFusedShrinkOnly (MID = IN . W1 only) or kFusedExpandOnly (MID is read)
};

struct TcMaps {
  CUtensorMap in16;   // IN boxes of 16 rows x 64 columns
  CUtensorMap out16;  // OUT boxes of 16 rows x 64 columns
};

// ---- tcgen05 wrappers ----------------------------------------------------------------------
__device__ __forceinline__ void tc_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_dst), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_c, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n}\n"
      ::"r"(tmem_c), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc), "r"(0), "r"(0), "r"(0), "r"(0)
      : "memory");
}
// 32 lanes x 32 consecutive columns of fp32: thread i of the warp gets row (lane base + i)
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// 16-byte cp.async whose completion is counted on an mbarrier (one arrival per thread)
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
}

// Shared-memory matrix descriptors (SWIZZLE_128B, descriptor version 1).
// K-major operand: rows of 128 bytes (64 elements of K), groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
  return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}
// MN-major operand: rows are K, each row holds blocks of 64 MN elements (128 bytes); groups of 8
// K-rows 1024 bytes apart (stride byte offset), 64-wide MN blocks `lbo` bytes apart.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr, uint32_t lbo) {
  return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(lbo >> 4) << 16) |
         (static_cast<uint64_t>(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
template <typename T> struct TcFormat { static constexpr uint32_t value = 0u; };        // fp16
template <> struct TcFormat<__nv_bfloat16> { static constexpr uint32_t value = 1u; };
// Instruction descriptor of kind::f16: fp32 accumulator, A K-major, M = 128.
template <typename T>
__device__ __forceinline__ uint32_t tc_idesc(int n, bool b_mn_major) {
  const uint32_t fmt = TcFormat<T>::value;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((b_mn_major ? 1u : 0u) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(kTcRows >> 4) << 24);
}

template <typename T, int R16, bool RM>
__global__ void __launch_bounds__(kTcThreads, 1) fused_tc_kernel(const TcArgs a, const __grid_constant__ TcMaps tm) {
  extern __shared__ unsigned char smem_raw[];
  using SM = TcSmem<R16>;
  constexpr int KP = SM::KP, NB = SM::NB, CH = SM::CH, KC = SM::KC, S = SM::kStages;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;

  if (!a.independent) pdl_wait();
  pdl_trigger();
  // the tall list starts behind the first list, whose capacity is recorded in its header
  const int* tall = a.plan + kPlanHeaderInts + 4 * (a.plan[2] + 1);
  const int count = tall[0];
  const int piece_idx = blockIdx.x;
  if (piece_idx >= count) {
    if (a.independent) pdl_wait();
    return;
  }
  const Piece pc = reinterpret_cast<const Piece*>(tall + kPlanHeaderInts)[piece_idx];
  const int nrows = pc.nrows;
  const int K1 = a.K1, R = a.R, N2 = a.N2;
  int* err = a.plan + 1;
  const T* w1 = a.mode == kFusedExpandOnly ? nullptr
                                            : static_cast<const T*>(adapter_ptr(a.w1_table, a.ids, a.n_table, pc.seg, err));
  const T* w2 = a.mode == kFusedShrinkOnly ? nullptr
                                            : static_cast<const T*>(adapter_ptr(a.w2_table, a.ids, a.n_table, pc.seg, err));
  const bool w_ok = (a.mode == kFusedExpandOnly || w1 != nullptr) && (a.mode == kFusedShrinkOnly || w2 != nullptr);
  const float sc = adapter_scale(a.scale, a.ids, a.n_table, pc.seg);
  const float sc_mid = a.scale_mid ? sc : 1.0f;
  const float sc_out = a.scale_mid ? 1.0f : sc;

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t bar0 = base + SM::kBarOff;
  const uint32_t full0 = bar0, empty0 = bar0 + S * 8;
  const uint32_t acc1_full = bar0 + 2 * S * 8, mid_full = acc1_full + 8;
  const uint32_t w2_full0 = mid_full + 8, w2_empty0 = w2_full0 + 8 * kTcW2Bufs;
  const uint32_t acc2_full0 = w2_empty0 + 8 * kTcW2Bufs, acc2_empty0 = acc2_full0 + 16;
  const uint32_t tmem_slot = acc2_empty0 + 16;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - raw));

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full0 + s * 8, 1 + 128);  // the producer's expect_tx arrival + one per W1 loader thread
      mbar_init(empty0 + s * 8, 1);       // tcgen05.commit of the MMAs that read the stage
    }
    mbar_init(acc1_full, 1);
    mbar_init(mid_full, 128);
    for (int b = 0; b < kTcW2Bufs; ++b) {
      mbar_init(w2_full0 + b * 8, kTcW2Warps * 32);
      mbar_init(w2_empty0 + b * 8, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc2_full0 + b * 8, 1);
      mbar_init(acc2_empty0 + b * 8, 256);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tc_alloc(tmem_slot, SM::kTmemCols);
    tc_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;
  const uint32_t acc1 = tmem;               // columns [0, KP)
  const uint32_t acc2 = tmem + KP;          // two buffers of kTcNG columns

  // one half alone: the other half's loops run zero times (its barriers complete at once or are never waited for)
  const int ksteps = (w_ok && a.mode != kFusedExpandOnly) ? (K1 + KC - 1) / KC : 0;
  const int ngroups = (w_ok && a.mode != kFusedShrinkOnly) ? (N2 + kTcNG - 1) / kTcNG : 0;
  const int nblk = (nrows + 15) >> 4;
  bool dead = false;

  if (warp == 0) {
    // ============ phase 1: TMA producer of IN ============
    for (int it = 0; it < ksteps; ++it) {
      const int slot = it % S;
      const int k0 = it * KC;
      const uint32_t xs = base + slot * SM::kStage;
      const uint32_t fb = full0 + slot * 8;
      if (it >= S) mbar_wait(empty0 + slot * 8, ((it / S) - 1) & 1, err, dead);
      if (dead) break;  // nothing new is put in flight once a wait has given up
      const int nch = (min(KC, K1 - k0) + 63) >> 6;
      if (lane == 0) mbar_expect_tx(fb, 2048u * nblk * nch);
      __syncwarp();
      for (int i = lane; i < nblk * nch; i += 32) {
        const int b = i / nch, c = i - b * nch;
        tma_load_2d(xs + c * (kTcRows * 128) + b * 2048, &tm.in16, k0 + c * 64, pc.row0 + b * 16, fb);
      }
    }
  }
  if (warp == 0 || warp == 6 || warp == 7 || warp >= 12) {
    // ============ phase 3: three warps load the W2 slabs ============
    const int lt = (warp == 0 ? 0 : (warp >= 12 ? warp - 9 : warp - 5)) * 32 + lane;   // 0 .. 32 * kTcW2Warps - 1
    mbar_wait(acc1_full, 0, err, dead);  // the ring is no longer read once the shrink has completed
    for (int g = 0; g < ngroups; ++g) {
      const int buf = g % kTcW2Bufs;
      if (g >= kTcW2Bufs) mbar_wait(w2_empty0 + buf * 8, ((g / kTcW2Bufs) - 1) & 1, err, dead);
      if (dead) break;
      const int n0 = g * kTcNG;
      const int ncols = min(kTcNG, N2 - n0);
      const uint32_t ws = base + buf * SM::kW2Slab;
      if constexpr (!RM) {
        // W2 stored [N2][R] (K-major): per 64-wide rank block, [128 n-rows][128 B] swizzled
        for (int i = lt; i < kTcNG * NB * 8; i += kTcW2Warps * 32) {
          const int c = i & 7, n = (i >> 3) % kTcNG, blk = i / (8 * kTcNG);
          const int kcol = blk * 64 + c * 8;
          const bool ok = (n < ncols) && (kcol < R);
          const T* src = ok ? (w2 + static_cast<size_t>(n0 + n) * R + kcol) : w2;
          cp_async16(ws + blk * (kTcNG * 128) + n * 128 + ((c ^ (n & 7)) << 4), src, ok);
        }
      } else {
        // W2 stored [R][N2] (MN-major): per 64-column block, [KP k-rows][128 B] swizzled
        for (int i = lt; i < KP * (kTcNG / 64) * 8; i += kTcW2Warps * 32) {
          const int c = i & 7, k = (i >> 3) % KP, blk = i / (8 * KP);
          const int col = blk * 64 + c * 8;
          const bool ok = (k < R) && (col < ncols);
          const T* src = ok ? (w2 + static_cast<size_t>(k) * N2 + n0 + col) : w2;
          cp_async16(ws + blk * (KP * 128) + k * 128 + ((c ^ (k & 7)) << 4), src, ok);
        }
      }
      cp_async_arrive(w2_full0 + buf * 8);
    }
    cp_async_wait<0>();
  } else if (warp == 1) {
    // ============ the MMA issuer ============
    if (lane == 0) {
      // ---- phase 1: acc1 = IN . W1 ----
      const uint32_t idesc1 = tc_idesc<T>(KP, RM);
      for (int it = 0; it < ksteps; ++it) {
        const int slot = it % S;
        const uint32_t xs = base + slot * SM::kStage;
        const uint32_t ws = xs + SM::kXBytes;
        mbar_wait(full0 + slot * 8, (it / S) & 1, err, dead);
        fence_proxy_async();
        tc_fence_after();
        if (!dead) {
          const int k16 = (min(KC, K1 - it * KC) + 15) >> 4;
          for (int j = 0; j < k16; ++j) {
            const uint64_t ad = desc_kmajor(xs + (j >> 2) * (kTcRows * 128) + (j & 3) * 32);
            uint64_t bd;
            if constexpr (!RM) bd = desc_kmajor(ws + (j >> 2) * (KP * 128) + (j & 3) * 32);
            else bd = desc_mnmajor(ws + j * 2048, KC * 128);
            tc_mma(acc1, ad, bd, idesc1, (it > 0 || j > 0) ? 1u : 0u);
          }
        }
        tc_commit(empty0 + slot * 8);
      }
      tc_commit(acc1_full);
      // ---- phase 3: acc2[buf] = MID . W2 slab ----
      mbar_wait(mid_full, 0, err, dead);
      tc_fence_after();
      const uint32_t idesc2 = tc_idesc<T>(kTcNG, RM);
      const uint32_t mids = base + SM::kMidOff;
      for (int g = 0; g < ngroups; ++g) {
        const int buf = g & 1;              // accumulator buffer
        const int wbuf = g % kTcW2Bufs;     // W2 slab
        const uint32_t ws = base + wbuf * SM::kW2Slab;
        mbar_wait(w2_full0 + wbuf * 8, (g / kTcW2Bufs) & 1, err, dead);
        if (g >= 2) mbar_wait(acc2_empty0 + buf * 8, ((g >> 1) - 1) & 1, err, dead);
        fence_proxy_async();
        tc_fence_after();
        if (!dead) {
          for (int j = 0; j < KP / 16; ++j) {
            const uint64_t ad = desc_kmajor(mids + (j >> 2) * (kTcRows * 128) + (j & 3) * 32);
            uint64_t bd;
            if constexpr (!RM) bd = desc_kmajor(ws + (j >> 2) * (kTcNG * 128) + (j & 3) * 32);
            else bd = desc_mnmajor(ws + j * 2048, KP * 128);
            tc_mma(acc2 + buf * kTcNG, ad, bd, idesc2, j > 0 ? 1u : 0u);
          }
        }
        tc_commit(w2_empty0 + wbuf * 8);
        tc_commit(acc2_full0 + buf * 8);
      }
    }
    __syncwarp();
  } else {
    // ============ W1 loaders, then the epilogues (warps 2..5; warps 8..11 join for the second) ============
    const bool second = warp >= 8;              // drains columns 64..127 of every group, nothing else
    const int lt = tid - 64;                    // 0..127 for the W1 loaders
    const int sub = warp & 3;                   // TMEM subpartition this warp may read
    const int row = sub * 32 + lane;            // row of the piece held by this thread
    const uint32_t lane_base = static_cast<uint32_t>(sub * 32) << 16;
    for (int it = 0; !second && it < ksteps; ++it) {
      const int slot = it % S;
      const int k0 = it * KC;
      const uint32_t ws = base + slot * SM::kStage + SM::kXBytes;
      if (it >= S) mbar_wait(empty0 + slot * 8, ((it / S) - 1) & 1, err, dead);
      if (dead) break;
      if constexpr (!RM) {
        // W1 stored [R][K1] (K-major): per 64-column chunk of K, [KP rows][128 B] swizzled
        for (int i = lt; i < CH * KP * 8; i += 128) {
          const int c = i & 7, n = (i >> 3) % KP, ch = i / (8 * KP);
          const int kcol = k0 + ch * 64 + c * 8;
          const bool ok = (n < R) && (kcol < K1);
          const T* src = ok ? (w1 + static_cast<size_t>(n) * K1 + kcol) : w1;
          cp_async16(ws + ch * (KP * 128) + n * 128 + ((c ^ (n & 7)) << 4), src, ok);
        }
      } else {
        // W1 stored [K1][R] (MN-major): per 64-wide rank block, [KC k-rows][128 B] swizzled
        for (int i = lt; i < NB * KC * 8; i += 128) {
          const int c = i & 7, k = (i >> 3) % KC, blk = i / (8 * KC);
          const int n = blk * 64 + c * 8;
          const bool ok = (k0 + k < K1) && (n < R);
          const T* src = ok ? (w1 + static_cast<size_t>(k0 + k) * R + n) : w1;
          cp_async16(ws + blk * (KC * 128) + k * 128 + ((c ^ (k & 7)) << 4), src, ok);
        }
      }
      cp_async_arrive(full0 + slot * 8);
    }

    // ---- epilogue 1: acc1 -> MID (global, storage type) and the MID operand tile ----
    if (!second) {
      mbar_wait(acc1_full, 0, err, dead);
      tc_fence_after();
      const uint32_t mids = base + SM::kMidOff;
      T* mrow = static_cast<T*>(a.mid) + static_cast<size_t>(pc.row0 + row) * R;
#pragma unroll
      for (int blk = 0; blk < NB; ++blk) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t v[32];
          if (a.mode != kFusedExpandOnly) {
            tc_ld32(acc1 + lane_base + blk * 64 + h * 32, v);
            tc_wait_ld();
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {     // four 16-byte chunks of 8 elements
            uint32_t p[4];
            const int c = h * 4 + q;
            if (a.mode == kFusedExpandOnly) {
              // the expand alone: MID comes from global memory (rows past the piece and columns past R are zeros)
              uint4 m = make_uint4(0u, 0u, 0u, 0u);
              if (row < nrows && blk * 64 + c * 8 < R && w_ok) m = *reinterpret_cast<const uint4*>(mrow + blk * 64 + c * 8);
              p[0] = m.x; p[1] = m.y; p[2] = m.z; p[3] = m.w;
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int col = blk * 64 + h * 32 + q * 8 + e * 2;
                const float f0 = (w_ok && !dead && col < R) ? __uint_as_float(v[q * 8 + e * 2]) * sc_mid : 0.f;
                const float f1 = (w_ok && !dead && col + 1 < R) ? __uint_as_float(v[q * 8 + e * 2 + 1]) * sc_mid : 0.f;
                p[e] = pack2<T>(f0, f1);
              }
            }
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(mids + blk * (kTcRows * 128) + row * 128 +
                                                                         ((c ^ (row & 7)) << 4)),
                         "r"(p[0]), "r"(p[1]), "r"(p[2]), "r"(p[3])
                         : "memory");
            const int col0 = blk * 64 + c * 8;
            if (a.mode != kFusedExpandOnly && row < nrows && col0 < R && w_ok && !dead)
              *reinterpret_cast<uint4*>(mrow + col0) = make_uint4(p[0], p[1], p[2], p[3]);
          }
        }
      }
      tc_fence_before();
      fence_proxy_async();  // the MMA reads the MID tile through the async proxy
      mbar_arrive(mid_full);
    }

    // ---- epilogue 2: acc2[buf] -> OUT; this warp's 64 columns of every 128-column group ----
    constexpr int OB = SM::OB;
    const int half = second ? 1 : 0;
    const uint32_t ostage = base + SM::kOutOff + ((second ? warp - 4 : warp - 2)) * (OB * 4096);
    T* orow = static_cast<T*>(a.out) + static_cast<size_t>(pc.row0 + row) * N2;
    const int rows_here = min(32, nrows - sub * 32);   // rows of this warp that exist (may be <= 0)
    int obuf = 0;
    for (int g = 0; g < ngroups; ++g) {
      const int buf = g & 1;
      const int n0 = g * kTcNG;
      const int ncols = min(kTcNG, N2 - n0);
      mbar_wait(acc2_full0 + buf * 8, (g >> 1) & 1, err, dead);
      dead = __any_sync(0xffffffffu, dead);  // the warp leaves the store path together
      tc_fence_after();
      {   // one [32 rows][128 B] staging block
        if (lane == 0) bulk_wait_read<OB - 1>();
        __syncwarp();
        const uint32_t os = ostage + obuf * 4096;
        // both 32-column loads of the half are in flight before the one wait
        uint32_t v0[32], v1[32];
        tc_ld32(acc2 + buf * kTcNG + lane_base + half * 64, v0);
        tc_ld32(acc2 + buf * kTcNG + lane_base + half * 64 + 32, v1);
        tc_wait_ld();
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          uint32_t p[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t lo = q < 4 ? v0[q * 8 + e * 2] : v1[(q - 4) * 8 + e * 2];
            const uint32_t hi = q < 4 ? v0[q * 8 + e * 2 + 1] : v1[(q - 4) * 8 + e * 2 + 1];
            p[e] = pack2<T>(__uint_as_float(lo) * sc_out, __uint_as_float(hi) * sc_out);
          }
          asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(os + lane * 128 + ((q ^ (lane & 7)) << 4)),
                       "r"(p[0]), "r"(p[1]), "r"(p[2]), "r"(p[3])
                       : "memory");
        }
        // this warp's share is in registers / shared memory: the TMEM buffer may be overwritten once
        // all eight warps have said so
        tc_fence_before();
        mbar_arrive(acc2_empty0 + buf * 8);
        const int col0 = n0 + half * 64;
        if (col0 < n0 + ncols && rows_here > 0 && !dead) {
          fence_proxy_async();
          __syncwarp();
          // whole 16-row boxes go out as tensor stores; a ragged tail of rows as plain stores
          const int full_boxes = rows_here >= 32 ? 2 : (rows_here >= 16 ? 1 : 0);
          if (lane == 0) {
            for (int b = 0; b < full_boxes; ++b) {
              if (a.accumulate) tma_reduce_add_2d<T>(&tm.out16, col0, pc.row0 + sub * 32 + b * 16, os + b * 2048);
              else tma_store_2d(&tm.out16, col0, pc.row0 + sub * 32 + b * 16, os + b * 2048);
            }
            bulk_commit();
          }
          if (lane >= full_boxes * 16 && lane < rows_here) {
            for (int c = 0; c < 8; ++c) {
              const int col = half * 64 + c * 8;
              if (col < ncols) {
                uint4 vv;
                asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(vv.x), "=r"(vv.y), "=r"(vv.z), "=r"(vv.w)
                             : "r"(os + lane * 128 + ((c ^ (lane & 7)) << 4)));
                uint4* dst = reinterpret_cast<uint4*>(orow + n0 + col);
                if (a.accumulate) {
                  const uint4 old = *dst;
                  const uint32_t* ov = reinterpret_cast<const uint32_t*>(&old);
                  uint32_t* nv = reinterpret_cast<uint32_t*>(&vv);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 p0 = unpack2<T>(ov[e]);
                    const float2 p1 = unpack2<T>(nv[e]);
                    nv[e] = pack2<T>(p0.x + p1.x, p0.y + p1.y);
                  }
                }
                *dst = vv;
              }
            }
          }
          __syncwarp();
          obuf = (obuf + 1) % OB;
        }
      }
    }
    if (lane == 0) bulk_wait<0>();
    __syncwarp();
  }

  // everyone is done with tensor memory: hand it back
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tc_dealloc(tmem, SM::kTmemCols);
  if (a.independent) pdl_wait();
}

}  // namespace smlm
