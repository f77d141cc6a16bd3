// Segmented "shrink" GEMM: D[rows of piece, N] = scale * X[rows, K] . W_seg with
// small N (the LoRA rank, <= 128) and large K (the hidden size).
//
// Takes the place of the reference's shrink configuration of the grouped GEMM
// (kernel_src/csrc/smlm_forward/smlm_forward_cutlass.cuh:127-171): fp16/bf16
// operands, fp32 accumulation, result rounded to the operand type, rows of D inside
// a segment overwritten.  It is also the dV = gO.B step of the backward
// (src/loquetier_src/kernel_utils.py:142).
//
// Shape of the work: one CTA owns one piece (<= 64 rows of one segment) and one
// slice of K; the `KS` CTAs of a thread-block cluster own the K slices of the same
// piece and add their partial sums through distributed shared memory, in a fixed
// order, so the result is deterministic and no global scratch or atomics are
// needed.
//
// The stream of X is the HBM-bound part.  A producer warp feeds a ring of stages
// with TMA: one tiled tensor copy per stage brings a [rows x 64 columns] box of X
// (128-byte swizzle; the box height is the smallest of 8/16/32/64 covering the
// piece, rows past the piece are fetched but never stored), and untiled bulk
// copies bring the matching slice of the adapter panel from its raw pointer.  Four
// consumer warps wait on the stage's mbarrier and run ldmatrix + mma.sync m16n8k16;
// they split rows when the piece is tall and split the K slice when it is short
// (decode pieces have one row), and their partial sums meet in shared memory.
#pragma once
#include <cooperative_groups.h>
#include <cuda.h>

#include "smlm_common.cuh"

namespace smlm {

namespace cg = cooperative_groups;

constexpr int kShrinkStages = 6;
constexpr int kKC = 64;                     // K columns per pipeline stage
constexpr int kShrinkThreads = kThreads + 32;  // four consumer warps + one producer warp
constexpr int kWRowPad = 144;               // bytes between panel rows in shared memory ([N][K] layout)

struct XMaps {
  CUtensorMap m[4];  // box heights 8, 16, 32, 64
};

template <int NT, bool ROWMAJOR>
struct ShrinkSmem {
  static constexpr int kXBytes = kBM * kKC * 2;  // 8 KB, 1024-byte aligned for the 128-byte swizzle
  static constexpr int kWBytesRaw = ROWMAJOR ? kKC * NT * 16 : NT * 8 * kWRowPad;
  static constexpr int kWBytes = (kWBytesRaw + 1023) / 1024 * 1024;
  static constexpr int kStage = kXBytes + kWBytes;
  static constexpr int kPipe = kShrinkStages * kStage;
  static constexpr int kRed = 4 * 16 * NT * 8 * 4;  // one 16 x N fp32 block per consumer warp
  static constexpr int kBarOff = kPipe > kRed ? kPipe : kRed;
  static constexpr int kTotal = kBarOff + 2 * kShrinkStages * 8 + 1024;  // + alignment slack
};

struct ShrinkArgs {
  void* d;                     // [T, N]
  const void* x;               // [T, K]
  const void* const* w_table;  // device array of adapter pointers
  const int32_t* ids;          // per-segment adapter index into w_table, or null: w_table[seg]
  const float* scale;          // per-adapter (ids != null) or per-segment scale, or null
  int* plan;                   // header + pieces
  int n_table;
  int N, K;
  int ksplit;                  // cluster size along K
};

template <typename T, int NT, bool ROWMAJOR>
__global__ void __launch_bounds__(kShrinkThreads) shrink_kernel(const ShrinkArgs a,
                                                               const __grid_constant__ XMaps xm) {
  extern __shared__ unsigned char smem_raw[];
  using SM = ShrinkSmem<NT, ROWMAJOR>;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int KS = a.ksplit;
  const int piece_idx = blockIdx.x / KS;
  const int z = blockIdx.x - piece_idx * KS;  // == rank in the cluster (cluster dims are (KS,1,1))

  pdl_wait();
  pdl_trigger();
  const int count = a.plan[0];
  const Piece pc = reinterpret_cast<const Piece*>(a.plan + kPlanHeaderInts)[piece_idx];
  if (piece_idx >= count) return;  // whole cluster leaves together
  const int nrows = pc.nrows;
  const int N = a.N, K = a.K;
  int* err = a.plan + 1;

  const T* w = static_cast<const T*>(adapter_ptr(a.w_table, a.ids, a.n_table, pc.seg, err));
  const bool w_ok = (w != nullptr);

  // K slice of this CTA, in stages of kKC columns
  const int ksteps = (K + kKC - 1) / kKC;
  const int per = (ksteps + KS - 1) / KS;
  const int kbeg = z * per;
  const int kend = min(ksteps, kbeg + per);
  const int nk = w_ok ? max(0, kend - kbeg) : 0;

  // 1024-byte aligned carve-up of dynamic shared memory (same offset in every CTA)
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* smem = smem_raw + (base - raw);
  const uint32_t full0 = base + SM::kBarOff;
  const uint32_t empty0 = full0 + kShrinkStages * 8;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kShrinkStages; ++s) {
      mbar_init(full0 + s * 8, 1);
      mbar_init(empty0 + s * 8, 4);
    }
    fence_mbar_init();
  }
  if ((K % kKC) != 0) {
    // the last stage is only partly overwritten by the panel copies: start from zeros so that
    // the columns past K (which X supplies as zeros) never meet a non-finite leftover
    for (int s = 0; s < kShrinkStages; ++s) {
      uint4* wz = reinterpret_cast<uint4*>(smem + s * SM::kStage + SM::kXBytes);
      for (int i = tid; i < SM::kWBytes / 16; i += kShrinkThreads) wz[i] = make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async();
  }
  __syncthreads();

  // warp roles among the four consumer warps
  const int WM = nrows <= 16 ? 1 : (nrows <= 32 ? 2 : 4);
  const int WK = 4 / WM;
  const int wm = warp % WM;
  const int wk = warp / WM;
  bool dead = false;

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

  if (warp == 4) {
    // ---------------- producer ----------------
    const int hsel = nrows <= 8 ? 0 : (nrows <= 16 ? 1 : (nrows <= 32 ? 2 : 3));
    const uint32_t xbytes = (8u << hsel) * 128u;
    const CUtensorMap* xmap = &xm.m[hsel];
    for (int it = 0; it < nk; ++it) {
      const int slot = it % kShrinkStages;
      const int k0 = (kbeg + it) * kKC;
      const uint32_t xs = base + slot * SM::kStage;
      const uint32_t ws = xs + SM::kXBytes;
      const uint32_t fb = full0 + slot * 8;
      if (it >= kShrinkStages) mbar_wait(empty0 + slot * 8, ((it / kShrinkStages) - 1) & 1, err, dead);
      const int kcols = min(kKC, K - k0);
      if constexpr (!ROWMAJOR) {
        const uint32_t rowb = kcols * 2;
        if (lane == 0) {
          mbar_expect_tx(fb, xbytes + rowb * N);
          tma_load_2d(xs, xmap, k0, pc.row0, fb);
        }
        __syncwarp();
        for (int n = lane; n < N; n += 32) bulk_load(ws + n * kWRowPad, w + static_cast<size_t>(n) * K + k0, rowb, fb);
      } else {
        if (lane == 0) {
          const uint32_t wb = kcols * N * 2;
          mbar_expect_tx(fb, xbytes + wb);
          tma_load_2d(xs, xmap, k0, pc.row0, fb);
          bulk_load(ws, w + static_cast<size_t>(k0) * N, wb, fb);
        }
      }
    }
  } else {
    // ---------------- consumers ----------------
    const bool active = (wm * 16 < nrows);
    for (int it = 0; it < nk; ++it) {
      const int slot = it % kShrinkStages;
      const uint32_t xs = base + slot * SM::kStage;
      const uint32_t ws = xs + SM::kXBytes;
      mbar_wait(full0 + slot * 8, (it / kShrinkStages) & 1, err, dead);
      if (active) {
        for (int kk = wk; kk < kKC / 16; kk += WK) {
          uint32_t af[4];
          {
            const int m = lane >> 3;
            const int r = wm * 16 + (m & 1) * 8 + (lane & 7);
            const int c = kk * 2 + (m >> 1);
            ldsm_x4(af, xs + r * 128 + ((c ^ (r & 7)) << 4));
          }
          if constexpr (!ROWMAJOR) {
            if constexpr (NT == 1) {
              uint32_t bf[4];
              const int m = (lane >> 3) & 1;
              const int n = lane & 7;
              ldsm_x4(bf, ws + n * kWRowPad + ((kk * 2 + m) << 4));
              mma16816<T>(acc[0], af, bf[0], bf[1]);
            } else {
#pragma unroll
              for (int j = 0; j < NT; j += 2) {
                uint32_t bf[4];
                const int m = lane >> 3;
                const int n = (j + (m >> 1)) * 8 + (lane & 7);
                ldsm_x4(bf, ws + n * kWRowPad + ((kk * 2 + (m & 1)) << 4));
                mma16816<T>(acc[j], af, bf[0], bf[1]);
                mma16816<T>(acc[j + 1], af, bf[2], bf[3]);
              }
            }
          } else {
            // panel stored [K][N] with rows of N elements, exactly as in global memory
            const int rowb = N * 2;
            if constexpr (NT == 1) {
              uint32_t bf[4];
              const int m = (lane >> 3) & 1;
              const int k = kk * 16 + m * 8 + (lane & 7);
              ldsm_x4_t(bf, ws + k * rowb);
              mma16816<T>(acc[0], af, bf[0], bf[1]);
            } else {
#pragma unroll
              for (int j = 0; j < NT; j += 2) {
                uint32_t bf[4];
                const int m = lane >> 3;
                const int k = kk * 16 + (m & 1) * 8 + (lane & 7);
                const int c = j + (m >> 1);
                ldsm_x4_t(bf, ws + k * rowb + (c << 4));
                mma16816<T>(acc[j], af, bf[0], bf[1]);
                mma16816<T>(acc[j + 1], af, bf[2], bf[3]);
              }
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + slot * 8);
    }
  }
  __syncthreads();  // every stage has been consumed; the ring can be reused

  // every consumer warp parks its 16 x N block; red[warp][16][NT*8]
  float* red = reinterpret_cast<float*>(smem);
  constexpr int NP = NT * 8;
  if (warp < 4) {
    const int g = lane >> 2, t = lane & 3;
    float* my = red + warp * 16 * NP;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      *reinterpret_cast<float2*>(my + g * NP + j * 8 + 2 * t) = make_float2(acc[j][0], acc[j][1]);
      *reinterpret_cast<float2*>(my + (g + 8) * NP + j * 8 + 2 * t) = make_float2(acc[j][2], acc[j][3]);
    }
  }
  const float sc = adapter_scale(a.scale, a.ids, a.n_table, pc.seg);
  T* drow = static_cast<T*>(a.d) + static_cast<size_t>(pc.row0) * N;
  const int half_n = N >> 1;
  const int pairs = nrows * half_n;

  if (KS == 1) {
    __syncthreads();
    for (int e = tid; e < pairs; e += kShrinkThreads) {
      const int r = e / half_n;
      const int n = (e - r * half_n) * 2;
      const int fm = r >> 4, r16 = r & 15;
      float2 s = make_float2(0.f, 0.f);
      for (int q = 0; q < WK; ++q) {
        const float2 p = *reinterpret_cast<const float2*>(red + ((q * WM + fm) * 16 + r16) * NP + n);
        s.x += p.x;
        s.y += p.y;
      }
      if (w_ok) *reinterpret_cast<uint32_t*>(drow + static_cast<size_t>(r) * N + n) = pack2<T>(s.x * sc, s.y * sc);
    }
  } else {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    for (int e = z * kShrinkThreads + tid; e < pairs; e += KS * kShrinkThreads) {
      const int r = e / half_n;
      const int n = (e - r * half_n) * 2;
      const int fm = r >> 4, r16 = r & 15;
      float2 s = make_float2(0.f, 0.f);
      for (int cz = 0; cz < KS; ++cz) {
        const float* rr = cluster.map_shared_rank(red, cz);
        for (int q = 0; q < WK; ++q) {
          const float2 p = *reinterpret_cast<const float2*>(rr + ((q * WM + fm) * 16 + r16) * NP + n);
          s.x += p.x;
          s.y += p.y;
        }
      }
      if (w_ok) *reinterpret_cast<uint32_t*>(drow + static_cast<size_t>(r) * N + n) = pack2<T>(s.x * sc, s.y * sc);
    }
    cluster.sync();  // nobody leaves while a peer still reads its shared memory
  }
}

}  // namespace smlm
