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
// needed.  Inside a CTA the four warps split rows when the piece is tall and split
// the K slice when it is short (decode pieces have one row), and their partial sums
// meet in shared memory.
//
// The stream of X is the HBM-bound part: 4 stages of 64 rows x 64 columns move
// through shared memory with 16-byte cp.async copies (zero-filled past the piece's
// last row and past K); the rank-N contraction uses mma.sync m16n8k16.
#pragma once
#include <cooperative_groups.h>

#include "smlm_common.cuh"

namespace smlm {

namespace cg = cooperative_groups;

constexpr int kShrinkStages = 4;
constexpr int kKC = 64;  // K columns per pipeline stage

template <int NT, bool ROWMAJOR>
struct ShrinkSmem {
  static constexpr int kXBytes = kBM * kKC * 2;                 // 8 KB
  static constexpr int kWBytes = NT * 8 * kKC * 2;              // NT KB, either layout
  static constexpr int kStage = kXBytes + kWBytes;
  static constexpr int kPipe = kShrinkStages * kStage;
  static constexpr int kRed = 4 * 16 * NT * 8 * 4;              // one 16 x N fp32 block per warp
  static constexpr int kTotal = kPipe > kRed ? kPipe : kRed;
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
__global__ void __launch_bounds__(kThreads) shrink_kernel(const ShrinkArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  using SM = ShrinkSmem<NT, ROWMAJOR>;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int KS = a.ksplit;
  const int piece_idx = blockIdx.x / KS;
  const int z = blockIdx.x - piece_idx * KS;  // == rank in the cluster (cluster dims are (KS,1,1))

  const int count = a.plan[0];
  if (piece_idx >= count) return;  // whole cluster leaves together
  const Piece pc = reinterpret_cast<const Piece*>(a.plan + kPlanHeaderInts)[piece_idx];
  const int nrows = pc.nrows;
  const int N = a.N, K = a.K;

  const T* w = static_cast<const T*>(adapter_ptr(a.w_table, a.ids, a.n_table, pc.seg, a.plan + 1));
  const bool w_ok = (w != nullptr);
  if (!w_ok) w = static_cast<const T*>(a.x);  // never dereferenced: every copy is zero-filled

  // K slice of this CTA, in stages of kKC columns
  const int ksteps = (K + kKC - 1) / kKC;
  const int per = (ksteps + KS - 1) / KS;
  const int kbeg = z * per;
  const int kend = min(ksteps, kbeg + per);
  const int nk = max(0, kend - kbeg);

  // warp roles
  const int WM = nrows <= 16 ? 1 : (nrows <= 32 ? 2 : 4);
  const int WK = 4 / WM;
  const int wm = warp % WM;
  const int wk = warp / WM;
  const int load_rows = min(kBM, ((nrows + 15) >> 4) << 4);

  const T* xrow = static_cast<const T*>(a.x) + static_cast<size_t>(pc.row0) * K;
  const uint32_t smem_base = smem_u32(smem);

  auto load_stage = [&](int slot, int kstep) {
    const int k0 = kstep * kKC;
    const uint32_t xs = smem_base + slot * SM::kStage;
    const uint32_t ws = xs + SM::kXBytes;
    // X tile: load_rows x 8 chunks
    for (int i = tid; i < load_rows * 8; i += kThreads) {
      const int r = i >> 3, c = i & 7;
      const bool ok = (r < nrows) && (k0 + c * 8 < K);
      const T* src = ok ? (xrow + static_cast<size_t>(r) * K + k0 + c * 8) : static_cast<const T*>(a.x);
      cp_async16(xs + r * 128 + swz<8>(r, c) * 16, src, ok);
    }
    if constexpr (!ROWMAJOR) {
      // W stored [N][K]: NT*8 rows of 8 chunks
      for (int i = tid; i < NT * 8 * 8; i += kThreads) {
        const int n = i >> 3, c = i & 7;
        const bool ok = w_ok && (n < N) && (k0 + c * 8 < K);
        const T* src = ok ? (w + static_cast<size_t>(n) * K + k0 + c * 8) : static_cast<const T*>(a.x);
        cp_async16(ws + n * 128 + swz<8>(n, c) * 16, src, ok);
      }
    } else {
      // W stored [K][N]: kKC rows of NT chunks
      for (int i = tid; i < kKC * NT; i += kThreads) {
        const int k = i / NT, c = i - k * NT;
        const bool ok = w_ok && (k0 + k < K) && (c * 8 < N);
        const T* src = ok ? (w + static_cast<size_t>(k0 + k) * N + c * 8) : static_cast<const T*>(a.x);
        cp_async16(ws + k * (NT * 16) + swz<NT>(k, c) * 16, src, ok);
      }
    }
  };

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

#pragma unroll
  for (int s = 0; s < kShrinkStages - 1; ++s) {
    if (s < nk) load_stage(s, kbeg + s);
    cp_async_commit();
  }

  const bool active = (wm * 16 < nrows);
  for (int it = 0; it < nk; ++it) {
    cp_async_wait<kShrinkStages - 2>();
    __syncthreads();
    {
      const int nx = it + kShrinkStages - 1;
      if (nx < nk) load_stage(nx % kShrinkStages, kbeg + nx);
      cp_async_commit();
    }
    if (active) {
      const int slot = it % kShrinkStages;
      const uint32_t xs = smem_base + slot * SM::kStage;
      const uint32_t ws = xs + SM::kXBytes;
      for (int kk = wk; kk < kKC / 16; kk += WK) {
        uint32_t af[4];
        {
          const int m = lane >> 3;
          const int r = wm * 16 + (m & 1) * 8 + (lane & 7);
          const int c = kk * 2 + (m >> 1);
          ldsm_x4(af, xs + r * 128 + swz<8>(r, c) * 16);
        }
        if constexpr (!ROWMAJOR) {
          if constexpr (NT == 1) {
            uint32_t bf[4];
            const int m = (lane >> 3) & 1;
            const int n = lane & 7;
            const int c = kk * 2 + m;
            // lanes 16..31 repeat valid addresses; only the first two matrices are used
            ldsm_x4(bf, ws + n * 128 + swz<8>(n, c) * 16);
            mma16816<T>(acc[0], af, bf[0], bf[1]);
          } else {
#pragma unroll
            for (int j = 0; j < NT; j += 2) {
              uint32_t bf[4];
              const int m = lane >> 3;
              const int n = (j + (m >> 1)) * 8 + (lane & 7);
              const int c = kk * 2 + (m & 1);
              ldsm_x4(bf, ws + n * 128 + swz<8>(n, c) * 16);
              mma16816<T>(acc[j], af, bf[0], bf[1]);
              mma16816<T>(acc[j + 1], af, bf[2], bf[3]);
            }
          }
        } else {
          if constexpr (NT == 1) {
            uint32_t bf[4];
            const int m = (lane >> 3) & 1;
            const int k = kk * 16 + m * 8 + (lane & 7);
            ldsm_x4_t(bf, ws + k * 16);
            mma16816<T>(acc[0], af, bf[0], bf[1]);
          } else {
#pragma unroll
            for (int j = 0; j < NT; j += 2) {
              uint32_t bf[4];
              const int m = lane >> 3;
              const int k = kk * 16 + (m & 1) * 8 + (lane & 7);
              const int c = j + (m >> 1);
              ldsm_x4_t(bf, ws + k * (NT * 16) + swz<NT>(k, c) * 16);
              mma16816<T>(acc[j], af, bf[0], bf[1]);
              mma16816<T>(acc[j + 1], af, bf[2], bf[3]);
            }
          }
        }
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // every warp parks its 16 x N block; red[warp][16][NT*8]
  float* red = reinterpret_cast<float*>(smem);
  constexpr int NP = NT * 8;
  {
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
  const int pairs = nrows * (N >> 1);

  if (KS == 1) {
    __syncthreads();
    for (int e = tid; e < pairs; e += kThreads) {
      const int r = e / (N >> 1);
      const int n = (e - r * (N >> 1)) * 2;
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
    for (int e = z * kThreads + tid; e < pairs; e += KS * kThreads) {
      const int r = e / (N >> 1);
      const int n = (e - r * (N >> 1)) * 2;
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
