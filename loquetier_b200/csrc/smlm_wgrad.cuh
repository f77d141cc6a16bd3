// Per-partition weight gradient: G_p = scale * P[rows_p, :R]^T . Q[rows_p, :H]
// with R the LoRA rank (<= 128), H a hidden size, rows_p the token rows of train
// partition p.
//
// The reference has no native backward (kernel_src/csrc/loquetier_ops.cc:321-322);
// it forms these products with torch matmuls per partition
// (src/loquetier_src/kernel_utils.py:144-145):
//   dA = dV^T . X   (P = dV, Q = X)      dB = gO^T . V   (P = V, Q = gO)
// In the PEFT layout dA is [R, H] (stored as computed) and dB is [H, R] (stored
// transposed); the math layout swaps the two.
//
// One CTA owns 64 columns of Q for one partition and one slice of its tokens; the
// `KS` CTAs of a cluster own the token slices and add their partial sums through
// distributed shared memory in a fixed order (deterministic, no scratch, no
// atomics).  Q is streamed once through a 4-stage cp.async pipeline (64 tokens x
// 64 columns per stage, 128-byte rows); the contraction over tokens runs on
// mma.sync m16n8k16 with both operands fetched by transposing ldmatrix.
#pragma once
#include <cooperative_groups.h>

#include "smlm_common.cuh"

namespace smlm {

namespace cg = cooperative_groups;

constexpr int kWgStages = 4;
constexpr int kWgTok = 64;   // tokens per stage
constexpr int kWgCols = 64;  // columns of Q per CTA

template <int RT>
struct WgradSmem {
  static constexpr int kPBytes = kWgTok * RT * 32;   // [64 tokens][RT*16]
  static constexpr int kQBytes = kWgTok * kWgCols * 2;
  static constexpr int kStage = kPBytes + kQBytes;
  static constexpr int kPipe = kWgStages * kStage;
  static constexpr int kRed = RT * 16 * kWgCols * 4;
  static constexpr int kTotal = kPipe > kRed ? kPipe : kRed;
};

struct WgradArgs {
  void* const* g_table;        // device array of npart output pointers
  const void* p;               // [T, R]
  const void* q;               // [T, H]
  const int32_t* part_indptr;  // [npart + 1]
  const float* scale;          // per partition (ids == null) or per adapter, or null
  const int32_t* ids;          // per-partition adapter index for `scale`, or null
  int n_table;
  int* err;                    // error word (plan header + 1)
  int npart, T;
  int R, H;
  int ksplit;
  int transposed;              // 0: G is [R, H]; 1: G is [H, R]
  int accumulate;              // G += instead of G =
  int out_fp32;                // G holds fp32 instead of the operand type
};

template <typename T, int RT>
__global__ void __launch_bounds__(kThreads) wgrad_kernel(const WgradArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  using SM = WgradSmem<RT>;
  constexpr int PC = RT * 2;  // 16-byte chunks per P row
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int KS = a.ksplit;
  const int part = blockIdx.x / KS;
  const int z = blockIdx.x - part * KS;
  const int col0 = blockIdx.y * kWgCols;
  const int R = a.R, H = a.H;
  const int ncols = min(kWgCols, H - col0);

  int ra = a.part_indptr[part], rb = a.part_indptr[part + 1];
  if (ra < 0 || rb < ra || rb > a.T) {  // same verdict in every CTA of the cluster
    if (tid == 0) atomicOr(a.err, kErrBadIndptr);
    return;
  }
  void* gout = a.g_table[part];
  if (gout == nullptr || (reinterpret_cast<uintptr_t>(gout) & 15) != 0) {
    if (tid == 0) atomicOr(a.err, kErrBadPointer);
    return;
  }
  const int n = rb - ra;
  const int chunks = (n + kWgTok - 1) / kWgTok;
  const int per = (chunks + KS - 1) / KS;
  const int cbeg = z * per;
  const int cend = min(chunks, cbeg + per);
  const int nk = max(0, cend - cbeg);

  const T* P = static_cast<const T*>(a.p);
  const T* Q = static_cast<const T*>(a.q);
  const uint32_t smem_base = smem_u32(smem);
  const int rchunks = R >> 3;

  auto load_stage = [&](int slot, int chunk) {
    const int t0 = ra + chunk * kWgTok;
    const uint32_t ps = smem_base + slot * SM::kStage;
    const uint32_t qs = ps + SM::kPBytes;
    for (int i = tid; i < kWgTok * PC; i += kThreads) {
      const int t = i / PC, c = i - t * PC;
      const bool ok = (t0 + t < rb) && (c < rchunks);
      const T* src = ok ? (P + static_cast<size_t>(t0 + t) * R + c * 8) : P;
      cp_async16(ps + t * (PC * 16) + swz<PC>(t, c) * 16, src, ok);
    }
    for (int i = tid; i < kWgTok * 8; i += kThreads) {
      const int t = i >> 3, c = i & 7;
      const bool ok = (t0 + t < rb) && (c * 8 < ncols);
      const T* src = ok ? (Q + static_cast<size_t>(t0 + t) * H + col0 + c * 8) : Q;
      cp_async16(qs + t * 128 + swz<8>(t, c) * 16, src, ok);
    }
  };

  float acc[RT][2][4];
#pragma unroll
  for (int i = 0; i < RT; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

#pragma unroll
  for (int s = 0; s < kWgStages - 1; ++s) {
    if (s < nk) load_stage(s, cbeg + s);
    cp_async_commit();
  }
  for (int it = 0; it < nk; ++it) {
    cp_async_wait<kWgStages - 2>();
    __syncthreads();
    {
      const int nx = it + kWgStages - 1;
      if (nx < nk) load_stage(nx % kWgStages, cbeg + nx);
      cp_async_commit();
    }
    const int slot = it % kWgStages;
    const uint32_t ps = smem_base + slot * SM::kStage;
    const uint32_t qs = ps + SM::kPBytes;
#pragma unroll
    for (int kk = 0; kk < kWgTok / 16; ++kk) {
      const int m = lane >> 3;
      uint32_t bf[4];
      {
        // B operand: Q[token][col]; matrices (k lo, n lo), (k hi, n lo), (k lo, n hi), (k hi, n hi)
        const int t = kk * 16 + (m & 1) * 8 + (lane & 7);
        const int c = warp * 2 + (m >> 1);
        ldsm_x4_t(bf, qs + t * 128 + swz<8>(t, c) * 16);
      }
#pragma unroll
      for (int i = 0; i < RT; ++i) {
        // A operand: P^T, i.e. rows are rank indices, k are tokens; matrices
        // (m lo, k lo), (m hi, k lo), (m lo, k hi), (m hi, k hi)
        uint32_t af[4];
        const int t = kk * 16 + (m >> 1) * 8 + (lane & 7);
        const int c = i * 2 + (m & 1);
        ldsm_x4_t(af, ps + t * (PC * 16) + swz<PC>(t, c) * 16);
        mma16816<T>(acc[i][0], af, bf[0], bf[1]);
        mma16816<T>(acc[i][1], af, bf[2], bf[3]);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // park the CTA's [RT*16][64] fp32 partial sums
  float* red = reinterpret_cast<float*>(smem);
  {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int i = 0; i < RT; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int col = warp * 16 + j * 8 + 2 * t;
        *reinterpret_cast<float2*>(red + (i * 16 + g) * kWgCols + col) = make_float2(acc[i][j][0], acc[i][j][1]);
        *reinterpret_cast<float2*>(red + (i * 16 + g + 8) * kWgCols + col) =
            make_float2(acc[i][j][2], acc[i][j][3]);
      }
  }
  const float sc = adapter_scale(a.scale, a.ids, a.n_table, part);
  cg::cluster_group cluster = cg::this_cluster();
  if (KS > 1) cluster.sync(); else __syncthreads();

  // out element e in output order; consecutive threads write consecutive addresses
  const int total = R * ncols;
  for (int e = z * kThreads + tid; e < total; e += KS * kThreads) {
    int r, c;
    size_t off;
    if (a.transposed) {  // G[H][R]
      c = e / R;
      r = e - c * R;
      off = static_cast<size_t>(col0 + c) * R + r;
    } else {             // G[R][H]
      r = e / ncols;
      c = e - r * ncols;
      off = static_cast<size_t>(r) * H + col0 + c;
    }
    float s = 0.f;
    if (KS > 1) {
      for (int cz = 0; cz < KS; ++cz) s += cluster.map_shared_rank(red, cz)[r * kWgCols + c];
    } else {
      s = red[r * kWgCols + c];
    }
    s *= sc;
    if (a.out_fp32) {
      float* g = static_cast<float*>(gout) + off;
      *g = a.accumulate ? (*g + s) : s;
    } else {
      T* g = static_cast<T*>(gout) + off;
      if (a.accumulate) s += static_cast<float>(*g);
      *g = static_cast<T>(s);
    }
  }
  if (KS > 1) cluster.sync();
}

}  // namespace smlm
