// Segmented "expand" GEMM: D[rows of piece, N] (+)= scale * X[rows, K] . W_seg with
// small K (the LoRA rank, <= 128) and large N (the hidden size).
//
// Takes the place of the reference's expand configuration of the grouped GEMM
// (kernel_src/csrc/smlm_forward/smlm_forward_cutlass.cuh:82-126) and, with
// `accumulate` and a per-segment scale, of the two elementwise passes that follow
// it in the reference's LoRA linear (src/loquetier_src/models/mixed_lora.py:214-217).
// It is also the dX = dV.A step of the backward (src/loquetier_src/kernel_utils.py:143).
//
// One CTA owns one piece (<= 64 rows of one segment) and 256 output columns.  The
// piece's X rows and the 256 x K slab of W are staged once in shared memory with
// 16-byte cp.async copies; each warp keeps its X fragments in registers, walks the
// columns 64 at a time with mma.sync m16n8k16 (fp32 accumulation), and stages every
// 16 x 64 result block in shared memory so that the write of D - the HBM-bound part
// - leaves as full 128-byte rows.  Tall pieces give each warp 16 rows; short ones
// (decode pieces have one row) give each warp its own 64 columns.
#pragma once
#include "smlm_common.cuh"

namespace smlm {

constexpr int kNCH = 256;  // output columns per CTA

template <int KT>
struct ExpandSmem {
  static constexpr int kKP = KT * 16;                    // padded K
  static constexpr int kXBytes = kBM * kKP * 2;
  static constexpr int kWBytes = kNCH * kKP * 2;
  static constexpr int kOBytes = 4 * 16 * 64 * 2;        // one 16 x 64 block per warp
  static constexpr int kTotal = kXBytes + kWBytes + kOBytes;
};

struct ExpandArgs {
  void* d;                     // [T, N]
  const void* x;               // [T, K]
  const void* const* w_table;
  const int32_t* ids;
  const float* scale;
  int* plan;
  int n_table;
  int N, K;
  int accumulate;              // D += instead of D =
};

template <typename T, int KT, bool ROWMAJOR>
__global__ void __launch_bounds__(kThreads) expand_kernel(const ExpandArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  using SM = ExpandSmem<KT>;
  constexpr int XC = KT * 2;  // 16-byte chunks per X row (and per W row in the [N][K] layout)
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;

  pdl_wait();
  pdl_trigger();
  const int count = a.plan[0];
  const int piece_idx = blockIdx.x;
  if (piece_idx >= count) return;
  const Piece pc = reinterpret_cast<const Piece*>(a.plan + kPlanHeaderInts)[piece_idx];
  const int nrows = pc.nrows;
  const int N = a.N, K = a.K;
  const int n0 = blockIdx.y * kNCH;
  const int ncols = min(kNCH, N - n0);

  const T* w = static_cast<const T*>(adapter_ptr(a.w_table, a.ids, a.n_table, pc.seg, a.plan + 1));
  if (w == nullptr) return;

  const uint32_t xs = smem_u32(smem);
  const uint32_t ws = xs + SM::kXBytes;
  const uint32_t os = ws + SM::kWBytes + warp * (16 * 64 * 2);
  const int load_rows = min(kBM, ((nrows + 15) >> 4) << 4);
  const T* xrow = static_cast<const T*>(a.x) + static_cast<size_t>(pc.row0) * K;
  const int kchunks = K >> 3;

  for (int i = tid; i < load_rows * XC; i += kThreads) {
    const int r = i / XC, c = i - r * XC;
    const bool ok = (r < nrows) && (c < kchunks);
    const T* src = ok ? (xrow + static_cast<size_t>(r) * K + c * 8) : static_cast<const T*>(a.x);
    cp_async16(xs + r * (XC * 16) + swz<XC>(r, c) * 16, src, ok);
  }
  if constexpr (!ROWMAJOR) {
    // W stored [N][K]: the 256-row slab is one contiguous block of global memory
    for (int i = tid; i < kNCH * XC; i += kThreads) {
      const int n = i / XC, c = i - n * XC;
      const bool ok = (n < ncols) && (c < kchunks);
      const T* src = ok ? (w + static_cast<size_t>(n0 + n) * K + c * 8) : static_cast<const T*>(a.x);
      cp_async16(ws + n * (XC * 16) + swz<XC>(n, c) * 16, src, ok);
    }
  } else {
    // W stored [K][N]: KT*16 rows of 32 chunks (512 bytes) each
    for (int i = tid; i < KT * 16 * 32; i += kThreads) {
      const int k = i >> 5, c = i & 31;
      const bool ok = (k < K) && (c * 8 < ncols);
      const T* src = ok ? (w + static_cast<size_t>(k) * N + n0 + c * 8) : static_cast<const T*>(a.x);
      cp_async16(ws + k * 512 + ((c & ~7) | ((c ^ k) & 7)) * 16, src, ok);
    }
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  const int WM = nrows <= 16 ? 1 : (nrows <= 32 ? 2 : 4);
  const int WN = 4 / WM;
  const int wm = warp % WM;
  const int wn = warp / WM;
  if (wm * 16 >= nrows) return;  // no barrier is used past this point

  uint32_t af[KT][4];
#pragma unroll
  for (int kk = 0; kk < KT; ++kk) {
    const int m = lane >> 3;
    const int r = wm * 16 + (m & 1) * 8 + (lane & 7);
    const int c = kk * 2 + (m >> 1);
    ldsm_x4(af[kk], xs + r * (XC * 16) + swz<XC>(r, c) * 16);
  }
  const float sc = adapter_scale(a.scale, a.ids, a.n_table, pc.seg);
  T* dbase = static_cast<T*>(a.d) + static_cast<size_t>(pc.row0 + wm * 16) * N + n0;
  const int rows_here = min(16, nrows - wm * 16);
  const int ngroups = (ncols + 63) >> 6;

  for (int grp = wn; grp < ngroups; grp += WN) {
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KT; ++kk) {
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        uint32_t bf[4];
        const int m = lane >> 3;
        if constexpr (!ROWMAJOR) {
          const int n = grp * 64 + (j + (m >> 1)) * 8 + (lane & 7);
          const int c = kk * 2 + (m & 1);
          ldsm_x4(bf, ws + n * (XC * 16) + swz<XC>(n, c) * 16);
        } else {
          const int k = kk * 16 + (m & 1) * 8 + (lane & 7);
          const int c = grp * 8 + j + (m >> 1);
          ldsm_x4_t(bf, ws + k * 512 + ((c & ~7) | ((c ^ k) & 7)) * 16);
        }
        mma16816<T>(acc[j], af[kk], bf[0], bf[1]);
        mma16816<T>(acc[j + 1], af[kk], bf[2], bf[3]);
      }
    }
    // registers -> this warp's staging block [16][64] (128-byte rows, swizzled)
    {
      const int g = lane >> 2, t = lane & 3;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t lo = pack2<T>(acc[j][0] * sc, acc[j][1] * sc);
        const uint32_t hi = pack2<T>(acc[j][2] * sc, acc[j][3] * sc);
        asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(os + g * 128 + ((j ^ (g & 7)) * 16) + t * 4), "r"(lo));
        asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(os + (g + 8) * 128 + ((j ^ ((g + 8) & 7)) * 16) + t * 4),
                     "r"(hi));
      }
    }
    __syncwarp();
    // staging block -> global, 16 bytes per lane, four 128-byte rows per instruction
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int i = q * 32 + lane;
      const int r = i >> 3, c = i & 7;
      const int col = grp * 64 + c * 8;
      if (r < rows_here && col < ncols) {
        uint4 v;
        asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "r"(os + r * 128 + ((c ^ (r & 7)) * 16)));
        uint4* dst = reinterpret_cast<uint4*>(dbase + static_cast<size_t>(r) * N + col);
        if (a.accumulate) {
          const uint4 o = *dst;
          const uint32_t* ov = reinterpret_cast<const uint32_t*>(&o);
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

}  // namespace smlm
