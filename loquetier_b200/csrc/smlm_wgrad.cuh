// Per-partition weight gradients  G_p = scale * P[rows_p, :R]^T . Q[rows_p, :H]
// with R the LoRA rank (<= 128), H a hidden size, rows_p the token rows of train
// partition p.  One launch runs up to two such jobs side by side, which is how
// the backward computes dB and dA together.
//
// The reference has no native backward (kernel_src/csrc/loquetier_ops.cc:321-322);
// it forms these products with torch matmuls per partition
// (src/loquetier_src/kernel_utils.py:144-145):
//   dA = dV^T . X   (P = dV, Q = X)      dB = gO^T . V   (P = V, Q = gO)
// In the PEFT layout dA is [R, H] (stored as computed) and dB is [H, R] (stored
// transposed); the math layout swaps the two.
//
// Work is cut by tokens, not by partitions, so that one very long partition next
// to many short ones still spreads evenly: a CTA owns `G` consecutive pieces of
// the partition plan (64 tokens each) and one slab of Q's columns.  It streams its
// Q tiles - the HBM-bound read - through a ring of shared-memory stages fed by a
// producer warp with TMA ([16 tokens x 64 columns] tiled tensor copies with the
// 128-byte swizzle, issued so that each token row's consecutive chunks are requested
// together; the matching P rows as one untiled bulk copy).  Four consumer warps
// contract over tokens with mma.sync m16n8k16, both operands fetched by
// transposing ldmatrix, each warp on its own columns.
//
// Whenever the partition changes inside a CTA's pieces, each warp closes the run:
// a run that holds a whole partition is written out directly; otherwise the warp
// parks its fp32 partial sums in the caller's workspace and takes a ticket; the
// warp that draws the last ticket of a (partition, slab) adds all parked partials
// in group order - a fixed order, so results are deterministic - and writes G.
// Nobody waits on anybody: there is no spin loop and no atomic on data.
#pragma once
#include <cuda.h>

#include "smlm_common.cuh"

namespace smlm {

constexpr int kWgThreads = kThreads + 32;  // four consumer warps + one producer warp
constexpr int kWgTok = 64;                 // tokens per ring stage (= one piece)
constexpr int kWgStages = 2;               // two CTAs fit on one SM
constexpr int kWgMaxGroup = 64;            // pieces per CTA at most

// columns of Q per warp, chosen so that the accumulators stay within 64 registers
constexpr int wgrad_cols_per_warp(int rt) { return rt <= 2 ? 64 : (rt == 4 ? 32 : 16); }

template <int RT>
struct WgradSmem {
  static constexpr int KP = RT * 16;
  static constexpr int CW = wgrad_cols_per_warp(RT);
  static constexpr int SLAB = 4 * CW;                          // columns of Q per CTA
  static constexpr int NCH = (SLAB + 63) / 64;                 // 64-column chunks per stage
  static constexpr int kQBytes = 4 * NCH * 2048;               // 4 token blocks x NCH chunks of [16][64]
  static constexpr int kPBytes = (kWgTok * KP * 2 + 1023) / 1024 * 1024;
  static constexpr int kStage = kQBytes + kPBytes;
  static constexpr int kRing = kWgStages * kStage;
  static constexpr int kStageOff = kRing;                      // per warp [KP][CW] fp32
  // Piece[kWgMaxGroup], int2 bounds[kWgMaxGroup], void* gout[kWgMaxGroup], float scale[kWgMaxGroup]
  static constexpr int kPieceOff = kStageOff + KP * SLAB * 4;
  static constexpr int kBarOff = kPieceOff + kWgMaxGroup * 40;
  static constexpr int kTotal = kBarOff + 2 * kWgStages * 8 + 1024;
  static constexpr int kPartialFloats = KP * SLAB;             // one CTA's partial sums for one run
};

constexpr int kWgMaxJobs = 16;             // jobs one launch can serve (dB and dA of eight projections)

struct WgradJob {
  void* const* g_table;   // device array of npart output pointers
  const void* p;          // [T, R]
  int H;
  int transposed;         // 0: G is [R, H]; 1: G is [H, R]
  int use_scale;
  int slab_begin;         // first slab of this job among the slabs of the launch (grid.y)
};

struct WgradArgs {
  WgradJob job[kWgMaxJobs];
  int njobs;
  int slabs_total;             // slabs of all jobs = grid.y
  const int32_t* part_indptr;  // [npart + 1]
  const float* scale;          // per partition (ids == null) or per adapter, or null
  const int32_t* ids;          // per-partition adapter index for `scale`, or null
  int* plan;                   // plan built on part_indptr: header + pieces
  int* tickets;                // [npart][slabs of both jobs][4 warps], zero between launches
  float* scratch;              // [groups][2][slabs of both jobs][KP * SLAB]
  int n_table;
  int npart, T;
  int R;
  int group;                   // pieces per CTA (G)
  int accumulate;              // G += instead of G =
  int out_fp32;                // G holds fp32 instead of the operand type
  int independent;             // 1: reads nothing the previous kernel of the stream wrote, and
                               //    shares no workspace with it
};

struct WgradMaps {
  CUtensorMap q[kWgMaxJobs];  // Q of every job: boxes of 16 tokens x 64 columns
};

template <typename T, int RT>
__global__ void __launch_bounds__(kWgThreads) wgrad_kernel(const __grid_constant__ WgradArgs a,
                                                           const __grid_constant__ WgradMaps tm) {
  extern __shared__ unsigned char smem_raw[];
  using SM = WgradSmem<RT>;
  constexpr int CW = SM::CW;
  constexpr int SLAB = SM::SLAB;
  constexpr int NCH = SM::NCH;
  constexpr int NTW = CW / 8;  // n-tiles per warp
  constexpr int S = kWgStages;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int G = a.group;
  const int grp = blockIdx.x;
  const int slabs_total = a.slabs_total;
  const int slab_global = blockIdx.y;
  int ji = 0;
  for (int j = 1; j < a.njobs; ++j)
    if (slab_global >= a.job[j].slab_begin) ji = j;
  const WgradJob& jb = a.job[ji];
  void* const* g_table = jb.g_table;
  const T* P = static_cast<const T*>(jb.p);
  const int H = jb.H;
  const int transposed = jb.transposed;
  const int use_scale = jb.use_scale;
  const int col0 = (slab_global - jb.slab_begin) * SLAB;
  const int R = a.R;
  const int ncols = min(SLAB, H - col0);
  int* err = a.plan + 1;

  // dependent launches wait for their predecessor here; independent ones overlap with it and
  // wait just before they exit, so that completion stays in stream order
  if (!a.independent) pdl_wait();
  pdl_trigger();
  const int count = a.plan[0];
  const int pbeg = grp * G;
  const int np = max(0, min(count, pbeg + G) - pbeg);  // pieces of this CTA

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* smem = smem_raw + (base - raw);
  Piece* pcs = reinterpret_cast<Piece*>(smem + SM::kPieceOff);
  int2* bounds = reinterpret_cast<int2*>(smem + SM::kPieceOff + kWgMaxGroup * 16);
  void** gouts = reinterpret_cast<void**>(smem + SM::kPieceOff + kWgMaxGroup * 24);
  float* scales = reinterpret_cast<float*>(smem + SM::kPieceOff + kWgMaxGroup * 32);
  const uint32_t full0 = base + SM::kBarOff;
  const uint32_t empty0 = full0 + S * 8;

  // the first group also clears the gradients of partitions without tokens (they own no piece)
  if (grp == 0 && !a.accumulate) {
    for (int p = warp; p < a.npart; p += kWgThreads / 32) {
      const int ra = a.part_indptr[p], rb = a.part_indptr[p + 1];
      void* gout = g_table[p];
      if (rb != ra || gout == nullptr) continue;
      for (int e = lane; e < R * ncols; e += 32) {
        int r, c;
        if (transposed) { c = e / R; r = e - c * R; } else { r = e / ncols; c = e - r * ncols; }
        const size_t off = transposed ? static_cast<size_t>(col0 + c) * R + r : static_cast<size_t>(r) * H + col0 + c;
        if (a.out_fp32) static_cast<float*>(gout)[off] = 0.f;
        else static_cast<T*>(gout)[off] = static_cast<T>(0.f);
      }
    }
  }
  if (np == 0) {
    if (a.independent) pdl_wait();
    return;
  }

  if (tid < np) {
    Piece pc = reinterpret_cast<const Piece*>(a.plan + kPlanHeaderInts)[pbeg + tid];
    if (pc.pad != 0) {  // a gather piece of a grouped plan: not a row range of one partition
      atomicOr(err, kErrGrouped);
      pc.row0 = 0; pc.nrows = 0; pc.seg = 0;
    }
    pcs[tid] = pc;
    bounds[tid] = make_int2(a.part_indptr[pc.seg], a.part_indptr[pc.seg + 1]);
    gouts[tid] = g_table[pc.seg];
    scales[tid] = use_scale ? adapter_scale(a.scale, a.ids, a.n_table, pc.seg) : 1.0f;
  }
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < S; ++s) {
      mbar_init(full0 + s * 8, 1);
      mbar_init(empty0 + s * 8, 4);
    }
    fence_mbar_init();
  }
  __syncthreads();

  bool dead = false;
  const int nch = (ncols + 63) >> 6;

  if (warp == 4) {
    // ---------------- producer: one stage per piece ----------------
    for (int it = 0; it < np; ++it) {
      const int slot = it % S;
      const int t0 = pcs[it].row0;
      const int ntok = pcs[it].nrows;
      const int nblk = (ntok + 15) >> 4;
      const uint32_t qs = base + slot * SM::kStage;
      const uint32_t ps = qs + SM::kQBytes;
      const uint32_t fb = full0 + slot * 8;
      if (it >= S) mbar_wait(empty0 + slot * 8, ((it / S) - 1) & 1, err, dead);
      const uint32_t pbytes = static_cast<uint32_t>(ntok) * R * 2;
      if (lane == 0) {
        mbar_expect_tx(fb, 2048u * nblk * nch + pbytes);
        bulk_load(ps, P + static_cast<size_t>(t0) * R, pbytes, fb);
      }
      __syncwarp();
      for (int i = lane; i < nblk * nch; i += 32) {
        const int b = i / nch, c = i - b * nch;
        tma_load_2d(qs + (b * NCH + c) * 2048, &tm.q[ji], col0 + c * 64, t0 + b * 16, fb);
      }
    }
    return;
  }

  // ---------------- consumers: warp w owns columns [w*CW, (w+1)*CW) of the slab ----------------
  const int wcol = warp * CW;
  const int ch = wcol >> 6;          // 64-column chunk holding this warp's columns
  const int c0 = (wcol & 63) >> 3;   // first 16-byte chunk inside it
  const bool active = wcol < ncols;

  float acc[RT][NTW][4];
#pragma unroll
  for (int i = 0; i < RT; ++i)
#pragma unroll
    for (int j = 0; j < NTW; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

  // per-warp staging block [KP][CW] fp32: the accumulators leave the registers here, and
  // everything after (output, parking, adding parked partials) runs as short plain loops
  float* st = reinterpret_cast<float*>(smem + SM::kStageOff) + warp * (SM::KP * CW);
  constexpr int kWarpFloats = SM::KP * CW;
  const int cwv = min(CW, ncols - wcol);  // this warp's columns that exist

  auto stage_acc = [&]() {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int i = 0; i < RT; ++i)
#pragma unroll
      for (int j = 0; j < NTW; ++j) {
        *reinterpret_cast<float2*>(st + (i * 16 + g) * CW + j * 8 + 2 * t) = make_float2(acc[i][j][0], acc[i][j][1]);
        *reinterpret_cast<float2*>(st + (i * 16 + g + 8) * CW + j * 8 + 2 * t) =
            make_float2(acc[i][j][2], acc[i][j][3]);
        acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
      }
    __syncwarp();
  };

  // writes this warp's columns of G from the staging block; i0 = a piece of the partition
  auto emit = [&](int i0) {
    void* gout = gouts[i0];
    if (gout == nullptr || (reinterpret_cast<uintptr_t>(gout) & 15) != 0) {
      if (lane == 0) atomicOr(err, kErrBadPointer);
      return;
    }
    const float sc = scales[i0];
    // eight consecutive output elements per lane and step: 16-byte (or 2 x 16-byte fp32) stores
    const int r8 = R >> 3, c8 = (cwv + 7) >> 3;
    const int total = transposed ? cwv * r8 : R * c8;
    for (int e = lane; e < total; e += 32) {
      float v[8];
      size_t off;
      if (transposed) {  // G[H][R]: column c, ranks rh*8 .. rh*8+7
        const int c = e / r8, rh = e - c * r8;
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = st[(rh * 8 + k) * CW + c] * sc;
        off = static_cast<size_t>(col0 + wcol + c) * R + rh * 8;
      } else {           // G[R][H]: rank r, columns ch*8 .. ch*8+7
        const int r = e / c8, chh = e - r * c8;
        const float4 lo = *reinterpret_cast<const float4*>(st + r * CW + chh * 8);
        const float4 hi = *reinterpret_cast<const float4*>(st + r * CW + chh * 8 + 4);
        v[0] = lo.x * sc; v[1] = lo.y * sc; v[2] = lo.z * sc; v[3] = lo.w * sc;
        v[4] = hi.x * sc; v[5] = hi.y * sc; v[6] = hi.z * sc; v[7] = hi.w * sc;
        off = static_cast<size_t>(r) * H + col0 + wcol + chh * 8;
      }
      if (a.out_fp32) {
        float4* q = reinterpret_cast<float4*>(static_cast<float*>(gout) + off);
        if (a.accumulate) {
          const float4 o0 = q[0], o1 = q[1];
          v[0] += o0.x; v[1] += o0.y; v[2] += o0.z; v[3] += o0.w;
          v[4] += o1.x; v[5] += o1.y; v[6] += o1.z; v[7] += o1.w;
        }
        q[0] = make_float4(v[0], v[1], v[2], v[3]);
        q[1] = make_float4(v[4], v[5], v[6], v[7]);
      } else {
        uint4* q = reinterpret_cast<uint4*>(static_cast<T*>(gout) + off);
        if (a.accumulate) {
          const uint4 o = *q;
          const float2 p0 = unpack2<T>(o.x), p1 = unpack2<T>(o.y), p2 = unpack2<T>(o.z), p3 = unpack2<T>(o.w);
          v[0] += p0.x; v[1] += p0.y; v[2] += p1.x; v[3] += p1.y;
          v[4] += p2.x; v[5] += p2.y; v[6] += p3.x; v[7] += p3.y;
        }
        *q = make_uint4(pack2<T>(v[0], v[1]), pack2<T>(v[2], v[3]), pack2<T>(v[4], v[5]), pack2<T>(v[6], v[7]));
      }
    }
  };

  // closes the run of pieces [i0, i1] (indices inside this CTA), all of partition p
  auto close_run = [&](int i0, int i1) {
    const int p = pcs[i0].seg;
    const int ra = bounds[i0].x, rb = bounds[i0].y;
    const bool starts = pcs[i0].row0 == ra;
    const bool ends = pcs[i1].row0 + pcs[i1].nrows == rb;
    stage_acc();
    if (!active) return;
    if (starts && ends) {
      emit(i0);
    } else {
      // the partition's pieces are consecutive in the plan; which groups hold them?
      const int bm = a.plan[3];
      const int first_piece = pbeg + i0 - (pcs[i0].row0 - ra) / bm;
      const int last_piece = first_piece + (rb - ra + bm - 1) / bm - 1;
      const int first_g = first_piece / G, last_g = last_piece / G;
      float* mine = a.scratch + (static_cast<size_t>(grp * 2 + (starts ? 1 : 0)) * slabs_total + slab_global) *
                                    SM::kPartialFloats + warp * kWarpFloats;
      for (int e = lane * 4; e < kWarpFloats; e += 128)
        *reinterpret_cast<float4*>(mine + e) = *reinterpret_cast<const float4*>(st + e);
      __threadfence();
      __syncwarp();
      int* ticket = a.tickets + (static_cast<size_t>(p) * slabs_total + slab_global) * 4 + warp;
      int old = 0;
      if (lane == 0) old = atomicAdd(ticket, 1);
      old = __shfl_sync(0xffffffffu, old, 0);
      if (old == last_g - first_g) {
        // last contributor: add every group's partial in group order (loads of one group are
        // independent of each other and overlap)
        __threadfence();
        constexpr int NV = kWarpFloats / 128;
        float4 s4[NV];
#pragma unroll
        for (int q = 0; q < NV; ++q) s4[q] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 2
        for (int gg = first_g; gg <= last_g; ++gg) {
          const float* src = a.scratch + (static_cast<size_t>(gg * 2 + (gg == first_g ? 1 : 0)) * slabs_total +
                                          slab_global) * SM::kPartialFloats + warp * kWarpFloats + lane * 4;
          float4 v[NV];
#pragma unroll
          for (int q = 0; q < NV; ++q) v[q] = __ldcg(reinterpret_cast<const float4*>(src + q * 128));
#pragma unroll
          for (int q = 0; q < NV; ++q) {
            s4[q].x += v[q].x;
            s4[q].y += v[q].y;
            s4[q].z += v[q].z;
            s4[q].w += v[q].w;
          }
        }
#pragma unroll
        for (int q = 0; q < NV; ++q) *reinterpret_cast<float4*>(st + q * 128 + lane * 4) = s4[q];
        __syncwarp();
        emit(i0);
        if (lane == 0) *ticket = 0;  // leave the workspace ready for the next launch
      }
    }
    __syncwarp();
  };

  int run0 = 0;
  for (int it = 0; it < np; ++it) {
    const int slot = it % S;
    const uint32_t qs = base + slot * SM::kStage;
    const uint32_t ps = qs + SM::kQBytes;
    mbar_wait(full0 + slot * 8, (it / S) & 1, err, dead);
    if (active) {
      const int ntok = pcs[it].nrows;
      const int kmax = (ntok + 15) >> 4;
      for (int kk = 0; kk < kmax; ++kk) {
        const int m = lane >> 3;
        // tokens of this k16 step that exist; the rest of P's rows in the stage are leftovers
        const int valid = ntok - kk * 16;
        uint32_t af[RT][4];
#pragma unroll
        for (int i = 0; i < RT; ++i) {
          // A operand: P^T, rows are rank indices, k are tokens; matrices
          // (m lo, k lo), (m hi, k lo), (m lo, k hi), (m hi, k hi)
          const int t = kk * 16 + (m >> 1) * 8 + (lane & 7);
          ldsm_x4_t(af[i], ps + t * (R * 2) + ((i * 2 + (m & 1)) << 4));
        }
        // registers 0,1 hold tokens 2t, 2t+1; registers 2,3 hold tokens 2t+8, 2t+9 (in both operands)
        const int tk = (lane & 3) * 2;
        const uint32_t lo = (tk < valid ? 0x0000ffffu : 0u) | (tk + 1 < valid ? 0xffff0000u : 0u);
        const uint32_t hi = (tk + 8 < valid ? 0x0000ffffu : 0u) | (tk + 9 < valid ? 0xffff0000u : 0u);
        if (valid < 16) {
#pragma unroll
          for (int i = 0; i < RT; ++i) {
            af[i][0] &= lo;
            af[i][1] &= lo;
            af[i][2] &= hi;
            af[i][3] &= hi;
          }
        }
#pragma unroll
        for (int j = 0; j < NTW; j += 2) {
          // B operand: Q[token][col]; matrices (k lo, n lo), (k hi, n lo), (k lo, n hi), (k hi, n hi)
          uint32_t bf[4];
          const int t = (m & 1) * 8 + (lane & 7);
          const int c = c0 + j + (m >> 1);
          ldsm_x4_t(bf, qs + (kk * NCH + ch) * 2048 + t * 128 + ((c ^ (t & 7)) << 4));
          if (valid < 16) {
            // the Q rows past the piece's end belong to the next partition (or to rows that are not
            // fine-tuned at all): a non-finite value there must not meet the zeroed P (0 x Inf = NaN)
            bf[0] &= lo;
            bf[1] &= hi;
            bf[2] &= lo;
            bf[3] &= hi;
          }
#pragma unroll
          for (int i = 0; i < RT; ++i) {
            mma16816<T>(acc[i][j], af[i], bf[0], bf[1]);
            mma16816<T>(acc[i][j + 1], af[i], bf[2], bf[3]);
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + slot * 8);
    if (it + 1 == np || pcs[it + 1].seg != pcs[it].seg) {
      close_run(run0, it);
      run0 = it + 1;
    }
  }
  if (a.independent) pdl_wait();
}

}  // namespace smlm
