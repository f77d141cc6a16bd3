// Per-partition weight gradients  G_p = scale * P[rows_p, :R]^T . Q[rows_p, :H]  for ranks above 32
// on the 5th-generation tensor cores.  Same job description, work cut (a CTA owns `G` consecutive
// 64-token pieces of the partition plan and one slab of Q's columns), workspace and ticket scheme
// as wgrad_kernel (smlm_wgrad.cuh; the products of src/loquetier_src/kernel_utils.py:144-145);
// only the contraction differs: at rank 64 mma.sync with transposing ldmatrix is compute-bound
// at a third of the memory roofline.
//
// The product is formed transposed, D[128 columns of Q, KP ranks] += Q_tile^T . P_tile, so that
// all 128 TMEM lanes carry useful rows for any rank: operand A is the Q tile and operand B the P
// tile, both "MN-major" (tokens are the contraction dimension, rows of the tile), which is exactly
// what a tiled TMA copy of [16 tokens x 64 columns] boxes with the 128-byte swizzle leaves in
// shared memory.  fp32 accumulators live in tensor memory, two sets, so that closing a partition's
// run (TMEM -> registers -> gradient or workspace) overlaps with the next run's MMAs.
//
// Warp roles: warps 0-3 close runs (thread = one column of Q, registers = ranks), warp 4 is the TMA
// producer, warp 5 zeroes the P rows past a ragged piece's end, then issues the MMAs.
#pragma once
#include <cuda.h>

#include "smlm_common.cuh"
#include "smlm_fused_tc.cuh"
#include "smlm_wgrad.cuh"

namespace smlm {

constexpr int kWgTcThreads = 192;
constexpr int wg_tc_slab(int rt) { return rt <= 4 ? 512 : 256; }   // columns of Q per CTA
constexpr int wg_tc_stages(int rt) { return rt <= 4 ? 3 : 4; }

template <int RT>
struct WgradTcSmem {
  static constexpr int KP = RT * 16;                 // 32, 64 or 128
  static constexpr int NB = KP > 64 ? KP / 64 : 1;   // 64-rank blocks of P (a narrower P is zero-filled by TMA)
  static constexpr int SLAB = wg_tc_slab(RT);
  static constexpr int NT = SLAB / 128;              // MMA tiles (128 columns each)
  static constexpr int NCH = SLAB / 64;              // 64-column blocks of Q
  static constexpr int kQBytes = NCH * 8192;         // per block [64 tokens][128 B]
  static constexpr int kPBytes = NB * 8192;
  static constexpr int kStage = kQBytes + kPBytes;
  static constexpr int S = wg_tc_stages(RT);
  static constexpr int kRing = S * kStage;
  static constexpr int kPieceOff = kRing;            // Piece, int2, void*, float per piece of the group
  static constexpr int kBarOff = kPieceOff + kWgMaxGroup * 40;
  static constexpr int kNumBars = 2 * S + 4;
  static constexpr int kTotal = kBarOff + kNumBars * 8 + 16 + 1024;
  static constexpr int kTmemCols = 2 * NT * KP;      // two accumulator sets
  static constexpr int kPartialFloats = KP * SLAB;   // one CTA's partial sums for one run
  static_assert(kTmemCols == 512 || kTmemCols == 256, "tensor memory budget: a power of two, 512 columns at most");
  static_assert(kTotal <= 227 * 1024, "shared memory budget");
};

struct WgradTcMaps {
  CUtensorMap q[kWgMaxJobs];  // Q of every job: boxes of 16 tokens x 64 columns
  CUtensorMap p[kWgMaxJobs];  // P of every job: the same boxes over [T, R]
};

template <typename T, int RT>
__global__ void __launch_bounds__(kWgTcThreads, 1) wgrad_tc_kernel(const __grid_constant__ WgradArgs a,
                                                                   const __grid_constant__ WgradTcMaps tm) {
  extern __shared__ unsigned char smem_raw[];
  using SM = WgradTcSmem<RT>;
  constexpr int KP = SM::KP, NB = SM::NB, SLAB = SM::SLAB, NT = SM::NT, S = SM::S;
  constexpr int NCK = KP / 32;  // 32-rank register chunks per tile
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
  const int H = jb.H;
  const int transposed = jb.transposed;
  const int use_scale = jb.use_scale;
  const int col0 = (slab_global - jb.slab_begin) * SLAB;
  const int R = a.R;
  const int ncols = min(SLAB, H - col0);
  int* err = a.plan + 1;

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
  const uint32_t acc_full0 = empty0 + S * 8;
  const uint32_t acc_empty0 = acc_full0 + 16;
  const uint32_t tmem_slot = acc_empty0 + 16;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem + (tmem_slot - base));

  // the first group also clears the gradients of partitions without tokens (they own no piece)
  if (grp == 0 && !a.accumulate) {
    for (int p = warp; p < a.npart; p += kWgTcThreads / 32) {
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
    for (int s = 0; s < S; ++s) {
      mbar_init(full0 + s * 8, 1);   // the producer's expect_tx arrival; all data comes by TMA
      mbar_init(empty0 + s * 8, 1);  // tcgen05.commit of the MMAs that read the stage
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + b * 8, 1);
      mbar_init(acc_empty0 + b * 8, 128);
    }
    fence_mbar_init();
  }
  if (warp == 5) {
    tc_alloc(tmem_slot, SM::kTmemCols);
    tc_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;

  bool dead = false;
  const int nch = (ncols + 63) >> 6;

  if (warp == 4) {
    // ---------------- producer: one stage per piece ----------------
    for (int it = 0; it < np; ++it) {
      const int slot = it % S;
      const int t0 = pcs[it].row0;
      const int nblk = (pcs[it].nrows + 15) >> 4;
      const uint32_t qs = base + slot * SM::kStage;
      const uint32_t ps = qs + SM::kQBytes;
      const uint32_t fb = full0 + slot * 8;
      if (it >= S) mbar_wait(empty0 + slot * 8, ((it / S) - 1) & 1, err, dead);
      if (dead) break;  // nothing new is put in flight once a wait has given up
      const int per = nch + NB;
      if (lane == 0) mbar_expect_tx(fb, 2048u * nblk * per);
      __syncwarp();
      for (int i = lane; i < nblk * per; i += 32) {
        const int b = i / per, c = i - b * per;
        if (c < nch) tma_load_2d(qs + c * 8192 + b * 2048, &tm.q[ji], col0 + c * 64, t0 + b * 16, fb);
        else tma_load_2d(ps + (c - nch) * 8192 + b * 2048, &tm.p[ji], (c - nch) * 64, t0 + b * 16, fb);
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer ----------------
    // instruction descriptor: fp32 accumulate, A and B MN-major, M = 128, N = KP
    const uint32_t idesc = tc_idesc<T>(KP, true) | (1u << 15);
    int run_idx = 0;
    bool first = true;
    for (int it = 0; it < np; ++it) {
      const int slot = it % S;
      const uint32_t qs = base + slot * SM::kStage;
      const uint32_t ps = qs + SM::kQBytes;
      const int ab = run_idx & 1;
      mbar_wait(full0 + slot * 8, (it / S) & 1, err, dead);
      const int ntok = pcs[it].nrows;
      const int kmax = (ntok + 15) >> 4;
      if (ntok & 15) {
        // the last 16-token step reaches past the piece: those rows of P must not contribute, and the
        // same rows of Q - tokens of the next partition, or of rows that are not fine-tuned - are
        // cleared too, so that a non-finite value there never meets the zeroed P (0 x Inf = NaN).
        // A row is 128 bytes in every block, so clearing whole rows is independent of the swizzle.
        const int nz = kmax * 16 - ntok;
        for (int i = lane; i < NB * nz * 8; i += 32) {
          const int c = i & 7, r = ntok + (i >> 3) % nz, nb = i / (8 * nz);
          asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};\n" ::"r"(ps + nb * 8192 + r * 128 + (c << 4)), "r"(0)
                       : "memory");
        }
        for (int i = lane; i < nch * nz * 8; i += 32) {
          const int c = i & 7, r = ntok + (i >> 3) % nz, qb = i / (8 * nz);
          asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};\n" ::"r"(qs + qb * 8192 + r * 128 + (c << 4)), "r"(0)
                       : "memory");
        }
        fence_proxy_async();
      }
      __syncwarp();
      if (first && run_idx >= 2) mbar_wait(acc_empty0 + ab * 8, ((run_idx >> 1) - 1) & 1, err, dead);
      dead = __any_sync(0xffffffffu, dead);
      tc_fence_after();
      const bool last_of_run = (it + 1 == np) || (pcs[it + 1].seg != pcs[it].seg);
      if (lane == 0) {
        if (!dead) {
          for (int t = 0; t < NT; ++t) {
            if (t * 128 >= ncols) break;
            for (int kk = 0; kk < kmax; ++kk) {
              const uint64_t ad = desc_mnmajor(qs + t * 16384 + kk * 2048, 8192);
              const uint64_t bd = desc_mnmajor(ps + kk * 2048, 8192);
              tc_mma(tmem + (ab * NT + t) * KP, ad, bd, idesc, (first && kk == 0) ? 0u : 1u);
            }
          }
        }
        tc_commit(empty0 + slot * 8);
        if (last_of_run) tc_commit(acc_full0 + ab * 8);
      }
      __syncwarp();
      first = last_of_run;
      if (last_of_run) ++run_idx;
    }
  } else {
    // ---------------- run closers: thread = column (t*128 + 32*warp + lane) of the slab ----------------
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const bool active = warp * 32 < ncols;  // this warp has columns that exist (in tile 0 at least)
    constexpr int kWarpFloats = NT * KP * 32;

    // writes 32 consecutive ranks [r0, r0+32) of column c of the slab
    auto emit = [&](void* gout, float sc, int c, int r0, const uint32_t (&v)[32]) {
      const int nr = R - r0;  // ranks that exist from r0 on (a multiple of 8)
      if (c >= ncols || nr <= 0) return;
      // The old gradient is fetched with straight-line loads at clamped addresses (no branch per
      // element), so that all of them are in flight together; what is past the end is dropped later.
      float old[32];
#pragma unroll
      for (int k = 0; k < 32; ++k) old[k] = 0.f;
      if (transposed) {       // G[H][R]: the thread's ranks are contiguous
        const size_t off = static_cast<size_t>(col0 + c) * R + r0;
        if (a.accumulate) {
          if (a.out_fp32) {
            const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(gout) + off);
            float4 o[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) o[q] = __ldcg(src + (q * 4 < nr ? q : 0));
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              old[q * 4] = o[q].x; old[q * 4 + 1] = o[q].y; old[q * 4 + 2] = o[q].z; old[q * 4 + 3] = o[q].w;
            }
          } else {
            const uint4* src = reinterpret_cast<const uint4*>(static_cast<const T*>(gout) + off);
            uint4 o[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) o[q] = __ldcg(src + (q * 8 < nr ? q : 0));
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 p0 = unpack2<T>(o[q].x), p1 = unpack2<T>(o[q].y), p2 = unpack2<T>(o[q].z),
                           p3 = unpack2<T>(o[q].w);
              old[q * 8] = p0.x; old[q * 8 + 1] = p0.y; old[q * 8 + 2] = p1.x; old[q * 8 + 3] = p1.y;
              old[q * 8 + 4] = p2.x; old[q * 8 + 5] = p2.y; old[q * 8 + 6] = p3.x; old[q * 8 + 7] = p3.y;
            }
          }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (q * 8 < nr) {
            float f[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) f[k] = __uint_as_float(v[q * 8 + k]) * sc + old[q * 8 + k];
            if (a.out_fp32) {
              float4* dst = reinterpret_cast<float4*>(static_cast<float*>(gout) + off + q * 8);
              dst[0] = make_float4(f[0], f[1], f[2], f[3]);
              dst[1] = make_float4(f[4], f[5], f[6], f[7]);
            } else {
              *reinterpret_cast<uint4*>(static_cast<T*>(gout) + off + q * 8) =
                  make_uint4(pack2<T>(f[0], f[1]), pack2<T>(f[2], f[3]), pack2<T>(f[4], f[5]), pack2<T>(f[6], f[7]));
            }
          }
        }
      } else {                // G[R][H]: neighbouring lanes hold neighbouring columns of one rank
        const size_t off0 = static_cast<size_t>(r0) * H + col0 + c;
        if (a.accumulate) {
          if (a.out_fp32) {
            const float* src = static_cast<const float*>(gout) + off0;
#pragma unroll
            for (int k = 0; k < 32; ++k) old[k] = __ldcg(src + static_cast<size_t>(k < nr ? k : 0) * H);
          } else {
            const unsigned short* src = static_cast<const unsigned short*>(gout) + off0;
            unsigned short o[32];
#pragma unroll
            for (int k = 0; k < 32; ++k) o[k] = __ldcg(src + static_cast<size_t>(k < nr ? k : 0) * H);
#pragma unroll
            for (int k = 0; k < 32; ++k) old[k] = unpack2<T>(static_cast<uint32_t>(o[k])).x;
          }
        }
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          if (k < nr) {
            const float f = __uint_as_float(v[k]) * sc + old[k];
            if (a.out_fp32) static_cast<float*>(gout)[off0 + static_cast<size_t>(k) * H] = f;
            else static_cast<T*>(gout)[off0 + static_cast<size_t>(k) * H] = static_cast<T>(f);
          }
        }
      }
    };

    // Accumulating into G reads it first.  Those reads would sit at the end of a run behind a
    // saturated memory system, so the lines are pulled into L2 now, while the tokens stream.
    if (a.accumulate && active) {
      const int esize = a.out_fp32 ? 4 : 2;
      for (int i = 0; i < np; ++i) {
        if (i > 0 && pcs[i].seg == pcs[i - 1].seg) continue;
        const char* g = static_cast<const char*>(gouts[i]);
        if (g == nullptr) continue;
        for (int t = 0; t < NT; ++t) {
          const int c = t * 128 + warp * 32;
          if (c >= ncols) break;
          if (transposed) {   // rows of R elements, one per column; this lane's column
            if (c + lane < ncols)
              for (int b = 0; b < R * esize; b += 128)
                asm volatile("prefetch.global.L2::evict_last [%0];\n" ::"l"(g + (static_cast<size_t>(col0 + c + lane) * R) * esize + b));
          } else {            // per rank one stretch of this warp's 32 columns
            for (int r = lane; r < R; r += 32)
              asm volatile("prefetch.global.L2::evict_last [%0];\n" ::"l"(g + (static_cast<size_t>(r) * H + col0 + c) * esize));
          }
        }
      }
    }

    int run_idx = 0;
    int i0 = 0;
    while (i0 < np) {
      int i1 = i0;
      while (i1 + 1 < np && pcs[i1 + 1].seg == pcs[i0].seg) ++i1;
      const int ab = run_idx & 1;
      mbar_wait(acc_full0 + ab * 8, (run_idx >> 1) & 1, err, dead);
      dead = __any_sync(0xffffffffu, dead);
      tc_fence_after();
      const int p = pcs[i0].seg;
      const int ra = bounds[i0].x, rb = bounds[i0].y;
      const bool starts = pcs[i0].row0 == ra;
      const bool ends = pcs[i1].row0 + pcs[i1].nrows == rb;
      void* gout = gouts[i0];
      const float sc = scales[i0];
      const bool out_ok = gout != nullptr && (reinterpret_cast<uintptr_t>(gout) & 15) == 0;
      if (!out_ok && lane == 0 && active) atomicOr(err, kErrBadPointer);
      const uint32_t acc = tmem + lane_base + ab * NT * KP;
      if (!active || dead) {
        tc_fence_before();
        mbar_arrive(acc_empty0 + ab * 8);
      } else if (starts && ends) {
        // the run holds the whole partition: straight to the gradient
#pragma unroll 1
        for (int t = 0; t < NT; ++t) {
          if (t * 128 + warp * 32 < ncols) {
#pragma unroll 1
            for (int ck = 0; ck < NCK; ++ck) {
              uint32_t v[32];
              tc_ld32(acc + t * KP + ck * 32, v);
              tc_wait_ld();
              if (out_ok) emit(gout, sc, t * 128 + warp * 32 + lane, ck * 32, v);
            }
          }
        }
        tc_fence_before();
        mbar_arrive(acc_empty0 + ab * 8);
      } else {
        // park the partial sums in the workspace and take a ticket; the partition's pieces are
        // consecutive in the plan, so the groups that hold them are known
        const int bm = a.plan[3];
        const int first_piece = pbeg + i0 - (pcs[i0].row0 - ra) / bm;
        const int last_piece = first_piece + (rb - ra + bm - 1) / bm - 1;
        const int first_g = first_piece / G, last_g = last_piece / G;
        float* mine = a.scratch + (static_cast<size_t>(grp * 2 + (starts ? 1 : 0)) * slabs_total + slab_global) *
                                      SM::kPartialFloats + warp * kWarpFloats;
#pragma unroll 1
        for (int t = 0; t < NT; ++t) {
          if (t * 128 + warp * 32 < ncols) {
#pragma unroll 1
            for (int ck = 0; ck < NCK; ++ck) {
              uint32_t v[32];
              tc_ld32(acc + t * KP + ck * 32, v);
              tc_wait_ld();
#pragma unroll
              for (int q = 0; q < 8; ++q)
                *reinterpret_cast<uint4*>(mine + (((t * NCK + ck) * 8 + q) * 32 + lane) * 4) =
                    make_uint4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
            }
          }
        }
        tc_fence_before();
        mbar_arrive(acc_empty0 + ab * 8);
        __threadfence();
        __syncwarp();
        int* ticket = a.tickets + (static_cast<size_t>(p) * slabs_total + slab_global) * 4 + warp;
        int old = 0;
        if (lane == 0) old = atomicAdd(ticket, 1);
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old == last_g - first_g) {
          // last contributor: add every group's partial in group order, a fixed order
          __threadfence();
#pragma unroll 1
          for (int t = 0; t < NT; ++t) {
            if (t * 128 + warp * 32 < ncols) {
#pragma unroll 1
              for (int ck = 0; ck < NCK; ++ck) {
                float s[32];
#pragma unroll
                for (int k = 0; k < 32; ++k) s[k] = 0.f;
                for (int gg = first_g; gg <= last_g; ++gg) {
                  const float* src = a.scratch +
                                     (static_cast<size_t>(gg * 2 + (gg == first_g ? 1 : 0)) * slabs_total + slab_global) *
                                         SM::kPartialFloats +
                                     warp * kWarpFloats + (((t * NCK + ck) * 8) * 32 + lane) * 4;
                  float4 w[8];
#pragma unroll
                  for (int q = 0; q < 8; ++q) w[q] = __ldcg(reinterpret_cast<const float4*>(src + q * 128));
#pragma unroll
                  for (int q = 0; q < 8; ++q) {
                    s[q * 4] += w[q].x;
                    s[q * 4 + 1] += w[q].y;
                    s[q * 4 + 2] += w[q].z;
                    s[q * 4 + 3] += w[q].w;
                  }
                }
                uint32_t v[32];
#pragma unroll
                for (int k = 0; k < 32; ++k) v[k] = __float_as_uint(s[k]);
                if (out_ok) emit(gout, sc, t * 128 + warp * 32 + lane, ck * 32, v);
              }
            }
          }
          if (lane == 0) *ticket = 0;  // leave the workspace ready for the next launch
        }
        __syncwarp();
      }
      i0 = i1 + 1;
      ++run_idx;
    }
  }

  // everyone is done with tensor memory: hand it back
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 5) tc_dealloc(tmem, SM::kTmemCols);
  if (a.independent) pdl_wait();
}

}  // namespace smlm
