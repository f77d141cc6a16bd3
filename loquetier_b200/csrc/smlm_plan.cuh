// Work-list builder: cuts every segment of a batch into pieces of at most `bm` rows
// (bm <= kBM, a multiple of 8, chosen by the host so that the pieces fill whole waves of SMs).
//
// The segment index pointer lives in device memory (the caller of the reference
// operator passes it that way, kernel_src/csrc/loquetier_ops.cc:277-281), so the
// list is built on the device and no host synchronisation is needed.  It replaces
// the reference's per-segment argument kernel
// (kernel_src/csrc/smlm_forward/smlm_forward_cutlass.cuh:31-46): same inputs
// (indptr, per-segment weights), but the output is a list of row ranges instead of
// grouped-GEMM problem descriptors.
//
// Grouped plans.  When the caller also passes the per-segment adapter index, segments of at most
// kGatherMaxLen rows (decode tokens) do not become pieces of their own: their rows are listed, adapter
// by adapter and in batch order, in a row index array behind the piece lists, and every adapter's rows
// are cut into gather pieces of at most kGatherRows rows.  Only adapters with at least two short
// segments are grouped; a lone short segment stays an ordinary piece.  A consumer then fetches an adapter's panels once
// for all of its decode tokens wherever they sit in the batch - the effect the reference gets by
// sorting decode requests by adapter (src/loquetier_src/model_generation.py:186), without requiring
// the order.  The capacity of the list does not change: long and short rows together still need at
// most T / bm + nseg pieces.
//
// Plan buffer layout: int header[4] = {count, error, max_pieces, bm}, then
// Piece[max_pieces + 1]; after it a second list of the same form cut at `bm2` rows, 128
// at most (its error word is unused: faults are always recorded in the first header).
// The tall list feeds the tcgen05 kernel, whose MMA tile is 128 rows.  An indptr that
// is negative, decreasing or reaches past T yields count = 0 in both lists and the
// kErrBadIndptr bit, so that no consumer touches memory.
#pragma once
#include "smlm_common.cuh"

namespace smlm {

constexpr int kPlanThreads = 1024;

// One plan to build: CTA i of the launch builds job i, so the plans of a step (all segments, train
// partitions) cost one launch.
struct PlanJob {
  int* plan;
  const int32_t* indptr;
  const int32_t* ids;
  int nseg, T, max_pieces, bm, max_pieces2, bm2, n_table;
};
constexpr int kPlanMaxJobs = 4;
struct PlanJobs {
  PlanJob job[kPlanMaxJobs];
};

__global__ void __launch_bounds__(kPlanThreads) plan_pieces_kernel(const __grid_constant__ PlanJobs jobs) {
  const PlanJob& J = jobs.job[blockIdx.x];
  int* plan = J.plan;
  const int32_t* __restrict__ indptr = J.indptr;
  const int32_t* __restrict__ ids = J.ids;
  const int nseg = J.nseg, T = J.T, max_pieces2 = J.max_pieces2, bm2 = J.bm2, n_table = J.n_table;
  int max_pieces = J.max_pieces, bm = J.bm;
  __shared__ int s_off[kPlanThreads + 1];
  __shared__ int s_warp[32];
  __shared__ int s_base;
  __shared__ int s_bad;
  __shared__ int s_cnt[kGatherMaxTable];   // rows of short segments per adapter, then the adapter's cursor
  __shared__ int s_nseg[kGatherMaxTable];  // short segments per adapter
  const int tid = threadIdx.x;
  int* const plan0 = plan;
  const bool grouped = ids != nullptr && n_table > 0 && n_table <= kGatherMaxTable;
  int* const rowidx = plan0 + 2 * kPlanHeaderInts + 4 * (max_pieces + 1) + 4 * (max_pieces2 + 1);
  // a short segment with a usable adapter index; the others (a bad index included, which the
  // consumer reports) stay ordinary pieces
  auto is_short = [&](int i, int len) {
    if (!grouped || len < 1 || len > kGatherMaxLen) return false;
    const int a = ids[i];
    return a >= 0 && a < n_table;
  };
  auto is_gathered = [&](int i, int len) { return is_short(i, len) && s_nseg[ids[i]] >= 2; };

  if (tid == 0) {
    s_bad = 0;
    s_base = 0;
  }
  __syncthreads();
  // pass 1: validate the whole index pointer before anything is published
  int bad = 0;
  for (int i = tid; i < nseg; i += kPlanThreads) {
    const int a = indptr[i], b = indptr[i + 1];
    if (a < 0 || b < a || b > T) bad = 1;
  }
  if (bad) s_bad = 1;
  __syncthreads();
  if (s_bad) {
    if (tid == 0) {
      plan[0] = 0;
      plan[1] = kErrBadIndptr;
      plan[2] = max_pieces;
      plan[3] = bm;
      int* second = plan + kPlanHeaderInts + 4 * (max_pieces + 1);
      second[0] = 0;
      second[1] = 0;
      second[2] = max_pieces2;
      second[3] = bm2;
    }
    return;
  }

  if (grouped) {
    for (int a = tid; a < n_table; a += kPlanThreads) {
      s_cnt[a] = 0;
      s_nseg[a] = 0;
    }
    __syncthreads();
    for (int i = tid; i < nseg; i += kPlanThreads) {
      const int len = indptr[i + 1] - indptr[i];
      if (is_short(i, len)) {
        atomicAdd(&s_cnt[ids[i]], len);
        atomicAdd(&s_nseg[ids[i]], 1);
      }
    }
    __syncthreads();
  }

  for (int list = 0; list < 2; ++list) {
  if (list == 1) {
    plan = plan0 + kPlanHeaderInts + 4 * (max_pieces + 1);
    bm = bm2;
    max_pieces = max_pieces2;
    if (tid == 0) s_base = 0;
    __syncthreads();
  }
  Piece* pieces = reinterpret_cast<Piece*>(plan + kPlanHeaderInts);

  // pass 2: 1024 segments at a time: scan the piece counts, then let every
  // thread emit pieces of the chunk by position
  for (int base = 0; base < nseg; base += kPlanThreads) {
    const int i = base + tid;
    int a = 0, len = 0;
    if (i < nseg) {
      a = indptr[i];
      len = indptr[i + 1] - a;
    }
    const int np = (list == 0 && i < nseg && is_gathered(i, len)) ? 0 : (len + bm - 1) / bm;
    // inclusive scan inside the warp
    int v = np;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, v, d);
      if ((tid & 31) >= d) v += t;
    }
    if ((tid & 31) == 31) s_warp[tid >> 5] = v;
    __syncthreads();
    if (tid < 32) {
      int w = s_warp[tid];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, w, d);
        if (tid >= d) w += t;
      }
      s_warp[tid] = w;  // inclusive over warps
    }
    __syncthreads();
    const int excl = v - np + ((tid >> 5) > 0 ? s_warp[(tid >> 5) - 1] : 0);
    s_off[tid] = excl;
    if (tid == kPlanThreads - 1) s_off[kPlanThreads] = excl + np;
    __syncthreads();
    const int chunk_total = s_off[kPlanThreads];
    const int out_base = s_base;
    for (int q = tid; q < chunk_total; q += kPlanThreads) {
      // last segment j of the chunk with s_off[j] <= q (segments without pieces share offsets)
      int lo = 0, hi = kPlanThreads;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_off[mid] <= q) lo = mid; else hi = mid;
      }
      const int j = lo;
      const int seg = base + j;
      const int sa = indptr[seg], sb = indptr[seg + 1];
      const int k = q - s_off[j];
      const int r0 = sa + k * bm;
      if (out_base + q < max_pieces) {
        Piece p;
        p.row0 = r0;
        p.nrows = min(bm, sb - r0);
        p.seg = seg;
        p.pad = 0;
        pieces[out_base + q] = p;
      }
    }
    __syncthreads();
    if (tid == 0) s_base = out_base + chunk_total;
    __syncthreads();
  }
  if (list == 0 && grouped) {
    // ---- gather pieces: rows of short segments, adapter by adapter, in batch order ----
    Piece* gp = pieces;
    constexpr int gh = kGatherRows;
    // exclusive scans over the adapters (four per thread): first row slot and first piece of each
    int cnt4[4], rows = 0, pcs = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int a = tid * 4 + q;
      cnt4[q] = (a < n_table && s_nseg[a] >= 2) ? s_cnt[a] : 0;
      rows += cnt4[q];
      pcs += (cnt4[q] + gh - 1) / gh;
    }
    int vr = rows, vp = pcs;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int tr = __shfl_up_sync(0xffffffffu, vr, d);
      const int tp = __shfl_up_sync(0xffffffffu, vp, d);
      if ((tid & 31) >= d) {
        vr += tr;
        vp += tp;
      }
    }
    __syncthreads();
    if ((tid & 31) == 31) {
      s_warp[tid >> 5] = vr;
      s_off[tid >> 5] = vp;
    }
    __syncthreads();
    if (tid < 32) {
      int wr = s_warp[tid], wp = s_off[tid];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int tr = __shfl_up_sync(0xffffffffu, wr, d);
        const int tp = __shfl_up_sync(0xffffffffu, wp, d);
        if (tid >= d) {
          wr += tr;
          wp += tp;
        }
      }
      s_warp[tid] = wr;
      s_off[tid] = wp;
    }
    __syncthreads();
    int row_at = vr - rows + ((tid >> 5) > 0 ? s_warp[(tid >> 5) - 1] : 0);
    int piece_at = vp - pcs + ((tid >> 5) > 0 ? s_off[(tid >> 5) - 1] : 0);
    const int gather_total = s_off[31];
    const int c0 = s_base;
    __syncthreads();
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int a = tid * 4 + q;
      if (a < n_table) {
        // from here on: the adapter's cursor into the row index array, or -1 when it is not grouped
        s_cnt[a] = cnt4[q] > 0 ? row_at : -1;
        for (int r0 = 0; r0 < cnt4[q]; r0 += gh) {
          if (c0 + piece_at < max_pieces) {
            Piece p;
            p.row0 = row_at + r0;
            p.nrows = min(gh, cnt4[q] - r0);
            p.seg = a;
            p.pad = 1;
            gp[c0 + piece_at] = p;
          }
          ++piece_at;
        }
        row_at += cnt4[q];
      }
    }
    __syncthreads();
    // Stable placement: segments in batch order, 1024 at a time.  Inside a warp the lanes that share an
    // adapter split its cursor by lane order; the warps take their turns at the cursors one after the other.
    for (int base = 0; gather_total > 0 && base < nseg; base += kPlanThreads) {
      const int i = base + tid;
      int a0 = 0, len = 0;
      if (i < nseg) {
        a0 = indptr[i];
        len = indptr[i + 1] - a0;
      }
      const bool sh = i < nseg && is_short(i, len) && s_cnt[ids[i]] >= 0;
      const int key = sh ? ids[i] : (0x40000000 | tid);
      const int mylen = sh ? len : 0;
      const unsigned peers = __match_any_sync(0xffffffffu, key);
      int before = 0, total = 0;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int v = __shfl_sync(0xffffffffu, mylen, j);
        if ((peers >> j) & 1u) {
          total += v;
          if (j < (tid & 31)) before += v;
        }
      }
      const bool first = (peers & ((1u << (tid & 31)) - 1u)) == 0;
      int cur = 0;
      __syncthreads();  // every thread has read its cursor's sign before any cursor moves
      for (int w = 0; w < kPlanThreads / 32; ++w) {
        if ((tid >> 5) == w && sh && first) {
          cur = s_cnt[key];
          s_cnt[key] = cur + total;
        }
        __syncthreads();
      }
      cur = __shfl_sync(0xffffffffu, cur, __ffs(peers) - 1);
      if (sh)
        for (int r = 0; r < len; ++r) rowidx[cur + before + r] = a0 + r;
    }
    if (tid == 0) s_base = c0 + gather_total;
    __syncthreads();
  }
  if (tid == 0) {
    const int total = s_base;
    plan[0] = total <= max_pieces ? total : 0;
    if (list == 0) plan[1] = total <= max_pieces ? 0 : kErrBadIndptr;
    else plan[1] = 0;
    plan[2] = max_pieces;
    plan[3] = bm;
  }
  __syncthreads();
  }  // list
}

}  // namespace smlm
