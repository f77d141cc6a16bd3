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

__global__ void __launch_bounds__(kPlanThreads) plan_pieces_kernel(int* __restrict__ plan,
                                                                   const int32_t* __restrict__ indptr, int nseg,
                                                                   int T, int max_pieces, int bm, int max_pieces2,
                                                                   int bm2) {
  __shared__ int s_off[kPlanThreads + 1];
  __shared__ int s_warp[32];
  __shared__ int s_base;
  __shared__ int s_bad;
  const int tid = threadIdx.x;
  int* const plan0 = plan;

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
    const int np = (len + bm - 1) / bm;
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
