// Run-length merge of a step's requests into segments, on the device.
//
// The reference builds `lora_ids`, `lora_lens` and `segment` on the host with a Python loop
// over the ordered requests: neighbours with the same adapter id become one segment
// (src/loquetier_src/model_generation.py:267-283).  This kernel does the same from two device
// arrays (adapter id and token count per request, in batch row order), so that a serving loop
// that keeps its request table on the GPU never has to copy it back, and the whole step can be
// captured in a CUDA graph.  Integer work: the results are bit-identical to the host loop.
//
// Outputs have room for n entries (there are at most n segments).  Entries past the number of
// segments are zero-length (`seg_len` 0, `seg_indptr` = total tokens, `seg_ids` = last id), which
// every SMLM kernel treats as empty segments; `nseg_out[0]` holds the real count.
#pragma once
#include "smlm_common.cuh"

namespace smlm {

constexpr int kMergeThreads = 1024;

__global__ void __launch_bounds__(kMergeThreads) merge_segments_kernel(
    const int32_t* __restrict__ req_ids, const int32_t* __restrict__ req_len, int n, int32_t* __restrict__ seg_ids,
    int32_t* __restrict__ seg_len, int32_t* __restrict__ seg_indptr, int32_t* __restrict__ nseg_out) {
  __shared__ int s_warp_h[32], s_warp_t[32];
  __shared__ int s_carry_h, s_carry_t;
  const int tid = threadIdx.x;
  pdl_wait();
  pdl_trigger();
  if (tid == 0) {
    s_carry_h = 0;
    s_carry_t = 0;
  }
  __syncthreads();
  for (int base = 0; base < n; base += kMergeThreads) {
    const int i = base + tid;
    const bool in = i < n;
    const int id = in ? req_ids[i] : 0;
    const int len = in ? max(req_len[i], 0) : 0;
    const int head = in && (i == 0 || req_ids[i - 1] != id) ? 1 : 0;
    // inclusive scans of the head flags and of the token counts
    int vh = head, vt = len;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int th = __shfl_up_sync(0xffffffffu, vh, d);
      const int tt = __shfl_up_sync(0xffffffffu, vt, d);
      if ((tid & 31) >= d) {
        vh += th;
        vt += tt;
      }
    }
    if ((tid & 31) == 31) {
      s_warp_h[tid >> 5] = vh;
      s_warp_t[tid >> 5] = vt;
    }
    __syncthreads();
    if (tid < 32) {
      int wh = s_warp_h[tid], wt = s_warp_t[tid];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int th = __shfl_up_sync(0xffffffffu, wh, d);
        const int tt = __shfl_up_sync(0xffffffffu, wt, d);
        if (tid >= d) {
          wh += th;
          wt += tt;
        }
      }
      s_warp_h[tid] = wh;
      s_warp_t[tid] = wt;
    }
    __syncthreads();
    const int w = tid >> 5;
    const int heads_incl = s_carry_h + vh + (w > 0 ? s_warp_h[w - 1] : 0);
    const int tok_excl = s_carry_t + vt - len + (w > 0 ? s_warp_t[w - 1] : 0);
    if (head) {
      const int k = heads_incl - 1;  // segment index of this request
      seg_ids[k] = id;
      seg_indptr[k] = tok_excl;
    }
    __syncthreads();
    if (tid == kMergeThreads - 1) {
      s_carry_h = heads_incl;
      s_carry_t = tok_excl + len;
    }
    __syncthreads();
  }
  const int nseg = s_carry_h, total = s_carry_t;
  // close the index pointer, pad the tail with empty segments, then derive the lengths
  const int last_id = n > 0 ? req_ids[n - 1] : 0;
  for (int k = nseg + tid; k <= n; k += kMergeThreads) {
    seg_indptr[k] = total;
    if (k < n) seg_ids[k] = last_id;
  }
  if (tid == 0) nseg_out[0] = nseg;
  __syncthreads();
  for (int k = tid; k < n; k += kMergeThreads) seg_len[k] = seg_indptr[k + 1] - seg_indptr[k];
}

// Adapter indices for callers that only have one weight pointer per segment (the reference operator's
// arguments, kernel_src/csrc/loquetier_ops.cc:277-281): ids[i] = the first segment whose pointer equals
// w[i].  With the pointer array itself as the adapter table and these ids, a grouped plan gathers the decode
// tokens of one adapter into one piece exactly as it does for callers that keep an adapter table.  Integer
// work; n up to a few thousand, so the quadratic scan (shared-memory tiles of pointers) is microseconds.
constexpr int kGroupThreads = 256;
__global__ void __launch_bounds__(kGroupThreads) pointer_groups_kernel(const void* const* __restrict__ w, int n,
                                                                         int32_t* __restrict__ ids) {
  __shared__ const void* tile[kGroupThreads];
  pdl_wait();
  const int i = blockIdx.x * kGroupThreads + threadIdx.x;
  const void* mine = i < n ? w[i] : nullptr;
  int first = i;
  const int limit = min(n, (static_cast<int>(blockIdx.x) + 1) * kGroupThreads);   // only j < i matters
  for (int j0 = 0; j0 < limit; j0 += kGroupThreads) {
    const int j = j0 + threadIdx.x;
    tile[threadIdx.x] = j < n ? w[j] : nullptr;
    __syncthreads();
    if (i < n && first == i) {
      const int m = min(kGroupThreads, i - j0);   // candidates j0 .. i - 1 of this tile
      for (int k = 0; k < m; ++k) {
        if (tile[k] == mine) {
          first = j0 + k;
          break;
        }
      }
    }
    __syncthreads();
  }
  if (i < n) ids[i] = first;
}

}  // namespace smlm
