// Paged key-value cache: append of new keys/values and batch decode attention over the pages.
//
// The cache is the reference's: a pool of pages, each one tensor [layers, 2, kv_heads, page_size,
// head_dim] (kernel_src/src/loquetier/utils/kvcache.py:40-60; flashinfer's paged_kv_t with pointer
// storage, kernel_src/third_party/flashinfer/include/flashinfer/page.cuh:45-64), reached through a
// device array of page addresses, a page index pointer per request and the number of valid entries
// of each request's last page.  Keys are stored as projected - NOT rotated; the rotary position
// embedding is applied when they are read (decode.cuh:108-111), to the query at position
// seq_len - 1 (:489-494).
//
//   append_kv_kernel   one new token per request   (AppendPagedKVCacheDecodeKernel, page.cuh:368-396)
//   init_kv_kernel     a run of tokens per request (AppendPagedKVCachePrefillKernel, page.cuh:411-444)
//   paged_decode_kernel  o = softmax(rope(q) . rope(K)^T / sqrt(d)) . V per request and head
//                        (BatchDecodeWithPagedKVCacheKernel, decode.cuh:451-620)
//
// Decode is HBM-bound: every K and V page of a (request, kv head) is read exactly once, whatever the
// number of query heads that share the kv head (they are all served by the CTA that streams the
// pages).  A CTA owns one (request, kv head, split): it streams its pages through a ring of shared-
// memory stages (16-byte cp.async, several pages in flight), rotates each key once and dots it with
// the rotated queries of the group, and keeps a running softmax per head.  Rotation angles advance by
// a fixed stride per thread, so they are carried by the angle-addition recurrence (FMA pipe) and
// re-seeded with an accurate evaluation from time to time instead of costing 16 special-function operations
// per key.  Long sequences of small batches are cut into `splits` page ranges so that the machine is
// filled; the partial softmax states go through a workspace and the CTA that finishes last (a
// ticket, no waiting) merges them in split order - a fixed order, so the result does not depend on
// scheduling.
#pragma once
#include "smlm_common.cuh"

namespace smlm {

constexpr int kPdDim = 128;          // head dimension served
constexpr int kPdStages = 6;         // pages in flight per CTA
constexpr int kPdEntryLanes = 8;     // keys of a page processed side by side
constexpr int kPdMaxSplits = 16;
constexpr int kPdReseed = 64;        // keys between two accurate evaluations of the rotation
constexpr int kPdRec = kPdDim + 4;   // floats of a parked softmax state: m, d, two unused, then o[128] (16-byte aligned)

__host__ __device__ constexpr int pd_heads_per_thread(int g) { return g < 4 ? g : 4; }
__host__ __device__ constexpr int pd_threads(int g) { return 128 * (g / pd_heads_per_thread(g)); }

struct PdArgs {
  void* o;                        // [B, Nq, 128]
  const void* q;                  // [B, Nq, 128]
  const void* const* kv_ptrs;     // page addresses
  const int32_t* kv_indptr;       // [B + 1]
  const int32_t* last_page_offset;  // [B]
  int* err;                       // error word (bits of smlm_common.cuh), may be null
  int* tickets;                   // [B * Nkv], zero between launches
  float* partial;                 // [B * Nq * splits * kPdRec]
  int batch, num_kv_heads, num_layers, layer_idx, page_size, splits, total_pages;
  float log2_theta;               // log2(rope base)
};

struct AppendArgs {
  const void* const* kv_ptrs;
  const int32_t* kv_indptr;
  const int32_t* last_page_offset;
  const void* k;                  // [tokens, Nkv, 128]
  const void* v;
  const int32_t* append_indptr;   // [B + 1] for init_kv; null for append_kv (one token per request)
  int* err;
  int batch, num_kv_heads, num_layers, layer_idx, page_size, total_pages;
};

// ---------------------------------------------------------------------------------------------
// append
// ---------------------------------------------------------------------------------------------

// grid: (B * Nkv, token chunks); 16 threads move one 256-byte row each, 8 rows per step
template <typename T>
__global__ void __launch_bounds__(128) append_kv_kernel(const AppendArgs a) {
  const int b = blockIdx.x / a.num_kv_heads;
  const int h = blockIdx.x - b * a.num_kv_heads;
  const int tx = threadIdx.x & 15, row = threadIdx.x >> 4;
  pdl_wait();
  const int p0 = a.kv_indptr[b], p1 = a.kv_indptr[b + 1];
  const int npg = p1 - p0;
  if (npg <= 0 || p0 < 0 || p1 > a.total_pages) {
    if (npg != 0 && threadIdx.x == 0 && a.err != nullptr) atomicOr(a.err, kErrBadIndptr);
    return;
  }
  const int P = a.page_size;
  const int seq_len = (npg - 1) * P + a.last_page_offset[b];
  int src0, n;
  if (a.append_indptr == nullptr) {
    src0 = b;
    n = 1;
  } else {
    src0 = a.append_indptr[b];
    n = a.append_indptr[b + 1] - src0;
  }
  if (n <= 0) return;
  if (n > seq_len) {  // more new tokens than the pages hold
    if (threadIdx.x == 0 && a.err != nullptr) atomicOr(a.err, kErrBadIndptr);
    return;
  }
  const int start = seq_len - n;
  const T* K = static_cast<const T*>(a.k);
  const T* V = static_cast<const T*>(a.v);
  const size_t kv_delta = static_cast<size_t>(a.num_kv_heads) * P * kPdDim;
  for (int j = blockIdx.y * 8 + row; j < n; j += gridDim.y * 8) {
    const int pos = start + j;
    T* page = static_cast<T*>(const_cast<void*>(a.kv_ptrs[p0 + pos / P]));
    if (page == nullptr || (reinterpret_cast<uintptr_t>(page) & 15) != 0) {
      if (tx == 0 && a.err != nullptr) atomicOr(a.err, kErrBadPointer);
      continue;
    }
    T* kd = page + ((static_cast<size_t>(a.layer_idx) * 2 * a.num_kv_heads + h) * P + pos % P) * kPdDim + tx * 8;
    const size_t so = (static_cast<size_t>(src0 + j) * a.num_kv_heads + h) * kPdDim + tx * 8;
    *reinterpret_cast<uint4*>(kd) = *reinterpret_cast<const uint4*>(K + so);
    *reinterpret_cast<uint4*>(kd + kv_delta) = *reinterpret_cast<const uint4*>(V + so);
  }
}

// ---------------------------------------------------------------------------------------------
// decode
// ---------------------------------------------------------------------------------------------

template <typename T>
__device__ __forceinline__ void load8(float (&f)[8], const T* p) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack2<T>(u.x), b = unpack2<T>(u.y), c = unpack2<T>(u.z), d = unpack2<T>(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

// online-softmax state merge in the base-2 domain: (m, d, o) <- (m, d, o) + (m2, d2, o2)
__device__ __forceinline__ void pd_merge(float& m, float& d, float (&o)[8], float m2, float d2, const float (&o2)[8]) {
  if (d2 == 0.f) return;             // an empty state carries no information (and its m may be -inf)
  if (d == 0.f) {
    m = m2; d = d2;
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = o2[i];
    return;
  }
  const float mn = fmaxf(m, m2);
  const float s1 = exp2f(m - mn), s2 = exp2f(m2 - mn);
  d = d * s1 + d2 * s2;
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = o[i] * s1 + o2[i] * s2;
  m = mn;
}

template <typename T, int G>
__global__ void __launch_bounds__(pd_threads(G)) paged_decode_kernel(const PdArgs a) {
  constexpr int HPT = pd_heads_per_thread(G);   // query heads per thread
  constexpr int NT = pd_threads(G);
  extern __shared__ unsigned char pd_smem[];
  __shared__ int s_last;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int tx = lane & 15;                     // dims tx*8 .. tx*8+7
  const int ty = warp >> 2;                     // head block of this thread
  const int ez = ((warp & 3) << 1) | (lane >> 4);   // entry lane 0..7
  const unsigned hmask = (lane & 16) ? 0xffff0000u : 0x0000ffffu;

  const int S = a.splits;
  const int s = blockIdx.x % S;
  const int bh = blockIdx.x / S;
  const int kvh = bh % a.num_kv_heads;
  const int b = bh / a.num_kv_heads;
  const int Nq = a.num_kv_heads * G;
  const int P = a.page_size;
  const int head0 = kvh * G + ty * HPT;

  pdl_wait();
  int p0 = a.kv_indptr[b], p1 = a.kv_indptr[b + 1];
  if (p0 < 0 || p1 < p0 || p1 > a.total_pages) {
    if (tid == 0 && a.err != nullptr) atomicOr(a.err, kErrBadIndptr);
    p1 = p0 = 0;
  }
  const int npages = p1 - p0;
  int last_valid = npages > 0 ? a.last_page_offset[b] : 0;
  if (last_valid < 0 || last_valid > P) {
    if (tid == 0 && a.err != nullptr) atomicOr(a.err, kErrBadIndptr);
    last_valid = 0;
  }
  const int seq_len = npages > 0 ? (npages - 1) * P + last_valid : 0;
  const int per = (npages + S - 1) / S;
  const int pg0 = s * per;
  const int npg = max(0, min(npages, pg0 + per) - pg0);   // pages of this split

  // ---- rotation frequencies and the rotated, pre-scaled queries ----
  float freq[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int dm = (tx * 8 + i) & 63;
    // angles are kept in half-turns (angle / pi): sincospif reduces its argument exactly, whereas the
    // library is built with fast math, under which sincosf loses accuracy at the large angles long
    // sequences reach
    freq[i] = exp2f(-a.log2_theta * static_cast<float>(2 * dm) * (1.0f / kPdDim)) * 0.31830988618379067f;
  }
  const float sgn = tx < 8 ? -1.f : 1.f;       // first half: x cos - partner sin; second: x cos + partner sin
  float qv[HPT][8];
  {
    const float qscale = 1.4426950408889634f * rsqrtf(static_cast<float>(kPdDim));   // log2(e) / sqrt(d)
    const T* Q = static_cast<const T*>(a.q);
    float cq[8], sq[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) sincospif(static_cast<float>(max(seq_len - 1, 0)) * freq[i], &sq[i], &cq[i]);
#pragma unroll
    for (int g = 0; g < HPT; ++g) {
      const T* qp = Q + (static_cast<size_t>(b) * Nq + head0 + g) * kPdDim;
      float own[8], par[8];
      load8<T>(own, qp + tx * 8);
      load8<T>(par, qp + ((tx * 8 + 64) & 127));
#pragma unroll
      for (int i = 0; i < 8; ++i) qv[g][i] = (own[i] * cq[i] + sgn * par[i] * sq[i]) * qscale;
    }
  }

  // ---- stream the pages ----
  const int stage_bytes = 2 * P * kPdDim * static_cast<int>(sizeof(T));
  const uint32_t ring = smem_u32(pd_smem);
  const size_t head_off = (static_cast<size_t>(a.layer_idx) * 2 * a.num_kv_heads + kvh) * P * kPdDim;
  const size_t kv_delta = static_cast<size_t>(a.num_kv_heads) * P * kPdDim;
  const int chunks = P * 16;   // 16-byte chunks per K (or V) page of one head
  bool bad_ptr = false;
  auto issue = [&](int j) {
    if (j < npg) {
      const T* page = static_cast<const T*>(a.kv_ptrs[p0 + pg0 + j]);
      const bool ok = page != nullptr && (reinterpret_cast<uintptr_t>(page) & 15) == 0;
      if (!ok) bad_ptr = true;
      const T* kp = ok ? page + head_off : nullptr;
      const uint32_t dst = ring + (j % kPdStages) * stage_bytes;
      for (int c = tid; c < 2 * chunks; c += NT) {
        const T* src = c < chunks ? kp + c * 8 : kp + kv_delta + (c - chunks) * 8;
        cp_async16(dst + c * 16, ok ? src : static_cast<const T*>(a.q), ok);   // a bad page reads as zeros
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int j = 0; j < kPdStages - 1; ++j) issue(j);

  float m[HPT], d[HPT], o[HPT][8];
#pragma unroll
  for (int g = 0; g < HPT; ++g) {
    m[g] = -INFINITY;
    d[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) o[g][i] = 0.f;
  }
  // rotation of the key this thread handles next: position pos, then pos + 8, pos + 16, ...
  float c8[8], s8[8], cc[8], ss[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) sincospif(8.f * freq[i], &s8[i], &c8[i]);
  int pos = pg0 * P + ez;
  int since_seed = kPdReseed;

  for (int it = 0; it < npg; ++it) {
    issue(it + kPdStages - 1);
    cp_async_wait<kPdStages - 1>();
    __syncthreads();
    const unsigned char* st = pd_smem + (it % kPdStages) * stage_bytes;
    const T* ks = reinterpret_cast<const T*>(st);
    const T* vs = ks + P * kPdDim;
    const int valid = (pg0 + it == npages - 1) ? last_valid : P;
    for (int e = ez; e < valid; e += kPdEntryLanes) {
      if (since_seed >= kPdReseed) {
#pragma unroll
        for (int i = 0; i < 8; ++i) sincospif(static_cast<float>(pos) * freq[i], &ss[i], &cc[i]);
        since_seed = 0;
      }
      float own[8], par[8], kr[8];
      load8<T>(own, ks + e * kPdDim + tx * 8);
      load8<T>(par, ks + e * kPdDim + ((tx * 8 + 64) & 127));
#pragma unroll
      for (int i = 0; i < 8; ++i) kr[i] = own[i] * cc[i] + sgn * par[i] * ss[i];
      float x[HPT];
#pragma unroll
      for (int g = 0; g < HPT; ++g) {
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc = fmaf(qv[g][i], kr[i], acc);
        x[g] = acc;
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1)
#pragma unroll
        for (int g = 0; g < HPT; ++g) x[g] += __shfl_xor_sync(hmask, x[g], off);
      float vv[8];
      load8<T>(vv, vs + e * kPdDim + tx * 8);
#pragma unroll
      for (int g = 0; g < HPT; ++g) {
        const float mn = fmaxf(m[g], x[g]);
        const float sc = exp2f(m[g] - mn);   // exp2f(-inf) = 0 on the first key
        const float p = exp2f(x[g] - mn);
        d[g] = d[g] * sc + p;
#pragma unroll
        for (int i = 0; i < 8; ++i) o[g][i] = fmaf(p, vv[i], o[g][i] * sc);
        m[g] = mn;
      }
      // advance the rotation by eight positions
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float cn = cc[i] * c8[i] - ss[i] * s8[i];
        ss[i] = ss[i] * c8[i] + cc[i] * s8[i];
        cc[i] = cn;
      }
      pos += kPdEntryLanes;
      ++since_seed;
    }
    // a page with fewer valid entries than lanes leaves some lanes behind: keep every lane's position
    // in step with the pages (only the request's last page can be short, so this runs at most once)
    if (valid < P) {
      const int done = ez < valid ? (valid - 1 - ez) / kPdEntryLanes + 1 : 0;
      pos += (P / kPdEntryLanes - done) * kPdEntryLanes;
      since_seed = kPdReseed;
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();
  if (bad_ptr && tid == 0 && a.err != nullptr) atomicOr(a.err, kErrBadPointer);

  // ---- merge the entry lanes in lane order (a fixed order) ----
  // per (ty, ez, g): m, d, then o[128]
  float* red = reinterpret_cast<float*>(pd_smem);
  constexpr int REC = kPdRec;
  {
#pragma unroll
    for (int g = 0; g < HPT; ++g) {
      float* r = red + ((ty * kPdEntryLanes + ez) * HPT + g) * REC;
      if (tx == 0) {
        r[0] = m[g];
        r[1] = d[g];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) r[4 + tx * 8 + i] = o[g][i];
    }
  }
  __syncthreads();
  const bool merger = ez == 0;   // the first half-warp of each head block
  if (merger) {
#pragma unroll
    for (int g = 0; g < HPT; ++g) {
      for (int z = 1; z < kPdEntryLanes; ++z) {
        const float* r = red + ((ty * kPdEntryLanes + z) * HPT + g) * REC;
        float o2[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o2[i] = r[4 + tx * 8 + i];
        pd_merge(m[g], d[g], o[g], r[0], r[1], o2);
      }
    }
  }

  T* O = static_cast<T*>(a.o);
  auto store_out = [&](int g) {
    const float inv = d[g] > 0.f ? 1.0f / d[g] : 0.f;   // a request without keys gives zeros
    uint4 u;
    u.x = pack2<T>(o[g][0] * inv, o[g][1] * inv);
    u.y = pack2<T>(o[g][2] * inv, o[g][3] * inv);
    u.z = pack2<T>(o[g][4] * inv, o[g][5] * inv);
    u.w = pack2<T>(o[g][6] * inv, o[g][7] * inv);
    *reinterpret_cast<uint4*>(O + (static_cast<size_t>(b) * Nq + head0 + g) * kPdDim + tx * 8) = u;
  };

  if (S == 1) {
    if (merger) {
#pragma unroll
      for (int g = 0; g < HPT; ++g) store_out(g);
    }
    return;
  }

  // ---- several splits: park the partial state, the last CTA of the (request, kv head) merges ----
  if (merger) {
#pragma unroll
    for (int g = 0; g < HPT; ++g) {
      float* r = a.partial + ((static_cast<size_t>(b) * Nq + head0 + g) * S + s) * REC;
      if (tx == 0) {
        r[0] = m[g];
        r[1] = d[g];
      }
      *reinterpret_cast<float4*>(r + 4 + tx * 8) = make_float4(o[g][0], o[g][1], o[g][2], o[g][3]);
      *reinterpret_cast<float4*>(r + 4 + tx * 8 + 4) = make_float4(o[g][4], o[g][5], o[g][6], o[g][7]);
    }
    __threadfence();
  }
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(a.tickets + bh, 1);
    s_last = old == S - 1;
    if (old == S - 1) a.tickets[bh] = 0;   // leave the workspace ready for the next launch
  }
  __syncthreads();
  if (!s_last || !merger) return;
  __threadfence();
#pragma unroll
  for (int g = 0; g < HPT; ++g) {
    float mm = -INFINITY, dd = 0.f, oo[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int z = 0; z < S; ++z) {
      const float* r = a.partial + ((static_cast<size_t>(b) * Nq + head0 + g) * S + z) * REC;
      const float m2 = __ldcg(r), d2 = __ldcg(r + 1);
      const float4 lo = __ldcg(reinterpret_cast<const float4*>(r + 4 + tx * 8));
      const float4 hi = __ldcg(reinterpret_cast<const float4*>(r + 4 + tx * 8 + 4));
      const float o2[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
      pd_merge(mm, dd, oo, m2, d2, o2);
    }
    m[g] = mm;
    d[g] = dd;
#pragma unroll
    for (int i = 0; i < 8; ++i) o[g][i] = oo[i];
    store_out(g);
  }
}

}  // namespace smlm
