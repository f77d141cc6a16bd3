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
//                      or a run of tokens per request (AppendPagedKVCachePrefillKernel, page.cuh:411-444)
//   paged_decode_kernel  o = softmax(rope(q) . rope(K)^T / sqrt(d)) . V per request and head
//                        (BatchDecodeWithPagedKVCacheKernel, decode.cuh:451-620)
//
// Decode is HBM-bound: every K and V entry of a (request, kv head) is read exactly once, whatever the
// number of query heads that share the kv head - they are the rows of one tensor-core tile.  Long
// sequences of small batches are cut into `splits` ranges of key tiles so that the machine is filled; the
// partial softmax states go through a workspace and the CTA that finishes last (a ticket, no waiting)
// merges them in range order - a fixed order, so the result does not depend on scheduling.
#pragma once
#include "smlm_common.cuh"

namespace smlm {

constexpr int kPdDim = 128;          // head dimension served
constexpr int kPdStages = 2;         // tiles of 16 keys in flight per warp
constexpr int kPdMaxSplits = 16;
constexpr int kPdRec = kPdDim + 4;   // floats of a parked softmax state: m, d, two unused, then o[128] (16-byte aligned)

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
  // four tokens per thread and step: their page addresses and source rows are fetched together, so that a
  // step costs one round of memory latency instead of four
  constexpr int U = 4;
  const int stride = gridDim.y * 8;
  for (int j0 = blockIdx.y * 8 + row; j0 < n; j0 += U * stride) {
    T* kd[U];
    uint4 kk[U], vv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = j0 + u * stride;
      kd[u] = nullptr;
      kk[u] = vv[u] = make_uint4(0u, 0u, 0u, 0u);
      if (j < n) {
        const int pos = start + j;
        T* page = static_cast<T*>(const_cast<void*>(a.kv_ptrs[p0 + pos / P]));
        if (page == nullptr || (reinterpret_cast<uintptr_t>(page) & 15) != 0) {
          if (tx == 0 && a.err != nullptr) atomicOr(a.err, kErrBadPointer);
        } else {
          kd[u] = page + ((static_cast<size_t>(a.layer_idx) * 2 * a.num_kv_heads + h) * P + pos % P) * kPdDim + tx * 8;
        }
        const size_t so = (static_cast<size_t>(src0 + j) * a.num_kv_heads + h) * kPdDim + tx * 8;
        kk[u] = __ldg(reinterpret_cast<const uint4*>(K + so));
        vv[u] = __ldg(reinterpret_cast<const uint4*>(V + so));
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (kd[u] != nullptr) {
        *reinterpret_cast<uint4*>(kd[u]) = kk[u];
        *reinterpret_cast<uint4*>(kd[u] + kv_delta) = vv[u];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// decode
// ---------------------------------------------------------------------------------------------

// online-softmax state merge in the base-2 domain for N values: (m, d, o) <- (m, d, o) + (m2, d2, o2)
template <int N>
__device__ __forceinline__ void pd_merge(float& m, float& d, float (&o)[N], float m2, float d2, const float (&o2)[N]) {
  if (d2 == 0.f) return;             // an empty state carries no information (and its m may be -inf)
  if (d == 0.f) {
    m = m2; d = d2;
#pragma unroll
    for (int i = 0; i < N; ++i) o[i] = o2[i];
    return;
  }
  const float mn = fmaxf(m, m2);
  const float s1 = exp2f(m - mn), s2 = exp2f(m2 - mn);
  d = d * s1 + d2 * s2;
#pragma unroll
  for (int i = 0; i < N; ++i) o[i] = o[i] * s1 + o2[i] * s2;
  m = mn;
}

constexpr int kPdWarps = 4;                          // each warp streams its own tiles of 16 keys
constexpr int kPdTile = 16;
constexpr int kPdTileBytes = kPdTile * kPdDim * 2;   // one tile of K (or V) of one head: 4 KB
constexpr int kPdWarpRing = kPdStages * 2 * kPdTileBytes;
constexpr int kPdQOff = kPdWarps * kPdWarpRing;      // rotated queries [8 rows][128], then 16 bytes of zeros
constexpr int kPdSmem = kPdQOff + 8 * kPdDim * 2 + 64;

// One CTA = one (request, kv head, range of key tiles).  The G query heads that share the kv head are the
// rows of a 16-row MMA tile (rows G..15 are zero), so every key and value is read once for all of them:
//   S[heads, 16 keys] = Q . K^T  and  O[heads, 128] += P . V  with mma.sync m16n8k16, fp32 accumulation.
// Each warp owns every fourth tile of the range and a private ring of shared-memory stages filled with
// 16-byte cp.async copies (no CTA-wide barrier in the loop).  A tile's keys are rotated where they lie in
// shared memory before the MMA reads them: lane l owns the frequency pair (2l, 2l+1) and walks the 16
// positions of the tile with the angle-addition recurrence, re-seeded exactly at every tile.  The rotated
// keys are rounded to the storage type - what a cache that stores rotated keys holds anyway.
template <typename T, int G>
__global__ void __launch_bounds__(kPdWarps * 32, 3) paged_decode_kernel(const PdArgs a) {
  extern __shared__ __align__(128) unsigned char pd_smem[];
  __shared__ int s_last;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;       // MMA fragment coordinates: row (head) g, column pair t

  const int S = a.splits;
  const int s = blockIdx.x % S;
  const int bh = blockIdx.x / S;
  const int kvh = bh % a.num_kv_heads;
  const int b = bh / a.num_kv_heads;
  const int Nq = a.num_kv_heads * G;
  const int P = a.page_size;
  const int head0 = kvh * G;

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
  const int ntiles = (seq_len + kPdTile - 1) / kPdTile;
  const int per = (ntiles + S - 1) / S;
  const int tile0 = s * per;
  const int ntl = max(0, min(ntiles, tile0 + per) - tile0);   // tiles of this CTA
  const int ntw = ntl > warp ? (ntl - warp + kPdWarps - 1) / kPdWarps : 0;   // tiles of this warp

  // ---- the rotated, pre-scaled queries as the A operand: [8 rows][128] in shared memory ----
  // Angles are kept in half-turns (angle / pi): sincospif reduces its argument exactly, whereas the
  // library is built with fast math, under which sincosf loses accuracy at the angles long sequences reach.
  const uint32_t sbase = smem_u32(pd_smem);
  const uint32_t qs = sbase + kPdQOff;
  {
    const int row = tid >> 4;                 // 8 rows x 16 threads
    const int d0 = (tid & 15) * 4;            // dims d0..d0+3 and their partners d0+64..
    float own[4] = {0.f, 0.f, 0.f, 0.f}, par[4] = {0.f, 0.f, 0.f, 0.f};
    if (row < G) {
      const T* qp = static_cast<const T*>(a.q) + (static_cast<size_t>(b) * Nq + head0 + row) * kPdDim;
      const uint2 uo = *reinterpret_cast<const uint2*>(qp + d0);
      const uint2 up = *reinterpret_cast<const uint2*>(qp + d0 + 64);
      const float2 o0 = unpack2<T>(uo.x), o1 = unpack2<T>(uo.y), q0 = unpack2<T>(up.x), q1 = unpack2<T>(up.y);
      own[0] = o0.x; own[1] = o0.y; own[2] = o1.x; own[3] = o1.y;
      par[0] = q0.x; par[1] = q0.y; par[2] = q1.x; par[3] = q1.y;
    }
    const float qscale = 1.4426950408889634f * rsqrtf(static_cast<float>(kPdDim));   // log2(e) / sqrt(d)
    float ro[4], rp[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float f = exp2f(-a.log2_theta * static_cast<float>(2 * (d0 + i)) * (1.0f / kPdDim)) * 0.31830988618379067f;
      float sn, cs;
      sincospif(static_cast<float>(max(seq_len - 1, 0)) * f, &sn, &cs);
      ro[i] = (own[i] * cs - par[i] * sn) * qscale;
      rp[i] = (par[i] * cs + own[i] * sn) * qscale;
    }
    const int c_own = d0 >> 3, c_par = (d0 + 64) >> 3;
    const uint32_t off = (d0 & 7) * 2;
    asm volatile("st.shared.v2.b32 [%0], {%1, %2};\n" ::"r"(qs + row * 256 + ((c_own ^ row) << 4) + off),
                 "r"(pack2<T>(ro[0], ro[1])), "r"(pack2<T>(ro[2], ro[3])) : "memory");
    asm volatile("st.shared.v2.b32 [%0], {%1, %2};\n" ::"r"(qs + row * 256 + ((c_par ^ row) << 4) + off),
                 "r"(pack2<T>(rp[0], rp[1])), "r"(pack2<T>(rp[2], rp[3])) : "memory");
    if (tid < 4) asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(qs + 8 * 256 + tid * 4), "r"(0) : "memory");
  }
  __syncthreads();
  uint32_t qf[8][4];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    // matrices: (rows 0-7, k lo), (rows 8-15, k lo), (rows 0-7, k hi), (rows 8-15, k hi); rows 8-15 are zeros
    const int m = lane >> 3, r = lane & 7;
    const int chunk = ks * 2 + (m >> 1);
    const uint32_t addr = (m & 1) ? qs + 8 * 256 : qs + r * 256 + ((chunk ^ r) << 4);
    ldsm_x4(qf[ks], addr);
  }

  // ---- this warp's ring and its loader ----
  const uint32_t ring = sbase + warp * kPdWarpRing;
  const size_t head_off = (static_cast<size_t>(a.layer_idx) * 2 * a.num_kv_heads + kvh) * P * kPdDim;
  const size_t kv_delta = static_cast<size_t>(a.num_kv_heads) * P * kPdDim;
  bool bad_ptr = false;
  const int lp = 31 - __clz(P);   // the page size is a power of two (checked by the host)
  // The two halves of a tile (keys 0-7 and 8-15) each lie inside one page (pages hold a multiple of 8
  // entries).  Their addresses are looked up one tile ahead, so that the loads of the page table are
  // in flight while the previous tile is being computed and never sit in front of the copies.
  const T* half_ptr[2] = {nullptr, nullptr};
  auto lookup = [&](int j) {
    half_ptr[0] = half_ptr[1] = nullptr;
    if (j < ntw) {
      const int key0 = (tile0 + warp + j * kPdWarps) * kPdTile;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int gk = key0 + 8 * h;
        if (gk < seq_len) {
          const T* page = static_cast<const T*>(a.kv_ptrs[p0 + (gk >> lp)]);
          if (page == nullptr || (reinterpret_cast<uintptr_t>(page) & 15) != 0) bad_ptr = true;
          else half_ptr[h] = page + head_off + static_cast<size_t>(gk & (P - 1)) * kPdDim;
        }
      }
    }
  };
  auto issue = [&](int j) {   // j-th tile of this warp; its addresses were looked up before
    if (j < ntw) {
      const int key0 = (tile0 + warp + j * kPdWarps) * kPdTile;
      const uint32_t kst = ring + (j % kPdStages) * (2 * kPdTileBytes);
      const int cch = lane & 15;
#pragma unroll
      for (int k = 0; k < kPdTile / 2; ++k) {
        const int key = 2 * k + (lane >> 4);
        const T* hp = half_ptr[k >> 2];
        const bool ok = hp != nullptr && key0 + key < seq_len;
        const T* src = ok ? hp + (key & 7) * kPdDim + cch * 8 : static_cast<const T*>(a.q);
        const uint32_t dst = kst + key * 256 + ((cch ^ (key & 7)) << 4);
        cp_async16(dst, src, ok);                                             // keys past the end read as zeros
        cp_async16(dst + kPdTileBytes, ok ? src + kv_delta : src, ok);
      }
    }
    cp_async_commit();
    lookup(j + 1);
  };
  lookup(0);
#pragma unroll
  for (int j = 0; j < kPdStages - 1; ++j) issue(j);

  // ---- rotation state of this lane: frequencies 2l and 2l + 1 ----
  float fr[2], c1[2], s1[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    fr[i] = exp2f(-a.log2_theta * static_cast<float>(2 * (2 * lane + i)) * (1.0f / kPdDim)) * 0.31830988618379067f;
    sincospif(fr[i], &s1[i], &c1[i]);
  }

  float m_run = -INFINITY, l_run = 0.f;   // row g; l_run is this lane's share of the row sum
  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

  for (int j = 0; j < ntw; ++j) {
    issue(j + kPdStages - 1);
    cp_async_wait<kPdStages - 1>();
    __syncwarp();
    const int key0 = (tile0 + warp + j * kPdWarps) * kPdTile;
    const uint32_t kst = ring + (j % kPdStages) * (2 * kPdTileBytes);
    const uint32_t vst = kst + kPdTileBytes;
    // rotate the 16 keys in place (both frequencies of the lane at once: packed fp32 pairs)
    {
      float cc[2], ss[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) fast_sincospi(static_cast<float>(key0) * fr[i], &ss[i], &cc[i]);
      uint64_t c2 = pack_f32x2(cc[0], cc[1]), s2 = pack_f32x2(ss[0], ss[1]);
      const uint64_t c1p = pack_f32x2(c1[0], c1[1]), s1p = pack_f32x2(s1[0], s1[1]);
      const uint64_t ns1p = pack_f32x2(-s1[0], -s1[1]);
#pragma unroll
      for (int e = 0; e < kPdTile; ++e) {
        const uint32_t ao = kst + e * 256 + ((((lane >> 2) ^ (e & 7))) << 4) + (lane & 3) * 4;
        uint32_t wo, wp;
        asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(wo) : "r"(ao));
        asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(wp) : "r"(ao + 128));
        const float2 kof = unpack2<T>(wo), kpf = unpack2<T>(wp);
        const uint64_t ko = pack_f32x2(kof.x, kof.y), kp = pack_f32x2(kpf.x, kpf.y);
        const uint64_t ns2 = s2 ^ 0x8000000080000000ull;   // -s2: both sign bits flipped
        float a0, a1, b0, b1;
        unpack_f32x2(fma_f32x2(kp, ns2, mul_f32x2(ko, c2)), a0, a1);   // ko * c - kp * s
        unpack_f32x2(fma_f32x2(ko, s2, mul_f32x2(kp, c2)), b0, b1);    // kp * c + ko * s
        asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(ao), "r"(pack2<T>(a0, a1)) : "memory");
        asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(ao + 128), "r"(pack2<T>(b0, b1)) : "memory");
        const uint64_t cn = fma_f32x2(s2, ns1p, mul_f32x2(c2, c1p));   // c c1 - s s1
        s2 = fma_f32x2(c2, s1p, mul_f32x2(s2, c1p));                   // s c1 + c s1
        c2 = cn;
      }
    }
    __syncwarp();
    // S = Q . K^T
    // (even and odd k steps accumulate separately: two shorter chains of dependent MMAs)
    float sc[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t bf[4];
      const int m = lane >> 3;
      const int key = (m >> 1) * 8 + (lane & 7);
      const int chunk = ks * 2 + (m & 1);
      ldsm_x4(bf, kst + key * 256 + ((chunk ^ (key & 7)) << 4));
      mma16816<T>(sc[(ks & 1) * 2], qf[ks], bf[0], bf[1]);
      mma16816<T>(sc[(ks & 1) * 2 + 1], qf[ks], bf[2], bf[3]);
    }
    // running softmax of row g over this lane's keys 2t, 2t+1, 8+2t, 9+2t
    float x[4] = {sc[0][0] + sc[2][0], sc[0][1] + sc[2][1], sc[1][0] + sc[3][0], sc[1][1] + sc[3][1]};
    const int kb = key0 + 2 * t;
    if (kb >= seq_len) x[0] = -INFINITY;
    if (kb + 1 >= seq_len) x[1] = -INFINITY;
    if (kb + 8 >= seq_len) x[2] = -INFINITY;
    if (kb + 9 >= seq_len) x[3] = -INFINITY;
    float mx = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mn = fmaxf(m_run, mx);          // finite: every tile holds at least one valid key
    const float rescale = exp2f(m_run - mn);    // exp2f(-inf) = 0 on the first tile
    float pr[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) pr[i] = exp2f(x[i] - mn);
    l_run = l_run * rescale + (pr[0] + pr[1]) + (pr[2] + pr[3]);
    m_run = mn;
#pragma unroll
    for (int jn = 0; jn < 16; ++jn) {
      o[jn][0] *= rescale;
      o[jn][1] *= rescale;
    }
    // O += P . V ; P is the A operand straight from the registers (rows 8-15 zero)
    uint32_t pa[4] = {pack2<T>(pr[0], pr[1]), 0u, pack2<T>(pr[2], pr[3]), 0u};
#pragma unroll
    for (int jn = 0; jn < 16; jn += 2) {
      uint32_t bf[4];
      const int m = lane >> 3;
      const int key = (m & 1) * 8 + (lane & 7);
      const int chunk = jn + (m >> 1);
      ldsm_x4_t(bf, vst + key * 256 + ((chunk ^ (key & 7)) << 4));
      mma16816<T>(o[jn], pa, bf[0], bf[1]);
      mma16816<T>(o[jn + 1], pa, bf[2], bf[3]);
    }
    __syncwarp();   // the stage is free for the copy issued in the next iteration
  }
  cp_async_wait<0>();
  if (__any_sync(0xffffffffu, bad_ptr) && lane == 0 && a.err != nullptr) atomicOr(a.err, kErrBadPointer);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  __syncthreads();   // every warp is done with its ring: it becomes the merge area

  // ---- merge the warps in warp order (a fixed order): per (warp, row) m, d, 2 unused, o[128] ----
  float* red = reinterpret_cast<float*>(pd_smem);
  constexpr int REC = kPdRec;
  float ov[32];
#pragma unroll
  for (int jn = 0; jn < 16; ++jn) {
    ov[2 * jn] = o[jn][0];
    ov[2 * jn + 1] = o[jn][1];
  }
  if (warp > 0) {
    float* r = red + (warp * 8 + g) * REC;
    if (t == 0) {
      r[0] = m_run;
      r[1] = l_run;
    }
#pragma unroll
    for (int jn = 0; jn < 16; ++jn) *reinterpret_cast<float2*>(r + 4 + jn * 8 + 2 * t) = make_float2(ov[2 * jn], ov[2 * jn + 1]);
  }
  __syncthreads();
  if (warp != 0) {
    if (S == 1) return;
  } else {
    for (int w = 1; w < kPdWarps; ++w) {
      const float* r = red + (w * 8 + g) * REC;
      float o2[32];
#pragma unroll
      for (int jn = 0; jn < 16; ++jn) {
        const float2 v2 = *reinterpret_cast<const float2*>(r + 4 + jn * 8 + 2 * t);
        o2[2 * jn] = v2.x;
        o2[2 * jn + 1] = v2.y;
      }
      pd_merge<32>(m_run, l_run, ov, r[0], r[1], o2);
    }
  }

  T* O = static_cast<T*>(a.o);
  auto store_out = [&]() {   // warp 0: row g = head, this lane's 32 columns
    if (g >= G) return;
    const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;   // a request without keys gives zeros
    T* op = O + (static_cast<size_t>(b) * Nq + head0 + g) * kPdDim;
#pragma unroll
    for (int jn = 0; jn < 16; ++jn)
      *reinterpret_cast<uint32_t*>(op + jn * 8 + 2 * t) = pack2<T>(ov[2 * jn] * inv, ov[2 * jn + 1] * inv);
  };

  if (S == 1) {
    if (warp == 0) store_out();
    return;
  }

  // ---- several ranges: park the partial state, the last CTA of the (request, kv head) merges ----
  if (warp == 0 && g < G) {
    float* r = a.partial + ((static_cast<size_t>(b) * Nq + head0 + g) * S + s) * REC;
    if (t == 0) {
      r[0] = m_run;
      r[1] = l_run;
    }
#pragma unroll
    for (int jn = 0; jn < 16; ++jn) *reinterpret_cast<float2*>(r + 4 + jn * 8 + 2 * t) = make_float2(ov[2 * jn], ov[2 * jn + 1]);
    __threadfence();
  }
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(a.tickets + bh, 1);
    s_last = old == S - 1;
    if (old == S - 1) a.tickets[bh] = 0;   // leave the workspace ready for the next launch
  }
  __syncthreads();
  if (!s_last || warp != 0 || g >= G) return;
  __threadfence();
  m_run = -INFINITY;
  l_run = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) ov[i] = 0.f;
  for (int z = 0; z < S; ++z) {
    const float* r = a.partial + ((static_cast<size_t>(b) * Nq + head0 + g) * S + z) * REC;
    const float m2 = __ldcg(r), d2 = __ldcg(r + 1);
    float o2[32];
#pragma unroll
    for (int jn = 0; jn < 16; ++jn) {
      const float2 v2 = __ldcg(reinterpret_cast<const float2*>(r + 4 + jn * 8 + 2 * t));
      o2[2 * jn] = v2.x;
      o2[2 * jn + 1] = v2.y;
    }
    pd_merge<32>(m_run, l_run, ov, m2, d2, o2);
  }
  store_out();
}

}  // namespace smlm
