// Causal self-attention of a ragged batch of prompts over their paged key-value caches, on the
// 5th-generation tensor cores (BatchPrefillWithPagedKVCacheKernel,
// kernel_src/third_party/flashinfer/include/flashinfer/prefill.cuh:904-1060, with the settings of
// FlashInferBatchPrefillKernel, kernel_src/csrc/flashinfer_adapter/flashinfer_all.cu:48-83: causal,
// Llama rotary embedding applied to q and to the keys as they are read, rope scale 1).
//
// One CTA owns 128 rows of one (request, kv head): 128 / G consecutive query positions times the G query
// heads that share the kv head (row = position * G + head, the reference's fusion of the group into the
// row dimension, prefill.cuh:938-943), and walks the keys 0 .. its last position in tiles of 64:
//
//   S[128, 64]   = Q . K_tile^T      tcgen05.mma, A = Q and B = K both K-major in shared memory,
//                                    fp32 accumulator in tensor memory (two buffers: the product of the
//                                    next tile runs under the softmax of this one)
//   P            = exp2(S - m)       thread i owns row i (tensor-memory lane i): no shuffles
//   O[128, 128] += P . V_tile        A = P (written to shared memory as 16-bit), B = V MN-major, i.e.
//                                    exactly as the cache stores it; the accumulator stays in tensor
//                                    memory for the whole walk
//
// The running maximum of a row is only raised when the new one exceeds it by more than 2^8: until then P
// is formed against the old maximum (values up to 256, exact in fp32 sums and harmless in 16 bits), and
// the accumulator needs no rescaling.  When a row of a warp does cross the limit the warp rescales its 32
// rows in tensor memory (tcgen05.ld / tcgen05.st).  The result O / l does not depend on which maximum was
// used.
//
// Keys are stored unrotated, so every tile of K is rotated where it lies in shared memory before the MMA
// reads it (the position of a key is its index in the sequence, prefill.cuh:262,1000); the rotated keys
// are rounded to the storage type.  K and V tiles arrive with 16-byte cp.async copies straight from the
// pages into the 128-byte-swizzled layout that the MMA descriptors name; K and V have their own two-stage
// rings, because a K stage is free as soon as S is formed while V is held until P . V has been read.
// Every wait on an mbarrier is bounded.
#pragma once
#include "paged_kv.cuh"
#include "smlm_fused_tc.cuh"

namespace smlm {

constexpr int kPfRows = 128;                      // rows of a query tile
constexpr int kPfKeys = 64;                       // keys of a tile
constexpr int kPfThreads = 128;
constexpr int kPfQBytes = 2 * kPfRows * 128;      // two 64-dim panels of [128 rows][128 B]
constexpr int kPfKvBytes = 2 * kPfKeys * 128;     // two 64-dim panels of [64 keys][128 B]
constexpr int kPfKOff = kPfQBytes;                // K ring: 2 stages
constexpr int kPfVOff = kPfKOff + 2 * kPfKvBytes; // V ring: 2 stages
constexpr int kPfPOff = kPfVOff + 2 * kPfKvBytes; // P: [128 rows][128 B]
constexpr int kPfBarOff = kPfPOff + kPfRows * 128;
constexpr int kPfSmem = kPfBarOff + 64;           // 3 mbarriers, the tensor-memory address
constexpr int kPfTmemCols = 256;                  // S: 2 x 64 columns, O: 128 columns
constexpr float kPfRaise = 8.0f;                  // a row's maximum is raised when exceeded by this much (log2)
static_assert(2 * (kPfSmem + 1024) <= 228 * 1024, "two CTAs per SM");

struct PfArgs {
  void* o;                        // [total_q, Nq, 128]
  const void* q;                  // [total_q, Nq, 128]
  const int32_t* qo_indptr;       // [B + 1]
  const void* const* kv_ptrs;
  const int32_t* kv_indptr;       // [B + 1]
  const int32_t* last_page_offset;  // [B]
  int* err;                       // error word, may be null
  int batch, num_kv_heads, num_layers, layer_idx, page_size, total_pages, total_q;
  float log2_theta;
};

__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// bounded wait that also works without an error word
__device__ __forceinline__ void pf_wait(uint32_t bar, uint32_t parity, int* err, bool& dead) {
  if (dead) return;
  for (int i = 0; i < kWaitLimit; ++i)
    if (mbar_try_wait(bar, parity)) return;
  dead = true;
  if (err != nullptr) atomicOr(err, kErrTimeout);
}

// grid: (upper bound of query tiles over all requests) * Nkv; a CTA finds its request and tile itself,
// because the query lengths live on the device.
template <typename T, int G>
__global__ void __launch_bounds__(kPfThreads, 2) paged_prefill_kernel(const PfArgs a) {
  extern __shared__ __align__(1024) unsigned char pf_smem[];
  constexpr int PPT = kPfRows / G;   // query positions per tile
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int kvh = blockIdx.x % a.num_kv_heads;
  const int slot = blockIdx.x / a.num_kv_heads;
  const int Nq = a.num_kv_heads * G;
  const int P = a.page_size;

  pdl_wait();
  // ---- which (request, query tile) is slot? every warp runs the same scan ----
  int b = -1, local = 0, ntq = 0;
  {
    int base = 0;
    for (int b0 = 0; b0 < a.batch && b < 0; b0 += 32) {
      const int bb = b0 + lane;
      int n = 0;
      if (bb < a.batch) n = max(0, a.qo_indptr[bb + 1] - a.qo_indptr[bb]);
      const int nt = (n + PPT - 1) / PPT;
      int incl = nt;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
      }
      const unsigned hit = __ballot_sync(0xffffffffu, slot < base + incl);
      if (hit != 0) {
        const int src = __ffs(hit) - 1;
        b = b0 + src;
        ntq = __shfl_sync(0xffffffffu, nt, src);
        local = slot - (base + __shfl_sync(0xffffffffu, incl, src) - ntq);
      }
      base += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  if (b < 0) return;   // a slot past the last tile (uniform over the CTA)
  const int qt = ntq - 1 - local;   // the tiles with the most keys first
  const int qo0 = a.qo_indptr[b];
  const int qo_len = a.qo_indptr[b + 1] - qo0;
  if (qo0 < 0 || qo0 + qo_len > a.total_q) {
    if (tid == 0 && a.err != nullptr) atomicOr(a.err, kErrBadIndptr);
    return;
  }
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
  const int kv_len = npages > 0 ? (npages - 1) * P + last_valid : 0;
  if (kv_len < qo_len && tid == 0 && a.err != nullptr) atomicOr(a.err, kErrBadIndptr);   // more queries than keys
  const int pos0 = kv_len - qo_len;                       // position of the request's first query
  const int qi0 = qt * PPT;                               // first query of the tile
  const int nq = min(PPT, qo_len - qi0);                  // queries of the tile
  const int last_pos = pos0 + qi0 + nq - 1;               // the last key any row of the tile sees
  const int nkeys = max(0, min(kv_len, last_pos + 1));
  const int ntiles = (nkeys + kPfKeys - 1) / kPfKeys;

  const uint32_t sbase = smem_u32(pf_smem);
  if ((sbase & 1023u) != 0) {   // the swizzled layouts need the 1024-byte alignment asked for above
    if (tid == 0 && a.err != nullptr) atomicOr(a.err, kErrBadPointer);
    return;
  }
  const uint32_t qs = sbase;
  const uint32_t ks0 = sbase + kPfKOff;
  const uint32_t vs0 = sbase + kPfVOff;
  const uint32_t ps = sbase + kPfPOff;
  const uint32_t bar_s0 = sbase + kPfBarOff;      // two barriers: S buffers
  const uint32_t bar_o = bar_s0 + 16;
  const uint32_t tmem_slot = bar_s0 + 32;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(pf_smem + kPfBarOff + 32);

  T* O = static_cast<T*>(a.o);
  // this thread's row
  const int my_qi = qi0 + tid / G;
  const int my_head = kvh * G + tid % G;
  const bool my_valid = tid / G < nq;
  const int my_pos = my_valid ? pos0 + my_qi : last_pos;   // rows past the end behave like the last one

  if (ntiles == 0) {   // no key is visible: zeros
    if (my_valid) {
      uint4* op = reinterpret_cast<uint4*>(O + (static_cast<size_t>(qo0 + my_qi) * Nq + my_head) * kPdDim);
#pragma unroll
      for (int i = 0; i < 16; ++i) op[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    return;
  }

  if (tid == 0) {
    mbar_init(bar_s0, 1);
    mbar_init(bar_s0 + 8, 1);
    mbar_init(bar_o, 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tc_alloc(tmem_slot, kPfTmemCols);
    tc_relinquish();
  }

  // ---- loader of K and V tiles: thread = 16-byte column c16 of the 256-byte rows, keys (tid>>4) + 8 i ----
  const size_t head_off = (static_cast<size_t>(a.layer_idx) * 2 * a.num_kv_heads + kvh) * P * kPdDim;
  const size_t kv_delta = static_cast<size_t>(a.num_kv_heads) * P * kPdDim;
  const int lp = 31 - __clz(P);
  bool bad_ptr = false;
  const int c16 = tid & 15;
  const uint32_t ld_off = (c16 >> 3) * (kPfKeys * 128);
  auto load_tile = [&](int j, uint32_t stage, bool value) {
    if (j < ntiles) {
      const int key0 = j * kPfKeys;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int key = (tid >> 4) + 8 * i;
        const int gk = key0 + key;
        const T* src = static_cast<const T*>(a.q);
        bool ok = gk < nkeys;
        if (ok) {
          const T* page = static_cast<const T*>(a.kv_ptrs[p0 + (gk >> lp)]);
          if (page == nullptr || (reinterpret_cast<uintptr_t>(page) & 15) != 0) {
            bad_ptr = true;
            ok = false;
          } else {
            src = page + head_off + (value ? kv_delta : 0) + static_cast<size_t>(gk & (P - 1)) * kPdDim + c16 * 8;
          }
        }
        cp_async16(stage + ld_off + key * 128 + (((c16 & 7) ^ (key & 7)) << 4), src, ok);   // past the end: zeros
      }
    }
    cp_async_commit();
  };
  load_tile(0, ks0, false);
  load_tile(0, vs0, true);
  load_tile(1, ks0 + kPfKvBytes, false);
  load_tile(1, vs0 + kPfKvBytes, true);

  // ---- the rotated, pre-scaled queries: A operand, K-major ----
  {
    const int d0 = (tid & 15) * 4;            // dims d0..d0+3 and their partners d0+64..
    float fr[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      fr[i] = exp2f(-a.log2_theta * static_cast<float>(2 * (d0 + i)) * (1.0f / kPdDim)) * 0.31830988618379067f;
    const float qscale = 1.4426950408889634f * rsqrtf(static_cast<float>(kPdDim));   // log2(e) / sqrt(d)
    for (int r = tid >> 4; r < kPfRows; r += 8) {
      const int qi = qi0 + r / G;
      float ro[4] = {0.f, 0.f, 0.f, 0.f}, rp[4] = {0.f, 0.f, 0.f, 0.f};
      if (r / G < nq) {
        const T* qp = static_cast<const T*>(a.q) + (static_cast<size_t>(qo0 + qi) * Nq + kvh * G + r % G) * kPdDim;
        const uint2 uo = *reinterpret_cast<const uint2*>(qp + d0);
        const uint2 up = *reinterpret_cast<const uint2*>(qp + d0 + 64);
        const float2 o0 = unpack2<T>(uo.x), o1 = unpack2<T>(uo.y), q0 = unpack2<T>(up.x), q1 = unpack2<T>(up.y);
        const float own[4] = {o0.x, o0.y, o1.x, o1.y}, par[4] = {q0.x, q0.y, q1.x, q1.y};
        const float pos = static_cast<float>(max(pos0 + qi, 0));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float sn, cs;
          sincospif(pos * fr[i], &sn, &cs);
          ro[i] = (own[i] * cs - par[i] * sn) * qscale;
          rp[i] = (par[i] * cs + own[i] * sn) * qscale;
        }
      }
      const uint32_t addr = qs + r * 128 + (((d0 >> 3) ^ (r & 7)) << 4) + (d0 & 7) * 2;
      asm volatile("st.shared.v2.b32 [%0], {%1, %2};\n" ::"r"(addr), "r"(pack2<T>(ro[0], ro[1])),
                   "r"(pack2<T>(ro[2], ro[3])) : "memory");
      asm volatile("st.shared.v2.b32 [%0], {%1, %2};\n" ::"r"(addr + kPfRows * 128), "r"(pack2<T>(rp[0], rp[1])),
                   "r"(pack2<T>(rp[2], rp[3])) : "memory");
    }
  }

  // ---- rotation of a K tile in place: warp w owns keys 16 w .. 16 w + 15, lane l the frequencies 2l, 2l+1 ----
  float fr[2], c1[2], s1[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    fr[i] = exp2f(-a.log2_theta * static_cast<float>(2 * (2 * lane + i)) * (1.0f / kPdDim)) * 0.31830988618379067f;
    sincospif(fr[i], &s1[i], &c1[i]);
  }
  auto rotate_tile = [&](int j, uint32_t kst) {
    const int kbase = j * kPfKeys + warp * 16;
    float cc[2], ss[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) sincospif(static_cast<float>(kbase) * fr[i], &ss[i], &cc[i]);
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      const int key = warp * 16 + e;
      const uint32_t ao = kst + key * 128 + ((((lane >> 2) ^ (key & 7))) << 4) + (lane & 3) * 4;
      uint32_t wo, wp;
      asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(wo) : "r"(ao));
      asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(wp) : "r"(ao + kPfKeys * 128));
      const float2 ko = unpack2<T>(wo), kp = unpack2<T>(wp);
      const uint32_t no = pack2<T>(ko.x * cc[0] - kp.x * ss[0], ko.y * cc[1] - kp.y * ss[1]);
      const uint32_t np = pack2<T>(kp.x * cc[0] + ko.x * ss[0], kp.y * cc[1] + ko.y * ss[1]);
      asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(ao), "r"(no) : "memory");
      asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(ao + kPfKeys * 128), "r"(np) : "memory");
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float cn = cc[i] * c1[i] - ss[i] * s1[i];
        ss[i] = ss[i] * c1[i] + cc[i] * s1[i];
        cc[i] = cn;
      }
    }
  };

  tc_fence_before();
  __syncthreads();   // barriers, the tensor-memory address and Q are visible
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;
  const uint32_t my_tmem = tmem + (static_cast<uint32_t>(warp * 32) << 16);
  const uint32_t idesc_s = tc_idesc<T>(kPfKeys, false);
  const uint32_t idesc_o = tc_idesc<T>(kPdDim, true);
  bool dead = false;

  auto issue_s = [&](int j) {   // S(j) = Q . K(j)^T into S buffer j & 1
    const uint32_t kst = ks0 + (j & 1) * kPfKvBytes;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint64_t ad = desc_kmajor(qs + (kk >> 2) * (kPfRows * 128) + (kk & 3) * 32);
      const uint64_t bd = desc_kmajor(kst + (kk >> 2) * (kPfKeys * 128) + (kk & 3) * 32);
      tc_mma(tmem + (j & 1) * kPfKeys, ad, bd, idesc_s, kk > 0 ? 1u : 0u);
    }
    tc_commit(bar_s0 + (j & 1) * 8);
  };

  // first tile of K
  cp_async_wait<3>();
  __syncthreads();
  rotate_tile(0, ks0);
  fence_proxy_async();
  __syncthreads();
  if (tid == 0) {
    tc_fence_after();
    issue_s(0);
  }

  float m_ref = -INFINITY, l_run = 0.f;
  for (int j = 0; j < ntiles; ++j) {
    // A. the next tile's S runs on the tensor cores while this tile's softmax is computed
    if (j + 1 < ntiles) {
      cp_async_wait<1>();
      __syncthreads();
      rotate_tile(j + 1, ks0 + ((j + 1) & 1) * kPfKvBytes);
      fence_proxy_async();
      __syncthreads();
      if (tid == 0) {
        tc_fence_after();
        issue_s(j + 1);
      }
    }
    // B. S(j)
    pf_wait(bar_s0 + (j & 1) * 8, (j >> 1) & 1, a.err, dead);
    tc_fence_after();
    uint32_t sv[2][32];
    tc_ld32(my_tmem + (j & 1) * kPfKeys, sv[0]);
    tc_ld32(my_tmem + (j & 1) * kPfKeys + 32, sv[1]);
    tc_wait_ld();
    load_tile(j + 2, ks0 + (j & 1) * kPfKvBytes, false);   // the K stage of tile j is free
    // C. softmax of this thread's row
    const int lim = my_pos - j * kPfKeys;   // columns above lim are later keys
    float mx = -INFINITY;
    if (lim < kPfKeys - 1) {
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (h * 32 + i > lim) sv[h][i] = __float_as_uint(-INFINITY);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(sv[h][i]));
    float rescale = 1.0f;
    bool raise = false;
    if (mx > m_ref + kPfRaise || m_ref == -INFINITY) {   // (-inf + 8 = -inf: the first visible key always raises)
      if (mx != -INFINITY) {
        raise = m_ref != -INFINITY;
        rescale = exp2f(m_ref - mx);   // 0 when nothing was accumulated yet
        m_ref = mx;
      }
    }
    const float mm = m_ref == -INFINITY ? 0.f : m_ref;
    float sum = 0.f;
    uint32_t pw[32];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const float e0 = exp2f(__uint_as_float(sv[h][i]) - mm), e1 = exp2f(__uint_as_float(sv[h][i + 1]) - mm);
        sum += e0 + e1;
        pw[h * 16 + (i >> 1)] = pack2<T>(e0, e1);
      }
    l_run = l_run * rescale + sum;
    // D. P . V of the previous tile has been read: P, O and its V stage are free
    if (j > 0) {
      pf_wait(bar_o, (j - 1) & 1, a.err, dead);
      tc_fence_after();
      load_tile(j + 1, vs0 + ((j + 1) & 1) * kPfKvBytes, true);
      if (__any_sync(0xffffffffu, raise)) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t ov[32];
          tc_ld32(my_tmem + 2 * kPfKeys + c * 32, ov);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * rescale);
          tc_st32(my_tmem + 2 * kPfKeys + c * 32, ov);
        }
        tc_wait_st();
      }
    } else {
      cp_async_commit();   // keeps the count of copy groups the same in every iteration
    }
    // E. P as the A operand, then O += P . V(j)
#pragma unroll
    for (int c = 0; c < 8; ++c)
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(ps + tid * 128 + ((c ^ (tid & 7)) << 4)),
                   "r"(pw[4 * c]), "r"(pw[4 * c + 1]), "r"(pw[4 * c + 2]), "r"(pw[4 * c + 3]) : "memory");
    cp_async_wait<2>();   // V(j) has landed (this thread's part)
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const uint32_t vst = vs0 + (j & 1) * kPfKvBytes;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const uint64_t ad = desc_kmajor(ps + kk * 32);
        const uint64_t bd = desc_mnmajor(vst + kk * 2048, kPfKeys * 128);
        tc_mma(tmem + 2 * kPfKeys, ad, bd, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
      }
      tc_commit(bar_o);
    }
  }
  cp_async_wait<0>();
  if (__any_sync(0xffffffffu, bad_ptr) && lane == 0 && a.err != nullptr) atomicOr(a.err, kErrBadPointer);

  // ---- the result: O / l ----
  pf_wait(bar_o, (ntiles - 1) & 1, a.err, dead);
  tc_fence_after();
  const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
  T* op = O + (static_cast<size_t>(qo0 + my_qi) * Nq + my_head) * kPdDim;
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    uint32_t ov[32];
    tc_ld32(my_tmem + 2 * kPfKeys + c * 32, ov);
    tc_wait_ld();
    if (my_valid && !dead) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
          w[k] = pack2<T>(__uint_as_float(ov[i * 8 + 2 * k]) * inv, __uint_as_float(ov[i * 8 + 2 * k + 1]) * inv);
        *reinterpret_cast<uint4*>(op + c * 32 + i * 8) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) tc_dealloc(tmem, kPfTmemCols);
}

}  // namespace smlm
