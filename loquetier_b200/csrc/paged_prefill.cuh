// Causal self-attention of a ragged batch of prompts over their paged key-value caches, on the
// 5th-generation tensor cores (BatchPrefillWithPagedKVCacheKernel,
// kernel_src/third_party/flashinfer/include/flashinfer/prefill.cuh:904-1060, with the settings of
// FlashInferBatchPrefillKernel, kernel_src/csrc/flashinfer_adapter/flashinfer_all.cu:48-83: causal,
// Llama rotary embedding applied to q and to the keys as they are read, rope scale 1).
//
// Two launches.
//
// prefill_gather_kernel   reads every page of the batch once and writes the keys - rotated for their
//                         position, rounded to the storage type - and the values into a dense scratch
//                         [page slot = page * page_size + entry][K of all kv heads | V of all kv heads].  A
//                         request's slots are consecutive, so a tile of 64 keys of one head is two boxes of a 2-D
//                         tensor map: the attention kernel needs no address arithmetic, no page table and
//                         no rotation in its loop.  Unused entries of a request's last page become zeros.
//
// paged_prefill_kernel    one CTA owns 128 rows of one (request, kv head): 128 / G consecutive query
//                         positions times the G query heads that share the kv head (row = position * G +
//                         head, the reference's fusion of the group into the row dimension,
//                         prefill.cuh:938-943), and walks the keys 0 .. its last position in tiles of 64:
//
//   S[128, 64]   = Q . K_tile^T      tcgen05.mma, A = Q and B = K both K-major in shared memory, fp32
//                                    accumulator in tensor memory (two buffers: the product of the next
//                                    tile runs under the softmax of this one)
//   P            = exp2(S - m)       a row is a tensor-memory lane: two threads per row, no shuffles
//   O[128, 128] += P . V_tile        A = P (written to shared memory as 16-bit), B = V MN-major, i.e.
//                                    exactly as the cache stores it; the accumulator stays in tensor
//                                    memory for the whole walk
//
// Warp roles: warps 0-7 softmax (and the rotation of Q in the prologue) - two threads per row, each with
// half of the columns, because one warp issues a chain of dependent instructions too slowly to keep up
// with the tensor cores; warp 8 the TMA producer of K and V tiles (two-stage rings each: a K stage is free as
// soon as S is formed, V is held until P . V has been read), warp 9 issues the MMAs of S and warp 10 those
// of P . V.  All hand-offs are mbarriers (and one 64-thread barrier per row pair and tile); every wait is
// bounded.
//
// The running maximum of a row is only raised when the new one exceeds it by more than 2^8: until then P
// is formed against the old maximum (values up to 256, exact in fp32 sums and harmless in 16 bits), and
// the accumulator needs no rescaling.  When a row of a warp does cross the limit the warp rescales its 32
// rows in tensor memory (tcgen05.ld / tcgen05.st).  The result O / l does not depend on which maximum was
// used.
#pragma once
#include <cuda.h>

#include "paged_kv.cuh"
#include "smlm_fused_tc.cuh"

namespace smlm {

constexpr int kPfRows = 128;                      // rows of a query tile
// Keys per tile.  64: two S buffers (the next tile's product runs under this tile's softmax) and two-stage
// rings, two CTAs per SM.  128 (one S buffer of 128 columns, one-stage rings, still two CTAs per SM) halves the
// tcgen05.mma instructions per key, but the next S then has to wait for P . V of this tile, which reads P out
// of the same columns: measured slower (0.98 ms against 0.84 ms on the benchmark step).
constexpr int kPfKeys = 64;
constexpr int kPfSBufs = kPfKeys == 64 ? 2 : 1;   // S buffers in tensor memory
constexpr int kPfStages = kPfKeys == 64 ? 2 : 1;  // stages of the K ring and of the V ring
constexpr int kPfThreads = 352;                   // 8 softmax warps, the producer, two MMA issuers
constexpr int kPfQBytes = 2 * kPfRows * 128;      // two 64-dim panels of [128 rows][128 B]
constexpr int kPfKvBytes = 2 * kPfKeys * 128;     // two 64-dim panels of [keys][128 B]
constexpr int kPfKOff = kPfQBytes;
constexpr int kPfVOff = kPfKOff + kPfStages * kPfKvBytes;
constexpr int kPfBarOff = kPfVOff + kPfStages * kPfKvBytes;
constexpr int kPfSmem = kPfBarOff + 4 * kPfStages * 8 + 80;   // the rings' barriers, 8 more, the tensor-memory address
constexpr int kPfOCol = kPfSBufs * kPfKeys;       // first column of O
constexpr int kPfTmemCols = 256;                  // S buffers + O (128 columns)
constexpr int kPfCtasPerSm = 2;
constexpr int kPfHalf = kPfKeys / 2;              // columns of S per softmax thread
constexpr float kPfRaise = 8.0f;                  // a row's maximum is raised when exceeded by this much (log2)
static_assert(kPfKeys == 64 || kPfKeys == 128, "tile of 64 or 128 keys");
static_assert(kPfOCol + 128 <= kPfTmemCols, "tensor memory budget");
static_assert(kPfCtasPerSm * (kPfSmem + 1024) <= 228 * 1024, "shared memory budget");

struct PfArgs {
  void* o;                        // [total_q, Nq, 128]
  const void* q;                  // [total_q, Nq, 128]
  const int32_t* qo_indptr;       // [B + 1]
  const void* const* kv_ptrs;
  const int32_t* kv_indptr;       // [B + 1]
  const int32_t* last_page_offset;  // [B]
  void* scratch;                  // [total_pages * page_size][2 * Nkv * 128]: rotated K | V
  int* err;                       // error word, may be null
  int batch, num_kv_heads, num_layers, layer_idx, page_size, total_pages, total_q;
  float log2_theta;
#ifdef SMLM_PF_TIMING
  long long* timing;              // development builds only: clock stamps of CTA 0
#endif
};

#ifdef SMLM_PF_TIMING
#define PF_STAMP(role, j, k) \
  do { if (blockIdx.x == 0 && (j) < 64) a.timing[((role) * 64 + (j)) * 8 + (k)] = clock64(); } while (0)
#else
#define PF_STAMP(role, j, k) do { } while (0)
#endif

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

// A operand from tensor memory (lane = row, two 16-bit elements of K per 32-bit column), B from shared memory
__device__ __forceinline__ void tc_mma_ts(uint32_t tmem_c, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n}\n"
      ::"r"(tmem_c), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(acc), "r"(0), "r"(0), "r"(0), "r"(0)
      : "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// one column of 32 lanes
__device__ __forceinline__ void tc_st1(uint32_t taddr, uint32_t v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};\n" ::"r"(taddr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t tc_ld1(uint32_t taddr) {   // load and wait for it
  uint32_t v;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];\n"
               "tcgen05.wait::ld.sync.aligned;\n" : "=r"(v) : "r"(taddr) : "memory");
  return v;
}
// 64-thread barrier of the two warps that hold the same rows.  The barrier number is an immediate: with a
// register operand the compiler reserves all 16 hardware barriers for the CTA, and only one CTA fits an SM.
__device__ __forceinline__ void pair_barrier(int wq) {
  switch (wq) {
    case 0: asm volatile("bar.sync 1, 64;\n" ::: "memory"); break;
    case 1: asm volatile("bar.sync 2, 64;\n" ::: "memory"); break;
    case 2: asm volatile("bar.sync 3, 64;\n" ::: "memory"); break;
    default: asm volatile("bar.sync 4, 64;\n" ::: "memory"); break;
  }
}

// bounded wait that also works without an error word
__device__ __forceinline__ void pf_wait(uint32_t bar, uint32_t parity, int* err, bool& dead) {
  if (dead) return;
  for (int i = 0; i < kWaitLimit; ++i) {
#ifdef SMLM_PF_SOFT_NS
    if (mbar_try_wait_for(bar, parity, SMLM_PF_SOFT_NS)) return;
#else
    if (mbar_try_wait(bar, parity)) return;
#endif
  }
  dead = true;
  if (err != nullptr) atomicOr(err, kErrTimeout);
}

// the same for the single-thread roles (producer, issuers), which wait most of the time: polls up to 4 us apart
#ifndef SMLM_PF_ROLE_NS
#define SMLM_PF_ROLE_NS 4000
#endif
__device__ __forceinline__ void pf_wait_role(uint32_t bar, uint32_t parity, int* err, bool& dead) {
  if (dead) return;
  for (int i = 0; i < kWaitLimit; ++i)
    if (mbar_try_wait_for(bar, parity, SMLM_PF_ROLE_NS)) return;
  dead = true;
  if (err != nullptr) atomicOr(err, kErrTimeout);
}

// ---------------------------------------------------------------------------------------------
// gather: pages -> dense scratch, keys rotated
// ---------------------------------------------------------------------------------------------

// grid: one CTA per page of the batch.  Thread = (entry of the page, 8-dim chunk c and its partner c + 8):
// the sines and cosines of its eight frequencies at the entry's position serve all kv heads.
template <typename T>
__global__ void __launch_bounds__(128) prefill_gather_kernel(const PfArgs a) {
  const int pg = blockIdx.x;
  const int P = a.page_size;
  pdl_wait();
  // the request that owns page pg: the last b with kv_indptr[b] <= pg
  int lo = 0, hi = a.batch;   // invariant: kv_indptr[lo] <= pg < kv_indptr[hi] (if the table is sound)
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (a.kv_indptr[mid] <= pg) lo = mid; else hi = mid;
  }
  const int b = lo;
  const int p0 = a.kv_indptr[b], p1 = a.kv_indptr[b + 1];
  T* rowbase = static_cast<T*>(a.scratch) + static_cast<size_t>(pg) * P * (2 * a.num_kv_heads * kPdDim);
  const int row_elems = 2 * a.num_kv_heads * kPdDim;
  const T* page = static_cast<const T*>(a.kv_ptrs[pg]);
  int valid = 0;   // entries of this page that hold tokens
  if (pg >= p0 && pg < p1 && p0 >= 0 && p1 <= a.total_pages) {
    const int lv = a.last_page_offset[b];
    valid = pg == p1 - 1 ? min(max(lv, 0), P) : P;
  }
  if (valid > 0 && (page == nullptr || (reinterpret_cast<uintptr_t>(page) & 15) != 0)) {
    if (threadIdx.x == 0 && a.err != nullptr) atomicOr(a.err, kErrBadPointer);
    valid = 0;
  }
  const size_t kv_delta = static_cast<size_t>(a.num_kv_heads) * P * kPdDim;
  for (int idx = threadIdx.x; idx < P * 8; idx += blockDim.x) {
    const int e = idx >> 3, c = idx & 7;
    T* dst = rowbase + static_cast<size_t>(e) * row_elems;
    if (e >= valid) {   // zeros: nothing that is not a number may sit where a tile can reach
      for (int h = 0; h < a.num_kv_heads; ++h) {
        *reinterpret_cast<uint4*>(dst + h * kPdDim + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(dst + h * kPdDim + 64 + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(dst + (a.num_kv_heads + h) * kPdDim + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(dst + (a.num_kv_heads + h) * kPdDim + 64 + c * 8) = make_uint4(0u, 0u, 0u, 0u);
      }
      continue;
    }
    const float pos = static_cast<float>((pg - p0) * P + e);
    float cs[8], sn[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float f = exp2f(-a.log2_theta * static_cast<float>(2 * (c * 8 + i)) * (1.0f / kPdDim)) * 0.31830988618379067f;
      sincospif(pos * f, &sn[i], &cs[i]);
    }
    for (int h = 0; h < a.num_kv_heads; ++h) {
      const T* src = page + ((static_cast<size_t>(a.layer_idx) * 2 * a.num_kv_heads + h) * P + e) * kPdDim + c * 8;
      const uint4 ko = *reinterpret_cast<const uint4*>(src);
      const uint4 kp = *reinterpret_cast<const uint4*>(src + 64);
      const uint4 vo = *reinterpret_cast<const uint4*>(src + kv_delta);
      const uint4 vp = *reinterpret_cast<const uint4*>(src + kv_delta + 64);
      const uint32_t wo[4] = {ko.x, ko.y, ko.z, ko.w}, wp[4] = {kp.x, kp.y, kp.z, kp.w};
      uint32_t ro[4], rp[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 x = unpack2<T>(wo[i]), y = unpack2<T>(wp[i]);
        ro[i] = pack2<T>(x.x * cs[2 * i] - y.x * sn[2 * i], x.y * cs[2 * i + 1] - y.y * sn[2 * i + 1]);
        rp[i] = pack2<T>(y.x * cs[2 * i] + x.x * sn[2 * i], y.y * cs[2 * i + 1] + x.y * sn[2 * i + 1]);
      }
      *reinterpret_cast<uint4*>(dst + h * kPdDim + c * 8) = make_uint4(ro[0], ro[1], ro[2], ro[3]);
      *reinterpret_cast<uint4*>(dst + h * kPdDim + 64 + c * 8) = make_uint4(rp[0], rp[1], rp[2], rp[3]);
      *reinterpret_cast<uint4*>(dst + (a.num_kv_heads + h) * kPdDim + c * 8) = vo;
      *reinterpret_cast<uint4*>(dst + (a.num_kv_heads + h) * kPdDim + 64 + c * 8) = vp;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// attention
// ---------------------------------------------------------------------------------------------

// grid: (upper bound of query tiles over all requests) * Nkv; a CTA finds its request and tile itself,
// because the query lengths live on the device.  kvmap: the scratch as [slots][2 * Nkv * 128], boxes of a tile's
// slots x 64 columns with the 128-byte swizzle.
template <typename T, int G>
__global__ void __launch_bounds__(kPfThreads, kPfCtasPerSm) paged_prefill_kernel(const PfArgs a,
                                                                      const __grid_constant__ CUtensorMap kvmap) {
  extern __shared__ __align__(1024) unsigned char pf_smem[];
  constexpr int PPT = kPfRows / G;   // query positions per tile
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int kvh = blockIdx.x % a.num_kv_heads;
  const int slot = blockIdx.x / a.num_kv_heads;
  const int Nq = a.num_kv_heads * G;
  const int P = a.page_size;

  if (tid == 0) PF_STAMP(0, 63, 0);
  pdl_wait();
  // ---- which (request, query tile) is slot? every warp runs the same scan ----
  // (each lane also fetches its request's page range, so that everything arrives with one memory latency)
  int b = -1, local = 0, ntq = 0;
  int qo0 = 0, qo_len = 0, p0 = 0, p1 = 0, last_valid = 0;
  {
    int base = 0;
    for (int b0 = 0; b0 < a.batch && b < 0; b0 += 32) {
      const int bb = b0 + lane;
      int q0l = 0, q1l = 0, k0l = 0, k1l = 0, lvl = 0;
      if (bb < a.batch) {
        q0l = a.qo_indptr[bb]; q1l = a.qo_indptr[bb + 1];
        k0l = a.kv_indptr[bb]; k1l = a.kv_indptr[bb + 1];
        lvl = a.last_page_offset[bb];
      }
      const int n = max(0, q1l - q0l);
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
        qo0 = __shfl_sync(0xffffffffu, q0l, src);
        qo_len = __shfl_sync(0xffffffffu, q1l, src) - qo0;
        p0 = __shfl_sync(0xffffffffu, k0l, src);
        p1 = __shfl_sync(0xffffffffu, k1l, src);
        last_valid = __shfl_sync(0xffffffffu, lvl, src);
      }
      base += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  if (b < 0) return;   // a slot past the last tile (uniform over the CTA)
  const int qt = ntq - 1 - local;   // the tiles with the most keys first
  if (qo0 < 0 || qo0 + qo_len > a.total_q) {
    if (tid == 0 && a.err != nullptr) atomicOr(a.err, kErrBadIndptr);
    return;
  }
  if (p0 < 0 || p1 < p0 || p1 > a.total_pages) {
    if (tid == 0 && a.err != nullptr) atomicOr(a.err, kErrBadIndptr);
    p1 = p0 = 0;
  }
  const int npages = p1 - p0;
  if (npages == 0) last_valid = 0;
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
  const uint32_t bars = sbase + kPfBarOff;
  constexpr int NS = kPfStages;
  const uint32_t k_full = bars, k_empty = bars + NS * 8, v_full = bars + 2 * NS * 8, v_empty = bars + 3 * NS * 8;
  const uint32_t s_full = bars + 4 * NS * 8, s_empty = s_full + 16;                              // two each
  // o_done: two barriers used by alternate tiles.  A softmax thread consumes the completion of tile j - 1
  // after it has released tile j; with a single barrier the product of tile j could complete in between and
  // the parity of tile j - 1 could no longer be told from that of tile j + 1.
  const uint32_t p_full = s_full + 32, o_done = s_full + 40, q_full = s_full + 56;
  const uint32_t tmem_slot = s_full + 64;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(pf_smem + kPfBarOff + 4 * NS * 8 + 64);

  T* O = static_cast<T*>(a.o);
  if (ntiles == 0) {   // no key is visible: zeros
    if (tid < kPfRows && tid / G < nq) {
      uint4* op = reinterpret_cast<uint4*>(O + (static_cast<size_t>(qo0 + qi0 + tid / G) * Nq + kvh * G + tid % G) * kPdDim);
#pragma unroll
      for (int i = 0; i < 16; ++i) op[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    return;
  }

  // The queries of the tile: 16 threads per row (4 dims and their partners each), 16 rows per pass.  All loads
  // of a softmax thread go out here, so that their latency passes behind the barrier set-up and the
  // tensor-memory allocation below; the rotation that consumes them follows the allocation.
  uint2 qo_raw[kPfRows / 16], qp_raw[kPfRows / 16];
#pragma unroll
  for (int it = 0; it < kPfRows / 16; ++it) qo_raw[it] = qp_raw[it] = make_uint2(0u, 0u);
  if (warp < 8) {
    const int d0 = (tid & 15) * 4;
    const int rg = tid >> 4;
#pragma unroll
    for (int it = 0; it < kPfRows / 16; ++it) {
      const int r = rg + 16 * it;
      if (r / G < nq) {
        const T* qp = static_cast<const T*>(a.q) + (static_cast<size_t>(qo0 + qi0 + r / G) * Nq + kvh * G + r % G) * kPdDim;
        qo_raw[it] = __ldg(reinterpret_cast<const uint2*>(qp + d0));
        qp_raw[it] = __ldg(reinterpret_cast<const uint2*>(qp + d0 + 64));
      }
    }
  }

  if (tid == 0) PF_STAMP(0, 63, 1);
  if (tid == 0) {
    for (int i = 0; i < NS; ++i) {
      mbar_init(k_full + i * 8, 1);
      mbar_init(k_empty + i * 8, 1);
      mbar_init(v_full + i * 8, 1);
      mbar_init(v_empty + i * 8, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(s_full + i * 8, 1);
      mbar_init(s_empty + i * 8, 1);   // P lives in the S buffer: freed by the commit of P . V
    }
    mbar_init(p_full, 2 * kPfRows);
    mbar_init(o_done, 1);
    mbar_init(o_done + 8, 1);
    mbar_init(q_full, 2 * kPfRows);
    fence_mbar_init();
  }
  if (warp == 9) {
    tc_alloc(tmem_slot, kPfTmemCols);
    tc_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;
  bool dead = false;
  if (tid == 0) PF_STAMP(0, 63, 2);

  if (warp == 8) {
    // ---------------- producer: K and V tiles by TMA ----------------
    if (lane == 0) {
      const int row0 = p0 * P;                    // the request's first slot of the scratch
      const int xk = kvh * kPdDim, xv = (a.num_kv_heads + kvh) * kPdDim;
      for (int j = 0; j < ntiles; ++j) {
        const int st = j % NS, use = j / NS;
        const int y = row0 + j * kPfKeys;
        if (use > 0) pf_wait_role(k_empty + st * 8, (use - 1) & 1, a.err, dead);
        if (dead) break;   // nothing new is put in flight once a wait has given up
        mbar_expect_tx(k_full + st * 8, kPfKvBytes);
        tma_load_2d(ks0 + st * kPfKvBytes, &kvmap, xk, y, k_full + st * 8);
        tma_load_2d(ks0 + st * kPfKvBytes + kPfKeys * 128, &kvmap, xk + 64, y, k_full + st * 8);
        if (use > 0) pf_wait_role(v_empty + st * 8, (use - 1) & 1, a.err, dead);
        if (dead) break;
        mbar_expect_tx(v_full + st * 8, kPfKvBytes);
        tma_load_2d(vs0 + st * kPfKvBytes, &kvmap, xv, y, v_full + st * 8);
        tma_load_2d(vs0 + st * kPfKvBytes + kPfKeys * 128, &kvmap, xv + 64, y, v_full + st * 8);
      }
    }
  } else if (warp == 9) {
    // ---------------- issuer of S = Q . K^T: runs up to two tiles ahead of the softmax ----------------
    if (lane == 0) {
      const uint32_t idesc_s = tc_idesc<T>(kPfKeys, false);
      pf_wait_role(q_full, 0, a.err, dead);
      for (int j = 0; j < ntiles; ++j) {
        const int st = j % NS, sb = j % kPfSBufs, use = j / kPfSBufs;
        pf_wait_role(k_full + st * 8, (j / NS) & 1, a.err, dead);
        if (use > 0) pf_wait_role(s_empty + sb * 8, (use - 1) & 1, a.err, dead);
        tc_fence_after();
        if (!dead) {
          const uint32_t kst = ks0 + st * kPfKvBytes;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t ad = desc_kmajor(qs + (kk >> 2) * (kPfRows * 128) + (kk & 3) * 32);
            const uint64_t bd = desc_kmajor(kst + (kk >> 2) * (kPfKeys * 128) + (kk & 3) * 32);
            tc_mma(tmem + sb * kPfKeys, ad, bd, idesc_s, kk > 0 ? 1u : 0u);
          }
        }
        tc_commit(k_empty + st * 8);
        tc_commit(s_full + sb * 8);
        PF_STAMP(1, j, 0);
      }
    }
  } else if (warp == 10) {
    // ---------------- issuer of O += P . V (a thread of its own: one thread issuing both products was
    // the slowest link of the chain) ----------------
    if (lane == 0) {
      const uint32_t idesc_o = tc_idesc<T>(kPdDim, true);
      for (int j = 0; j < ntiles; ++j) {
        const int st = j % NS;
        pf_wait_role(v_full + st * 8, (j / NS) & 1, a.err, dead);
        PF_STAMP(1, j, 1);
        pf_wait_role(p_full, j & 1, a.err, dead);
        PF_STAMP(1, j, 2);
        tc_fence_after();
        if (!dead) {
          const uint32_t vst = vs0 + st * kPfKvBytes;
#pragma unroll
          for (int kk = 0; kk < kPfKeys / 16; ++kk) {
            const uint64_t bd = desc_mnmajor(vst + kk * 2048, kPfKeys * 128);
            // keys 16 kk .. 16 kk + 15: eight columns in the upper half of the columns of the thread that made them
            constexpr int PER = kPfHalf / 16;
            const uint32_t pa = tmem + (j % kPfSBufs) * kPfKeys + (kk / PER) * kPfHalf + kPfHalf / 2 + (kk % PER) * 8;
            tc_mma_ts(tmem + kPfOCol, pa, bd, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
          }
        }
        tc_commit(s_empty + (j % kPfSBufs) * 8);   // the S buffer held P: free for the next product into it
        tc_commit(v_empty + st * 8);
        tc_commit(o_done + (j & 1) * 8);
        PF_STAMP(1, j, 3);
      }
    }
  } else {
    // ---------------- softmax warps: thread = (row, half of the columns) ----------------
    // Warps w and w + 4 hold the same 32 rows (a warp reaches the tensor-memory lanes 32 (w mod 4) ...):
    // the first takes columns 0-31 of a tile of S and 0-63 of O, the second the rest.  The two threads of a
    // row agree on the row's maximum through tensor memory itself: each parks its half's maximum in a
    // column of the S buffer that it has already read, and reads the other's after a 64-thread barrier.
    const int half = warp >> 2;
    const int wq = warp & 3;
    const int row = wq * 32 + lane;
    const int my_qi = qi0 + row / G;
    const int my_head = kvh * G + row % G;
    const bool my_valid = row / G < nq;
    const int my_pos = my_valid ? pos0 + my_qi : last_pos;   // rows past the end behave like the last one
    const uint32_t my_tmem = tmem + (static_cast<uint32_t>(wq * 32) << 16);
    const uint32_t o_tmem = my_tmem + kPfOCol + half * 64;

    // the rotated, pre-scaled queries: A operand, K-major.  16 threads per row (4 dims and their partners
    // each), 16 rows per pass; the position advances by 16 / G per pass, so the angle is stepped, not recomputed
    {
      const int d0 = (tid & 15) * 4;
      const int rg = tid >> 4;
      constexpr int STEP = 16 / G;
      const float qscale = 1.4426950408889634f * rsqrtf(static_cast<float>(kPdDim));   // log2(e) / sqrt(d)
      // cos and sin of the four dimensions as two packed pairs, with the softmax scale folded in (a rotation
      // is linear, so the stepped pair keeps the factor); the step's own cos and sin carry none
      uint64_t cc2[2], ss2[2], c12[2], s12[2];
      {
        float cc[4], ss[4], c1[4], s1[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float f = exp2f(-a.log2_theta * static_cast<float>(2 * (d0 + i)) * (1.0f / kPdDim)) * 0.31830988618379067f;
          fast_sincospi(static_cast<float>(pos0 + qi0 + rg / G) * f, &ss[i], &cc[i]);
          fast_sincospi(static_cast<float>(STEP) * f, &s1[i], &c1[i]);
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          cc2[k] = pack_f32x2(cc[2 * k] * qscale, cc[2 * k + 1] * qscale);
          ss2[k] = pack_f32x2(ss[2 * k] * qscale, ss[2 * k + 1] * qscale);
          c12[k] = pack_f32x2(c1[2 * k], c1[2 * k + 1]);
          s12[k] = pack_f32x2(s1[2 * k], s1[2 * k + 1]);
        }
      }
      constexpr uint64_t kNeg2 = 0x8000000080000000ull;   // flips the sign of both halves
#pragma unroll
      for (int it = 0; it < kPfRows / 16; ++it) {
        const int r = rg + 16 * it;
        uint32_t wo[2] = {0u, 0u}, wp[2] = {0u, 0u};
        if (r / G < nq) {
          const uint32_t uo[2] = {qo_raw[it].x, qo_raw[it].y}, up[2] = {qp_raw[it].x, qp_raw[it].y};
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            const float2 o = unpack2<T>(uo[k]), q = unpack2<T>(up[k]);
            const uint64_t own = pack_f32x2(o.x, o.y), par = pack_f32x2(q.x, q.y);
            float x0, x1;
            unpack_f32x2(fma_f32x2(own, cc2[k], mul_f32x2(par, ss2[k] ^ kNeg2)), x0, x1);   // own cos - partner sin
            wo[k] = pack2<T>(x0, x1);
            unpack_f32x2(fma_f32x2(par, cc2[k], mul_f32x2(own, ss2[k])), x0, x1);           // partner cos + own sin
            wp[k] = pack2<T>(x0, x1);
          }
        }
        const uint32_t addr = qs + r * 128 + (((d0 >> 3) ^ (r & 7)) << 4) + (d0 & 7) * 2;
        asm volatile("st.shared.v2.b32 [%0], {%1, %2};\n" ::"r"(addr), "r"(wo[0]), "r"(wo[1]) : "memory");
        asm volatile("st.shared.v2.b32 [%0], {%1, %2};\n" ::"r"(addr + kPfRows * 128), "r"(wp[0]), "r"(wp[1]) : "memory");
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const uint64_t cn = fma_f32x2(cc2[k], c12[k], mul_f32x2(ss2[k] ^ kNeg2, s12[k]));
          ss2[k] = fma_f32x2(ss2[k], c12[k], mul_f32x2(cc2[k], s12[k]));
          cc2[k] = cn;
        }
      }
      fence_proxy_async();   // the MMA reads Q through the async proxy
      mbar_arrive(q_full);
      if (tid == 0) PF_STAMP(0, 63, 3);
    }

    float m_ref = -INFINITY;
    uint64_t l2 = pack_f32x2(0.f, 0.f);   // this thread's share of the row sum, two lanes
    for (int j = 0; j < ntiles; ++j) {
      const int sb = j % kPfSBufs;
      if (tid == 0) PF_STAMP(0, j, 0);
      pf_wait(s_full + sb * 8, (j / kPfSBufs) & 1, a.err, dead);
      if (tid == 0) PF_STAMP(0, j, 1);
      tc_fence_after();
      constexpr int HC = kPfHalf;
      constexpr int NCH = HC / 32;           // the thread's columns are handled 32 at a time
      const uint32_t my_s = my_tmem + sb * kPfKeys + half * HC;
      const int lim = my_pos - j * kPfKeys - half * HC;   // columns above lim are later keys
      uint32_t sv[32];
      auto load_chunk = [&](int c) {
        tc_ld32(my_s + c * 32, sv);
        tc_wait_ld();
        if (lim - c * 32 < 31) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i > lim - c * 32) sv[i] = __float_as_uint(-INFINITY);
        }
      };
      // pass 1: the maximum of the thread's columns
      float mx = -INFINITY;
      uint32_t first_col = 0u;               // column 0 is about to carry the exchanged maximum
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        load_chunk(c);
        if (c == 0) first_col = sv[0];
        float ma = max3(__uint_as_float(sv[0]), __uint_as_float(sv[1]), __uint_as_float(sv[2]));
        float mb = max3(__uint_as_float(sv[3]), __uint_as_float(sv[4]), __uint_as_float(sv[5]));
#pragma unroll
        for (int i = 6; i < 30; i += 4) {
          ma = max3(ma, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
          mb = max3(mb, __uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3]));
        }
        mx = max3(mx, max3(ma, __uint_as_float(sv[30]), __uint_as_float(sv[31])), mb);
      }
      if (tid == 0) PF_STAMP(0, j, 2);
      // exchange with the other half's thread: own maximum into the first column of the own half
      tc_st1(my_s, __float_as_uint(mx));
      tc_wait_st();
      tc_fence_before();
      pair_barrier(wq);
      tc_fence_after();
      const float other = __uint_as_float(tc_ld1(my_tmem + sb * kPfKeys + (half ^ 1) * HC));
      if (tid == 0) PF_STAMP(0, j, 3);
      mx = fmaxf(mx, other);
      float rescale = 1.0f;
      bool raise = false;
      if (mx > m_ref + kPfRaise || m_ref == -INFINITY) {   // (-inf + 8 = -inf: the first visible key always raises)
        if (mx != -INFINITY) {
          raise = m_ref != -INFINITY;
          rescale = exp2f(m_ref - mx);   // 0 when nothing was accumulated yet
          m_ref = mx;
        }
      }
      const float nm = m_ref == -INFINITY ? 0.f : -m_ref;
      const uint64_t nm2 = pack_f32x2(nm, nm);
      uint64_t sum2 = pack_f32x2(0.f, 0.f);
      // pass 2: P.  With two chunks the columns are read again (the registers would not hold 64 scores and 32
      // words of P with two CTAs on the SM), the upper chunk first: P will overwrite it.
      uint32_t pw[HC / 2];
#pragma unroll
      for (int cc = NCH - 1; cc >= 0; --cc) {
        if (NCH > 1) {
          load_chunk(cc);
          if (cc == 0) sv[0] = first_col;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float x0, x1;
          unpack_f32x2(add_f32x2(pack_f32x2(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])), nm2), x0, x1);
          const float e0 = exp2f(x0), e1 = exp2f(x1);
          sum2 = add_f32x2(sum2, pack_f32x2(e0, e1));
          pw[cc * 16 + (i >> 1)] = pack2<T>(e0, e1);
        }
      }
      l2 = add_f32x2(mul_f32x2(l2, pack_f32x2(rescale, rescale)), sum2);
      if (tid == 0) PF_STAMP(0, j, 4);
      bool waited = j == 0;
      auto wait_prev = [&]() {   // P . V of the previous tile has completed: O is stable
        if (!waited) {
          pf_wait(o_done + ((j - 1) & 1) * 8, ((j - 1) >> 1) & 1, a.err, dead);
          tc_fence_after();
          waited = true;
        }
      };
      if (j > 0 && __any_sync(0xffffffffu, raise)) {
        wait_prev();
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t ov[32];
          tc_ld32(o_tmem + c * 32, ov);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * rescale);
          tc_st32(o_tmem + c * 32, ov);
        }
        tc_wait_st();
      }
      if (tid == 0) PF_STAMP(0, j, 5);
      // P overwrites the upper half of the S columns this thread has read (the lower half keeps the exchanged
      // maximum); the other thread of the row has read its own columns before the exchange
      if constexpr (HC == 32) tc_st16(my_s + HC / 2, pw);
      else tc_st32(my_s + HC / 2, *reinterpret_cast<uint32_t (*)[32]>(&pw[0]));
      tc_wait_st();
      if (tid == 0) PF_STAMP(0, j, 6);
      tc_fence_before();
      mbar_arrive(p_full);
      wait_prev();   // every phase of the barrier is consumed, so that its parity stays readable
      if (tid == 0) PF_STAMP(0, j, 7);
    }

    // ---- the result: O / l; the two halves' sums meet through tensor memory as the maxima did ----
    if (tid == 0) PF_STAMP(0, 63, 4);
    pf_wait(o_done + ((ntiles - 1) & 1) * 8, ((ntiles - 1) >> 1) & 1, a.err, dead);
    tc_fence_after();
    if (tid == 0) PF_STAMP(0, 63, 5);
    float la, lb;
    unpack_f32x2(l2, la, lb);
    const float l_mine = la + lb;
    tc_st1(my_tmem + half * kPfHalf, __float_as_uint(l_mine));   // S buffer 0: no product is in flight any more
    tc_wait_st();
    tc_fence_before();
    pair_barrier(wq);
    tc_fence_after();
    const float l_other = __uint_as_float(tc_ld1(my_tmem + (half ^ 1) * kPfHalf));
    const float l_run = l_mine + l_other;
    const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
    // Through shared memory (the Q tile's space: every product that reads it has completed), so that the
    // stores to global memory are whole 256-byte rows instead of 64 bytes per thread at a row stride.
    // Staging layout: [128 rows][16 chunks of 16 B], chunk c of row r at slot c ^ (r & 15).
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
      uint32_t ov[32];
      tc_ld32(o_tmem + c * 32, ov);
      tc_wait_ld();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
          w[k] = pack2<T>(__uint_as_float(ov[i * 8 + 2 * k]) * inv, __uint_as_float(ov[i * 8 + 2 * k + 1]) * inv);
        const int ch = half * 8 + c * 4 + i;
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(qs + row * 256 + ((ch ^ (row & 15)) << 4)),
                     "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
      }
    }
    asm volatile("bar.sync 5, 256;\n" ::: "memory");
    if (!dead) {
#pragma unroll
      for (int it = 0; it < kPfRows * 16 / 256; ++it) {
        const int idx = it * 256 + tid;
        const int r = idx >> 4, ch = idx & 15;
        if (r / G < nq) {
          uint4 v;
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                       : "r"(qs + r * 256 + ((ch ^ (r & 15)) << 4)));
          *reinterpret_cast<uint4*>(O + (static_cast<size_t>(qo0 + qi0 + r / G) * Nq + kvh * G + r % G) * kPdDim + ch * 8) = v;
        }
      }
    }
    (void)my_head;
    (void)my_valid;
  }

  // everyone is done with tensor memory: hand it back
  if (tid == 0) PF_STAMP(0, 63, 6);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 9) tc_dealloc(tmem, kPfTmemCols);
  if (tid == 0) PF_STAMP(0, 63, 7);
}

}  // namespace smlm
