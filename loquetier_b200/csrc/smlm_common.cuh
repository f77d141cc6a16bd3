// Device-side building blocks shared by the SMLM kernels (sm_100a).
//
// Everything here is a thin wrapper over one PTX instruction or one piece of
// index arithmetic: 16-byte asynchronous copies with zero fill, ldmatrix,
// the m16n8k16 tensor-core MMA with fp32 accumulation, the shared-memory chunk
// swizzle, and conversions between fp32 and the two 16-bit storage types.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace smlm {

constexpr int kThreads = 128;       // 4 warps per CTA in every kernel
constexpr int kBM = 64;             // most rows a piece (a slice of one segment) can have
constexpr int kPlanHeaderInts = 4;  // {count, error, max_pieces, rows per piece}

// error bits a kernel may OR into the plan header's error word
constexpr int kErrBadIndptr = 1;    // indptr not monotone, negative or beyond T
constexpr int kErrBadPointer = 2;   // an adapter pointer is null or not 16-byte aligned
constexpr int kErrBadIndex = 4;     // an adapter index outside the table
constexpr int kErrTimeout = 8;      // a bounded wait on a shared-memory barrier ran out
constexpr int kErrGrouped = 16;     // a kernel that needs contiguous pieces was handed a grouped plan

constexpr int kGatherMaxLen = 8;    // segments of at most this many rows are grouped by adapter
constexpr int kGatherRows = 48;     // rows of a gather piece at most (its rows sit padded in a ring stage)
constexpr int kGatherMaxTable = 4096;  // largest adapter table a grouped plan is built for

struct __align__(16) Piece {
  int row0;   // first token row; gather piece: first entry of its rows in the plan's row index array
  int nrows;  // 1..kBM
  int seg;    // segment (or train partition) the rows belong to; gather piece: the adapter index itself
  int pad;    // 0: nrows consecutive rows of one segment; 1: gather piece, rows of short segments of one adapter
};

// Where the row index array of a grouped plan starts (ints from the start of the plan buffer): behind the
// two piece lists, whose capacities are recorded in their headers.
__device__ __forceinline__ const int* plan_row_index(const int* plan) {
  const int* tall = plan + kPlanHeaderInts + 4 * (plan[2] + 1);
  return tall + kPlanHeaderInts + 4 * (tall[2] + 1);
}

// ---------------------------------------------------------------------------
// shared-memory addressing
// ---------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// A tile is stored as rows of `C` 16-byte chunks (C a power of two).  Rows
// narrower than 128 bytes are grouped so that eight consecutive ldmatrix rows of
// one chunk column land in eight different 16-byte bank groups.
template <int C>
__device__ __forceinline__ int swz(int row, int chunk) {
  if constexpr (C >= 8) {
    return chunk ^ (row & 7);
  } else if constexpr (C == 1) {
    return chunk;
  } else {
    constexpr int rows_per_128 = 8 / C;
    return chunk ^ ((row / rows_per_128) & (C - 1));
  }
}

// ---------------------------------------------------------------------------
// global -> shared asynchronous copy, 16 bytes, zero-filled when !valid
// ---------------------------------------------------------------------------

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------
// ldmatrix / mma
// ---------------------------------------------------------------------------

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);

template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                 uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The same MMA starting from zero: D = A . B, with no accumulator registers to clear first.
template <typename T>
__device__ __forceinline__ void mma16816_z(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);

template <>
__device__ __forceinline__ void mma16816_z<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                   uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};\n"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}
template <>
__device__ __forceinline__ void mma16816_z<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};\n"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}

// ---------------------------------------------------------------------------
// conversions
// ---------------------------------------------------------------------------

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t u);
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t u) {
  return __half22float2(*reinterpret_cast<__half2*>(&u));
}
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t u) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
}

// Round to the 16-bit storage type and back: what the reference does to every
// intermediate it materialises.
template <typename T>
__device__ __forceinline__ float round_through(float a);
template <>
__device__ __forceinline__ float round_through<__half>(float a) {
  return __half2float(__float2half_rn(a));
}
template <>
__device__ __forceinline__ float round_through<__nv_bfloat16>(float a) {
  return __bfloat162float(__float2bfloat16_rn(a));
}

// ---------------------------------------------------------------------------
// adapter lookup: per-segment pointer table, or an adapter table indexed by a
// per-segment adapter id.  Records a fault instead of touching a bad address.
// ---------------------------------------------------------------------------

__device__ __forceinline__ const void* adapter_ptr(const void* const* table, const int32_t* ids, int n_table,
                                                   int seg, int* err) {
  int idx = seg;
  if (ids != nullptr) {
    idx = ids[seg];
    if (idx < 0 || idx >= n_table) {
      atomicOr(err, kErrBadIndex);
      return nullptr;
    }
  }
  const void* p = table[idx];
  if (p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) != 0) {
    atomicOr(err, kErrBadPointer);
    return nullptr;
  }
  return p;
}

__device__ __forceinline__ float adapter_scale(const float* scale, const int32_t* ids, int n_table, int seg) {
  if (scale == nullptr) return 1.0f;
  int idx = seg;
  if (ids != nullptr) {
    idx = ids[seg];
    if (idx < 0 || idx >= n_table) return 0.0f;
  }
  return scale[idx];
}

// packed pairs of fp32 (one instruction for two lanes on sm_100) and the three-input maximum
__device__ __forceinline__ uint64_t pack_f32x2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;\n" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;\n" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

// what a fused launch computes: both products, or one half alone (one reference operator call)
constexpr int kFusedBoth = 0;
constexpr int kFusedShrinkOnly = 1;
constexpr int kFusedExpandOnly = 2;

// sin and cos of pi * x on the special-function unit: x (half-turns) is reduced to [-1, 1] exactly, then the
// hardware approximations are good to about 1e-6 absolute - far below the rounding of 16-bit operands.  The
// library routine sincospif costs an order of magnitude more instructions; it stays where a value is computed
// once per kernel.
__device__ __forceinline__ void fast_sincospi(float x, float* s, float* c) {
  const float r = x - 2.0f * rintf(0.5f * x);
  *s = __sinf(3.14159265358979f * r);
  *c = __cosf(3.14159265358979f * r);
}

// ---------------------------------------------------------------------------
// mbarrier + TMA (bulk asynchronous copies).  Every CTA fetches its own tiles; no
// copy is shared between CTAs.
// ---------------------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same poll with an explicit upper bound (in nanoseconds) on the time the thread stays suspended: it
// still resumes as soon as the phase completes, but a warp that mostly waits polls that much less often
// and leaves the issue slots to the warps that compute.
__device__ __forceinline__ bool mbar_try_wait_for(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after kWaitLimit polls (each poll already suspends the
// thread for a hardware-defined interval), records kErrTimeout and lets the caller
// run to completion instead of hanging the GPU.
constexpr int kWaitLimit = 1 << 18;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err, bool& dead) {
  if (dead) return false;
  for (int i = 0; i < kWaitLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  dead = true;
  atomicOr(err, kErrTimeout);
  return false;
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}
// 2-D tiled TMA load: box at element coordinates (x = innermost, y = row)
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
      ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// untiled bulk load: 16-byte aligned addresses, size a multiple of 16
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const void* tmap, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];\n"
               ::"l"(tmap), "r"(x), "r"(y), "r"(src)
               : "memory");
}
template <typename T>
__device__ __forceinline__ void tma_reduce_add_2d(const void* tmap, int x, int y, uint32_t src);
template <>
__device__ __forceinline__ void tma_reduce_add_2d<__half>(const void* tmap, int x, int y, uint32_t src) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%1, %2}], [%3];\n"
               ::"l"(tmap), "r"(x), "r"(y), "r"(src)
               : "memory");
}
template <>
__device__ __forceinline__ void tma_reduce_add_2d<__nv_bfloat16>(const void* tmap, int x, int y, uint32_t src) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%1, %2}], [%3];\n"
               ::"l"(tmap), "r"(x), "r"(y), "r"(src)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;\n" ::"n"(N) : "memory");
}
// Programmatic dependent launch: a kernel launched with the programmatic-serialization
// attribute may start while its predecessor in the stream is still running.  pdl_wait()
// blocks until the predecessor has completed and its writes are visible; pdl_trigger()
// tells the scheduler that the successor may be started now.  Without the launch
// attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

__device__ __forceinline__ void stsm_x4(uint32_t addr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1,%2,%3,%4};\n"
               ::"r"(addr), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
               : "memory");
}

}  // namespace smlm
