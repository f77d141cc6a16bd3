// TEST INFRASTRUCTURE ONLY: a C-ABI doorway to the reference's own CUDA kernels, so that GPU tests
// can call them as a second witness next to the CPU oracle and time them next to this library's.
// Nothing in the product package links, loads or calls this.
//
// The kernels themselves are NOT here: oracle/build_ref.py compiles them from where they lie in a
// checkout of the reference (kernel_src/csrc/smlm_forward/smlm_forward_cutlass.cu and
// kernel_src/csrc/rms_norm/rms_norm_cutlass.cu), against the CUTLASS headers of this image, and
// links this file to them; the attention kernels are templates of the reference's vendored
// flashinfer headers (third_party/flashinfer/include) and are instantiated from there.  The wrappers below do what the reference's dispatchers do with the
// same arguments (kernel_src/csrc/loquetier_ops.cc:277-319 and :326-358): pick the template
// instantiation from the dtype and the layout flag, and derive the weight leading dimension.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "cutlass/layout/matrix.h"
#include "flashinfer/decode.cuh"
#include "flashinfer/page.cuh"
#include "rms_norm/rms_norm.h"
#include "smlm_forward/smlm_forward.h"

namespace {

using flashinfer::paged_kv_t;
using flashinfer::PageStorage;
using flashinfer::RotaryMode;

// What FlashInferBatchDecodeKernel does for one (page size, group size, head dim) it was generated for
// (kernel_src/csrc/flashinfer_adapter/flashinfer_all.cu:85-108): paged cache with pointer storage, Llama
// rotary mode, rope scale 1, no temporary buffer (so the non-cooperative kernel runs).  The adapter's
// dispatch tables are generated at the reference's build time; here the instantiations the tests need
// are spelled out: page size 16, head dim 128, group sizes 1, 4 and 8.
template <typename T, uint32_t GROUP>
bool ref_decode_one(T* o, T* q, T** kv_ptrs, int32_t* kv_indptr, int32_t* last_page_offset, int32_t* aux,
                    int num_layers, int layer_idx, int num_kv_heads, float rope_theta, int batch_size,
                    cudaStream_t stream) {
  paged_kv_t<PageStorage::kPointer, T, int32_t> paged_kv(num_layers, layer_idx, num_kv_heads, 16, 128, batch_size,
                                                         kv_ptrs, kv_indptr, last_page_offset, aux);
  auto status = flashinfer::BatchDecodeWithPagedKVCacheDispatched<16, GROUP, 128, PageStorage::kPointer,
                                                                  RotaryMode::kLlama>(q, paged_kv, o, nullptr, 1.f,
                                                                                      rope_theta, stream);
  return status == cudaSuccess;
}

template <typename T>
bool ref_decode_t(void* o, void* q, void** kv_ptrs, int32_t* kv_indptr, int32_t* last_page_offset, int32_t* aux,
                  int num_layers, int layer_idx, int group, int num_kv_heads, float rope_theta, int batch_size,
                  cudaStream_t st) {
  T* oo = static_cast<T*>(o);
  T* qq = static_cast<T*>(q);
  T** pp = reinterpret_cast<T**>(kv_ptrs);
  switch (group) {
    case 1: return ref_decode_one<T, 1>(oo, qq, pp, kv_indptr, last_page_offset, aux, num_layers, layer_idx, num_kv_heads, rope_theta, batch_size, st);
    case 4: return ref_decode_one<T, 4>(oo, qq, pp, kv_indptr, last_page_offset, aux, num_layers, layer_idx, num_kv_heads, rope_theta, batch_size, st);
    case 8: return ref_decode_one<T, 8>(oo, qq, pp, kv_indptr, last_page_offset, aux, num_layers, layer_idx, num_kv_heads, rope_theta, batch_size, st);
    default: return false;
  }
}

// FlashInferAppendKvKernel / FlashInferInitKvKernel (flashinfer_all.cu:110-153) for head dim 128.
template <typename T>
bool ref_append_t(void** kv_ptrs, int32_t* kv_indptr, int32_t* last_page_offset, void* key, void* value,
                  int32_t* seqlen_indptr, int num_layers, int layer_idx, int num_kv_heads, int page_size,
                  int batch_size, cudaStream_t stream) {
  constexpr uint32_t head_dim = 128;
  paged_kv_t<PageStorage::kPointer, T, int32_t> paged_kv(num_layers, layer_idx, num_kv_heads, page_size, head_dim,
                                                         batch_size, reinterpret_cast<T**>(kv_ptrs), kv_indptr,
                                                         last_page_offset);
  constexpr size_t vec_size = 16 / sizeof(T) > head_dim / 32 ? 16 / sizeof(T) : head_dim / 32;
  constexpr size_t bdx = head_dim / vec_size;
  constexpr size_t bdy = 1;
  dim3 nblks(paged_kv.batch_size * paged_kv.num_heads / bdy);
  dim3 nthrs(bdx, bdy);
  if (seqlen_indptr == nullptr)
    flashinfer::AppendPagedKVCacheDecodeKernel<head_dim, vec_size, bdx, bdy, PageStorage::kPointer, T, int32_t>
        <<<nblks, nthrs, 0, stream>>>(paged_kv, static_cast<T*>(key), static_cast<T*>(value));
  else
    flashinfer::AppendPagedKVCachePrefillKernel<head_dim, vec_size, bdx, bdy, PageStorage::kPointer, T, int32_t>
        <<<nblks, nthrs, 0, stream>>>(paged_kv, static_cast<T*>(key), static_cast<T*>(value), seqlen_indptr);
  return cudaStreamSynchronize(stream) == cudaSuccess;
}

}  // namespace

extern "C" {

size_t ref_smlm_forward_tmp_size(int num_problems) { return smlm_forward_tmp_size(num_problems); }

// dtype: 0 = fp16, 1 = bf16.  Returns 1 on success (the reference's bool), 0 for "No suitable kernel."
int ref_smlm_forward(void* y, void* x, void** w, int32_t* s, void* tmp, int num_problems, int d_in, int d_out,
                     int dtype, int is_row_major, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int w_ld = is_row_major ? d_out : d_in;   // loquetier_ops.cc:297-303
  if (dtype == 0) {
    return is_row_major
               ? smlm_forward<nv_half, cutlass::layout::RowMajor>(static_cast<nv_half*>(y), static_cast<nv_half*>(x),
                                                                  reinterpret_cast<nv_half**>(w), s, tmp,
                                                                  num_problems, d_in, d_out, w_ld, st)
               : smlm_forward<nv_half, cutlass::layout::ColumnMajor>(static_cast<nv_half*>(y),
                                                                     static_cast<nv_half*>(x),
                                                                     reinterpret_cast<nv_half**>(w), s, tmp,
                                                                     num_problems, d_in, d_out, w_ld, st);
  }
  if (dtype == 1) {
    return is_row_major ? smlm_forward<nv_bfloat16, cutlass::layout::RowMajor>(
                              static_cast<nv_bfloat16*>(y), static_cast<nv_bfloat16*>(x),
                              reinterpret_cast<nv_bfloat16**>(w), s, tmp, num_problems, d_in, d_out, w_ld, st)
                        : smlm_forward<nv_bfloat16, cutlass::layout::ColumnMajor>(
                              static_cast<nv_bfloat16*>(y), static_cast<nv_bfloat16*>(x),
                              reinterpret_cast<nv_bfloat16**>(w), s, tmp, num_problems, d_in, d_out, w_ld, st);
  }
  return 0;
}

int ref_rms_norm(void* out, float* rms_out, const void* in, const void* weight, int rows, int cols, float eps,
                 int dtype, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    return rms_norm<nv_half>(static_cast<nv_half*>(out), rms_out, static_cast<const nv_half*>(in),
                             static_cast<const nv_half*>(weight), rows, cols, eps, st);
  if (dtype == 1)
    return rms_norm<nv_bfloat16>(static_cast<nv_bfloat16*>(out), rms_out, static_cast<const nv_bfloat16*>(in),
                                 static_cast<const nv_bfloat16*>(weight), rows, cols, eps, st);
  return 0;
}

// aux: 4 * (batch_size + 1) int32 of device scratch, the head of the reference's `tmpbuf`
// (flashinfer_all.cu:93).  Page size 16 and head dim 128 only; group size 1, 4 or 8.
int ref_batch_decode(void* o, void* q, void** kv_ptrs, int32_t* kv_indptr, int32_t* last_page_offset, int32_t* aux,
                     int num_layers, int layer_idx, int group_size, int num_kv_heads, float rope_theta, int batch_size,
                     int dtype, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    return ref_decode_t<nv_half>(o, q, kv_ptrs, kv_indptr, last_page_offset, aux, num_layers, layer_idx, group_size,
                                 num_kv_heads, rope_theta, batch_size, st);
  if (dtype == 1)
    return ref_decode_t<nv_bfloat16>(o, q, kv_ptrs, kv_indptr, last_page_offset, aux, num_layers, layer_idx,
                                     group_size, num_kv_heads, rope_theta, batch_size, st);
  return 0;
}

// seqlen_indptr == NULL: one token per request (append_kv); otherwise a run per request (init_kv).
int ref_append_kv(void** kv_ptrs, int32_t* kv_indptr, int32_t* last_page_offset, void* key, void* value,
                  int32_t* seqlen_indptr, int num_layers, int layer_idx, int num_kv_heads, int page_size,
                  int batch_size, int dtype, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    return ref_append_t<nv_half>(kv_ptrs, kv_indptr, last_page_offset, key, value, seqlen_indptr, num_layers,
                                 layer_idx, num_kv_heads, page_size, batch_size, st);
  if (dtype == 1)
    return ref_append_t<nv_bfloat16>(kv_ptrs, kv_indptr, last_page_offset, key, value, seqlen_indptr, num_layers,
                                     layer_idx, num_kv_heads, page_size, batch_size, st);
  return 0;
}

}  // extern "C"
