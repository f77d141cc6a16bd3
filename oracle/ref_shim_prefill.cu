// TEST INFRASTRUCTURE ONLY: C-ABI doorway to the reference's prefill attention kernel, a template of its
// vendored flashinfer headers (third_party/flashinfer/include/flashinfer/prefill.cuh), as a second witness
// next to the CPU oracle and a timing baseline.  Nothing in the product package links, loads or calls this.
//
// This file is compiled to compute_80 PTX, which the driver translates for the GPU it finds: the
// reference's store-matrix wrapper for sm_90 and later (flashinfer/mma.cuh:96-99) declares its inputs as
// asm outputs and does not compile, so the kernel is built the way it is built for the reference's own
// sm_80 targets, where that wrapper's shuffle fallback is used.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "flashinfer/page.cuh"
#include "flashinfer/utils.cuh"
// The host compiler of this image (gcc 13) rejects `constexpr size_t GROUP_SIZE` as the uint32_t template
// argument of tensor_info_t inside the single-request dispatchers of prefill.cuh (:1101, :1223), functions
// that the batch path never calls.  The macro that declares the constant is restated with the type the
// template wants before the header is read; the kernels and the batch dispatcher do not use it.
#undef SWITCH_GQA_GROUP_SIZE
#define SWITCH_GQA_GROUP_SIZE(group_size, GROUP_SIZE, ...) \
  if (group_size == 1) {                                   \
    constexpr uint32_t GROUP_SIZE = 1;                     \
    __VA_ARGS__                                            \
  } else if (group_size == 4) {                            \
    constexpr uint32_t GROUP_SIZE = 4;                     \
    __VA_ARGS__                                            \
  } else if (group_size == 8) {                            \
    constexpr uint32_t GROUP_SIZE = 8;                     \
    __VA_ARGS__                                            \
  }
#include "flashinfer/prefill.cuh"

namespace {

using flashinfer::paged_kv_t;
using flashinfer::PageStorage;
using flashinfer::RotaryMode;

// What FlashInferBatchPrefillKernel does (flashinfer_all.cu:48-83): causal, Llama rotary mode, rope scale 1, fp32
// logits.  Page size 16, head dim 128; group sizes 1, 4 and 8.  The dispatcher copies qo_indptr to the host,
// builds its tile lists there and synchronises the stream (prefill.cuh:1427-1484).
template <typename T, uint32_t GROUP>
bool ref_prefill_one(T* o, T* q, int32_t* qo_indptr, T** kv_ptrs, int32_t* kv_indptr, int32_t* last_page_offset,
                     int32_t* aux, float* tmp, int num_layers, int layer_idx, int num_kv_heads, float rope_theta,
                     int batch_size, cudaStream_t stream) {
  paged_kv_t<PageStorage::kPointer, T, int32_t> paged_kv(num_layers, layer_idx, num_kv_heads, 16, 128, batch_size,
                                                         kv_ptrs, kv_indptr, last_page_offset, aux);
  auto status = flashinfer::BatchPrefillWithPagedKVCacheDispatched<16, GROUP, 128, PageStorage::kPointer,
                                                                   RotaryMode::kLlama, false, true>(
      q, paged_kv, qo_indptr, o, tmp, static_cast<uint32_t>(num_kv_heads * GROUP), 1.f, rope_theta, stream);
  return status == cudaSuccess;
}

template <typename T>
bool ref_prefill_t(void* o, void* q, int32_t* qo_indptr, void** kv_ptrs, int32_t* kv_indptr, int32_t* last_page_offset,
                   int32_t* aux, float* tmp, int num_layers, int layer_idx, int group, int num_kv_heads,
                   float rope_theta, int batch_size, cudaStream_t st) {
  T* oo = static_cast<T*>(o);
  T* qq = static_cast<T*>(q);
  T** pp = reinterpret_cast<T**>(kv_ptrs);
  switch (group) {
    case 1: return ref_prefill_one<T, 1>(oo, qq, qo_indptr, pp, kv_indptr, last_page_offset, aux, tmp, num_layers, layer_idx, num_kv_heads, rope_theta, batch_size, st);
    case 4: return ref_prefill_one<T, 4>(oo, qq, qo_indptr, pp, kv_indptr, last_page_offset, aux, tmp, num_layers, layer_idx, num_kv_heads, rope_theta, batch_size, st);
    case 8: return ref_prefill_one<T, 8>(oo, qq, qo_indptr, pp, kv_indptr, last_page_offset, aux, tmp, num_layers, layer_idx, num_kv_heads, rope_theta, batch_size, st);
    default: return false;
  }
}

}  // namespace

extern "C" {

// aux as for ref_batch_decode; tmp: the rest of the reference's `tmpbuf` (64 MiB there).
int ref_batch_prefill(void* o, void* q, int32_t* qo_indptr, void** kv_ptrs, int32_t* kv_indptr,
                      int32_t* last_page_offset, int32_t* aux, float* tmp, int num_layers, int layer_idx,
                      int group_size, int num_kv_heads, float rope_theta, int batch_size, int dtype, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    return ref_prefill_t<nv_half>(o, q, qo_indptr, kv_ptrs, kv_indptr, last_page_offset, aux, tmp, num_layers,
                                  layer_idx, group_size, num_kv_heads, rope_theta, batch_size, st);
  if (dtype == 1)
    return ref_prefill_t<nv_bfloat16>(o, q, qo_indptr, kv_ptrs, kv_indptr, last_page_offset, aux, tmp, num_layers,
                                      layer_idx, group_size, num_kv_heads, rope_theta, batch_size, st);
  return 0;
}

}  // extern "C"
