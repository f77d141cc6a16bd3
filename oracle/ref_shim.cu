// TEST INFRASTRUCTURE ONLY: a C-ABI doorway to the reference's own CUDA kernels, so that GPU tests
// can call them as a second witness next to the CPU oracle and time them next to this library's.
// Nothing in the product package links, loads or calls this.
//
// The kernels themselves are NOT here: oracle/build_ref.py compiles them from where they lie in a
// checkout of the reference (kernel_src/csrc/smlm_forward/smlm_forward_cutlass.cu and
// kernel_src/csrc/rms_norm/rms_norm_cutlass.cu), against the CUTLASS headers of this image, and
// links this file to them.  The wrappers below do what the reference's dispatchers do with the
// same arguments (kernel_src/csrc/loquetier_ops.cc:277-319 and :326-358): pick the template
// instantiation from the dtype and the layout flag, and derive the weight leading dimension.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "cutlass/layout/matrix.h"
#include "rms_norm/rms_norm.h"
#include "smlm_forward/smlm_forward.h"

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

}  // extern "C"
