"""ctypes binding of ``oracle/_ref/libref.so``: the reference's own CUDA kernels of this path, built by
``oracle/build_ref.py``.  Test infrastructure (a GPU-side witness); the tests that use it are skipped when
the library has not been built."""
import ctypes
import os
from ctypes import c_float, c_int, c_size_t, c_void_p

import torch

LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libref.so")


def available() -> bool:
    return os.path.exists(LIB_PATH)


_lib = None


def lib():
    global _lib
    if _lib is None:
        L = ctypes.CDLL(LIB_PATH)
        L.ref_smlm_forward_tmp_size.restype = c_size_t
        L.ref_smlm_forward_tmp_size.argtypes = [c_int]
        L.ref_smlm_forward.restype = c_int
        L.ref_smlm_forward.argtypes = [c_void_p] * 5 + [c_int] * 5 + [c_void_p]
        L.ref_rms_norm.restype = c_int
        L.ref_rms_norm.argtypes = [c_void_p] * 4 + [c_int, c_int, c_float, c_int, c_void_p]
        L.ref_batch_decode.restype = c_int
        L.ref_batch_decode.argtypes = [c_void_p] * 6 + [c_int] * 4 + [c_float, c_int, c_int, c_void_p]
        L.ref_batch_prefill.restype = c_int
        L.ref_batch_prefill.argtypes = [c_void_p] * 8 + [c_int] * 4 + [c_float, c_int, c_int, c_void_p]
        L.ref_append_kv.restype = c_int
        L.ref_append_kv.argtypes = [c_void_p] * 6 + [c_int] * 6 + [c_void_p]
        _lib = L
    return _lib


def _code(t):
    return {torch.float16: 0, torch.bfloat16: 1}[t.dtype]


def smlm_forward_cutlass(y, x, w_ptr, s, is_row_major=False):
    """One call of the reference operator (kernel_src/csrc/loquetier_ops.cc:277-319) on its own kernel.
    Allocates the scratch the reference asks its caller for.  The reference synchronises the stream itself."""
    n = int(s.numel()) - 1
    tmp = torch.empty(max(1, int(lib().ref_smlm_forward_tmp_size(n))), dtype=torch.uint8, device=x.device)
    st = torch.cuda.current_stream(x.device).cuda_stream
    ok = lib().ref_smlm_forward(y.data_ptr(), x.data_ptr(), w_ptr.data_ptr(), s.data_ptr(), tmp.data_ptr(), n,
                                int(x.size(1)), int(y.size(1)), _code(x), int(bool(is_row_major)), st)
    if not ok:
        raise RuntimeError("No suitable kernel.")
    return y


def rms_norm(out, rms_out, x, w, eps):
    """The reference's RMSNorm kernel (kernel_src/csrc/rms_norm/rms_norm_cutlass.cu:158-186).  It launches on
    the default stream and then synchronises the given one, so the caller brackets it with device syncs."""
    torch.cuda.synchronize()
    st = torch.cuda.current_stream(x.device).cuda_stream
    ok = lib().ref_rms_norm(out.data_ptr(), rms_out.data_ptr(), x.data_ptr(), w.data_ptr(), int(x.size(0)),
                            int(x.size(1)), float(eps), _code(x), st)
    torch.cuda.synchronize()
    if not ok:
        raise RuntimeError("No suitable kernel.")
    return out


def batch_decode(o, q, kv_ptrs, kv_indptr, last_page_offset, num_layers, layer_idx, num_kv_heads, base):
    """The reference's decode attention (flashinfer's BatchDecodeWithPagedKVCacheKernel with the adapter's
    settings); page size 16, head dim 128, group size 1, 4 or 8."""
    B = int(q.size(0))
    aux = torch.zeros(4 * (B + 1), dtype=torch.int32, device=q.device)
    torch.cuda.synchronize()
    ok = lib().ref_batch_decode(o.data_ptr(), q.data_ptr(), kv_ptrs.data_ptr(), kv_indptr.data_ptr(),
                                last_page_offset.data_ptr(), aux.data_ptr(), int(num_layers), int(layer_idx),
                                int(q.size(1)) // int(num_kv_heads), int(num_kv_heads), float(base), B, _code(q),
                                torch.cuda.current_stream(q.device).cuda_stream)
    torch.cuda.synchronize()
    if not ok:
        raise RuntimeError("No suitable kernel.")
    return o


def batch_prefill(o, q, qo_indptr, kv_ptrs, kv_indptr, last_page_offset, num_layers, layer_idx, num_kv_heads, base):
    """The reference's prefill attention (flashinfer's BatchPrefillWithPagedKVCacheKernel with the adapter's
    settings: causal, Llama rotary mode); page size 16, head dim 128, group size 1, 4 or 8.  The dispatcher
    reads ``qo_indptr`` back to the host and synchronises."""
    B = int(last_page_offset.numel())
    aux = torch.zeros(4 * (B + 1), dtype=torch.int32, device=q.device)
    tmp = torch.zeros(1024, dtype=torch.float32, device=q.device)   # handed to the kernel, which never reads it
    torch.cuda.synchronize()
    ok = lib().ref_batch_prefill(o.data_ptr(), q.data_ptr(), qo_indptr.data_ptr(), kv_ptrs.data_ptr(),
                                 kv_indptr.data_ptr(), last_page_offset.data_ptr(), aux.data_ptr(), tmp.data_ptr(),
                                 int(num_layers), int(layer_idx), int(q.size(1)) // int(num_kv_heads),
                                 int(num_kv_heads), float(base), B, _code(q),
                                 torch.cuda.current_stream(q.device).cuda_stream)
    torch.cuda.synchronize()
    if not ok:
        raise RuntimeError("No suitable kernel.")
    return o


def append_kv(kv_ptrs, kv_indptr, last_page_offset, k, v, num_layers, layer_idx, num_kv_heads, page_size,
              seqlen_indptr=None):
    """The reference's append kernels: one token per request, or (with ``seqlen_indptr``) a run per request."""
    torch.cuda.synchronize()
    ok = lib().ref_append_kv(kv_ptrs.data_ptr(), kv_indptr.data_ptr(), last_page_offset.data_ptr(), k.data_ptr(),
                             v.data_ptr(), None if seqlen_indptr is None else seqlen_indptr.data_ptr(),
                             int(num_layers), int(layer_idx), int(num_kv_heads), int(page_size),
                             int(last_page_offset.numel()), _code(k), torch.cuda.current_stream(k.device).cuda_stream)
    torch.cuda.synchronize()
    if not ok:
        raise RuntimeError("No suitable kernel.")
