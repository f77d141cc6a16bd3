"""Drop-in for the reference's native module ``loquetier.ops._kernels`` on the SMLM
path, for the RMSNorm next to it and for the decode side of the paged key-value cache: the same
names with the same arguments and error behaviour (pybind registrations at
kernel_src/csrc/loquetier_ops.cc:365-373).

``install_as_loquetier_kernels()`` registers this module under that import name so
that the reference's ``from loquetier.ops import _kernels as kernel``
(src/loquetier_src/kernel_utils.py:8) resolves to it."""
from __future__ import annotations

import sys
import types

import torch

from . import ops
from .cabi import lib


def smlm_forward_cutlass_tmp_size(num_problems: int) -> int:
    """Bytes of the ``tmp`` tensor the caller must pass (60 per segment)."""
    return int(lib.smlm_b200_tmp_size(int(num_problems)))


def smlm_forward_cutlass(y: torch.Tensor, x: torch.Tensor, w_ptr: torch.Tensor, s: torch.Tensor,
                         tmp: torch.Tensor, is_row_major: bool) -> None:
    """Y[s_i:s_{i+1}] = X[s_i:s_{i+1}] . W_i for every segment i.

    Same checks as dispatch_smlm_forward_cutlass (loquetier_ops.cc:277-319): all
    tensors CUDA and contiguous, y/x 2-D, w_ptr/s/tmp 1-D, ``tmp`` exactly
    ``smlm_forward_cutlass_tmp_size(len(s) - 1)`` bytes, dtype fp16 or bf16 taken
    from ``x``.  ``tmp`` is accepted for compatibility and not used.  Unlike the
    reference (smlm_forward_cutlass.cuh:173) the call does not synchronise the
    stream."""
    for t, name, dim in ((y, "y", 2), (x, "x", 2), (w_ptr, "w_ptr", 1), (s, "s", 1), (tmp, "tmp", 1)):
        ops._chk_cuda_contig(t, name, dim)
    nseg = s.size(0) - 1
    want = smlm_forward_cutlass_tmp_size(nseg)
    if tmp.size(0) != want:
        raise RuntimeError(
            f"CHECK_EQ(tmp.size(0), static_cast<int64_t>(smlm_forward_tmp_size(num_problems))) failed. "
            f"{tmp.size(0)} vs {want}")
    if x.dtype != y.dtype or x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError(f"No suitable kernel. dtype={x.dtype}")
    if w_ptr.dtype != torch.int64 or w_ptr.numel() < nseg:
        raise RuntimeError("w_ptr must hold one int64 device address per segment")
    if y.size(0) != x.size(0):
        raise RuntimeError("y and x must have the same number of rows")
    if nseg <= 0 or x.size(0) == 0:
        return
    T = int(x.size(0))
    if 16 <= nseg <= 4096 and T <= 32 * nseg:
        # Many short segments (a decode batch): segments that share a weight pointer share an adapter.  Their
        # indices are derived on the device and a grouped plan gathers each adapter's decode tokens into one
        # piece, so that its panel is fetched once - sorted batch or not.  Nothing is read back to the host.
        ids = torch.empty(nseg, dtype=torch.int32, device=x.device)
        with torch.cuda.device(x.device):
            ops.check(lib.smlm_b200_group_ids_from_pointers(w_ptr.data_ptr(), nseg, ids.data_ptr(),
                                                            torch.cuda.current_stream(x.device).cuda_stream),
                      "smlm_b200_group_ids_from_pointers")
        plan = ops.Plan(s, T, seg_ids=ids, n_table=nseg)
        ops.gemm(y, x, w_ptr[:nseg], plan, is_row_major=bool(is_row_major), seg_ids=ids)
        return
    plan = ops.Plan(s, T)
    ops.gemm(y, x, w_ptr, plan, is_row_major=bool(is_row_major))


def rms_norm(output: torch.Tensor, rms_output: torch.Tensor, input: torch.Tensor, weight: torch.Tensor,
             epsilon: float) -> None:
    """output = input * rsqrt(mean(input^2) + epsilon) * weight per row; rms_output [rows, 1] fp32
    receives the rsqrt.  Same checks as dispatch_rms_norm (loquetier_ops.cc:326-358).  Runs on the
    current stream and does not synchronise (the reference launches on the default stream and then
    synchronises the current one, rms_norm_cutlass.cu:170-173)."""
    for t, name, dim in ((output, "output", 2), (rms_output, "rms_output", 2), (input, "input", 2),
                         (weight, "weight", 1)):
        ops._chk_cuda_contig(t, name, dim)
    if output.shape != input.shape:
        raise RuntimeError("CHECK_SHAPE(output, input) failed")
    if rms_output.size(0) != input.size(0) or rms_output.size(1) != 1:
        raise RuntimeError("CHECK_EQ(input.size(0), rms_output.size(0)) / CHECK_EQ(1, rms_output.size(1)) failed")
    if weight.size(0) != input.size(1):
        raise RuntimeError("CHECK_EQ(input.size(input.dim() - 1), weight.size(0)) failed")
    if weight.dtype != input.dtype or output.dtype != input.dtype:
        raise RuntimeError("CHECK_EQ(input.scalar_type(), weight.scalar_type()) failed")
    if rms_output.dtype != torch.float32:
        raise RuntimeError("rms_output must be float32")
    if input.dtype not in (torch.float16, torch.bfloat16) or input.size(1) % 8 != 0:
        raise RuntimeError(f"No suitable kernel. dtype={input.dtype} columns={input.size(1)}")
    if input.size(0) == 0:
        return
    ops.rms_norm(output, rms_output, input, weight, epsilon)


def _chk_kv(kv_ptrs, kv_indptr, last_page_offset, batch_size):
    for t, name in ((kv_ptrs, "kv_ptrs"), (kv_indptr, "kv_indptr"), (last_page_offset, "last_page_offset")):
        ops._chk_cuda_contig(t, name, 1)
    if kv_ptrs.dtype != torch.int64 or kv_indptr.dtype != torch.int32 or last_page_offset.dtype != torch.int32:
        raise RuntimeError("kv_ptrs must be int64, kv_indptr and last_page_offset int32")
    if kv_indptr.size(0) != batch_size + 1:
        raise RuntimeError(f"CHECK_EQ(kv_indptr.size(0), batch_size + 1) failed. {kv_indptr.size(0)} vs {batch_size + 1}")
    if last_page_offset.size(0) != batch_size:
        raise RuntimeError(f"CHECK_EQ(last_page_offset.size(0), batch_size) failed. "
                           f"{last_page_offset.size(0)} vs {batch_size}")


def _no_kernel(e, q, page_size, group_size):
    from .cabi import SmlmError
    if isinstance(e, SmlmError) and e.status in (2, 3):
        return RuntimeError(f"No suitable kernel. dtype={q.dtype} page_size={page_size} group_size={group_size} "
                            f"head_dim={q.size(2)}")
    return e


def batch_prefill(o: torch.Tensor, q: torch.Tensor, qo_indptr: torch.Tensor, kv_ptrs: torch.Tensor,
                  kv_indptr: torch.Tensor, last_page_offset: torch.Tensor, tmpbuf: torch.Tensor, num_layers: int,
                  layer_idx: int, num_kv_heads: int, base: float, page_size: int) -> None:
    """Causal prefill attention over the paged cache with the arguments and checks of the reference's
    binding (batch_prefill, loquetier_ops.cc:90-136).  ``tmpbuf`` is accepted for compatibility and not
    used (the reference wants 64 MiB of it and copies ``qo_indptr`` to the host).  Does not synchronise."""
    from . import kvcache
    for t, name in ((o, "o"), (q, "q")):
        ops._chk_cuda_contig(t, name, 3)
    ops._chk_cuda_contig(qo_indptr, "qo_indptr", 1)
    if o.shape != q.shape:
        raise RuntimeError("CHECK_SHAPE(o, q) failed")
    batch_size = int(last_page_offset.size(0)) if last_page_offset.dim() == 1 else 0
    num_qo_heads = int(o.size(1))
    group_size = num_qo_heads // max(int(num_kv_heads), 1)
    if num_qo_heads != group_size * num_kv_heads:
        raise RuntimeError(f"CHECK_EQ(num_qo_heads, group_size * num_kv_heads) failed. "
                           f"{num_qo_heads} vs {group_size * num_kv_heads}")
    _chk_kv(kv_ptrs, kv_indptr, last_page_offset, batch_size)
    if qo_indptr.dtype != torch.int32:
        raise RuntimeError("expected scalar type Int but found " + str(qo_indptr.dtype))
    if qo_indptr.size(0) != batch_size + 1:
        raise RuntimeError(f"CHECK_EQ(qo_indptr.size(0), batch_size + 1) failed. {qo_indptr.size(0)} vs {batch_size + 1}")
    if tmpbuf.numel() * tmpbuf.element_size() < 4 * (4 * batch_size + 1):
        raise RuntimeError("CHECK_GE(tmpbuf.nbytes(), sizeof(int32_t) * (4 * batch_size + 1)) failed")
    try:
        kvcache.batch_prefill_into(o, q, qo_indptr, kv_ptrs, kv_indptr, last_page_offset, num_layers, layer_idx,
                                   num_kv_heads, base, page_size)
    except RuntimeError as e:
        raise _no_kernel(e, q, page_size, group_size) from None


def batch_decode(o: torch.Tensor, q: torch.Tensor, kv_ptrs: torch.Tensor, kv_indptr: torch.Tensor,
                 last_page_offset: torch.Tensor, tmpbuf: torch.Tensor, num_layers: int, layer_idx: int,
                 num_kv_heads: int, base: float, page_size: int) -> None:
    """Decode attention over the paged cache with the arguments and checks of the reference's binding
    (batch_decode, loquetier_ops.cc:138-180).  ``tmpbuf`` is accepted for compatibility (the reference
    wants at least 64 MiB of it) and not used: its contents are undefined, whereas this kernel's
    workspace has to start zeroed, so the workspace is kept by the wrapper.  Does not synchronise."""
    from . import kvcache
    for t, name in ((o, "o"), (q, "q")):
        ops._chk_cuda_contig(t, name, 3)
    if o.shape != q.shape:
        raise RuntimeError("CHECK_SHAPE(o, q) failed")
    batch_size, num_qo_heads = int(o.size(0)), int(o.size(1))
    group_size = num_qo_heads // max(int(num_kv_heads), 1)
    if num_qo_heads != group_size * num_kv_heads:
        raise RuntimeError(f"CHECK_EQ(num_qo_heads, group_size * num_kv_heads) failed. "
                           f"{num_qo_heads} vs {group_size * num_kv_heads}")
    _chk_kv(kv_ptrs, kv_indptr, last_page_offset, batch_size)
    if tmpbuf.numel() * tmpbuf.element_size() < 4 * (4 * batch_size + 1):
        raise RuntimeError("CHECK_GE(tmpbuf.nbytes(), sizeof(int32_t) * (4 * batch_size + 1)) failed")
    try:
        kvcache.batch_decode_into(o, q, kv_ptrs, kv_indptr, last_page_offset, num_layers, layer_idx, num_kv_heads,
                                  base, page_size)
    except RuntimeError as e:
        raise _no_kernel(e, q, page_size, group_size) from None


def init_kv(kv_ptrs: torch.Tensor, kv_indptr: torch.Tensor, last_page_offset: torch.Tensor, k: torch.Tensor,
            v: torch.Tensor, seqlen_indptr: torch.Tensor, num_layers: int, layer_idx: int, num_kv_heads: int,
            page_size: int) -> None:
    """Copies a run of keys/values per request into its pages (init_kv, loquetier_ops.cc:182-228)."""
    from . import kvcache
    for t, name in ((k, "k"), (v, "v")):
        ops._chk_cuda_contig(t, name, 3)
    if k.shape != v.shape:
        raise RuntimeError("CHECK_SHAPE(k, v) failed")
    batch_size = int(last_page_offset.size(0))
    _chk_kv(kv_ptrs, kv_indptr, last_page_offset, batch_size)
    ops._chk_cuda_contig(seqlen_indptr, "seqlen_indptr", 1)
    if seqlen_indptr.size(0) != batch_size + 1:
        raise RuntimeError(f"CHECK_EQ(seqlen_indptr.size(0), batch_size + 1) failed. "
                           f"{seqlen_indptr.size(0)} vs {batch_size + 1}")
    try:
        kvcache.init_kv_raw(kv_ptrs, kv_indptr, last_page_offset, k, v, seqlen_indptr, num_layers, layer_idx,
                            num_kv_heads, page_size)
    except RuntimeError as e:
        raise _no_kernel(e, k, page_size, 1) from None


def append_kv(kv_ptrs: torch.Tensor, kv_indptr: torch.Tensor, last_page_offset: torch.Tensor, k: torch.Tensor,
              v: torch.Tensor, num_layers: int, layer_idx: int, num_kv_heads: int, page_size: int) -> None:
    """Writes one new key/value per request into its cache (append_kv, loquetier_ops.cc:230-273)."""
    from . import kvcache
    for t, name in ((k, "k"), (v, "v")):
        ops._chk_cuda_contig(t, name, 3)
    if k.shape != v.shape:
        raise RuntimeError("CHECK_SHAPE(k, v) failed")
    _chk_kv(kv_ptrs, kv_indptr, last_page_offset, int(k.size(0)))
    try:
        kvcache.append_kv_raw(kv_ptrs, kv_indptr, last_page_offset, k, v, num_layers, layer_idx, num_kv_heads,
                              page_size)
    except RuntimeError as e:
        raise _no_kernel(e, k, page_size, 1) from None


def install_as_loquetier_kernels() -> types.ModuleType:
    """Make ``import loquetier.ops._kernels`` resolve to this module.  It carries the names of the SMLM
    path, ``rms_norm`` and the paged-cache attention (``batch_prefill``, ``batch_decode``, ``init_kv``,
    ``append_kv``): every name the reference's extension module exports."""
    me = sys.modules[__name__]
    pkg = sys.modules.get("loquetier")
    if pkg is None:
        pkg = types.ModuleType("loquetier")
        pkg.__path__ = []
        sys.modules["loquetier"] = pkg
    opsmod = sys.modules.get("loquetier.ops")
    if opsmod is None:
        opsmod = types.ModuleType("loquetier.ops")
        opsmod.__path__ = []
        sys.modules["loquetier.ops"] = opsmod
        pkg.ops = opsmod
    opsmod._kernels = me
    sys.modules["loquetier.ops._kernels"] = me
    return me
