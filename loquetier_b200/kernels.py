"""Drop-in for the reference's native module ``loquetier.ops._kernels`` on the SMLM
path and for the RMSNorm next to it: the same names with the same arguments and error
behaviour (pybind registrations at kernel_src/csrc/loquetier_ops.cc:371-373).

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
    plan = ops.Plan(s, x.size(0))
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


def install_as_loquetier_kernels() -> types.ModuleType:
    """Make ``import loquetier.ops._kernels`` resolve to this module (only the names of
    the SMLM path and ``rms_norm`` exist on it)."""
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
