"""Host side of the SMLM path, mirroring src/loquetier_src/kernel_utils.py:
``BatchLenInfo`` (row-range bookkeeping, :11-98) and the ``add_lora`` autograd
function (:101-147) with the same call signature and return structure.

Differences that stay inside the reference's contract:
* forward plans the batch once and runs shrink and expand from that plan; no
  stream synchronisation, ``v`` is kept for the backward instead of recomputed;
* backward runs native kernels.  The reference's formulas only type-check for the
  math layout while its forward passes the PEFT layout
  (A [r, h_in], B [h_out, r]); this backward returns the gradients in the layout
  of the weights that forward used, which for the math layout are exactly the
  reference's expressions."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch
from torch.autograd.function import Function, FunctionCtx

from . import ops


class BatchLenInfo:
    """Lengths of one flattened batch whose rows are ordered
    train | eval + prefill | decode."""

    def __init__(self, trains: List[Tuple[int, ...]], prefills: List[int], decode: int,
                 evals: List[Tuple[int, ...]], indptr_device: torch.device,
                 indptr_dtype: torch.dtype = torch.int32):
        self._train_batches = trains
        self._eval_batches = evals
        self._prefills = list(prefills)
        self._decode = decode
        tl = np.asarray([int(t[0]) * int(t[1]) for t in trains], dtype=np.int64)
        if tl.size:
            self._train_partition = np.concatenate([[0], np.cumsum(tl)])
            self._tlen = self._train_partition[-1]
        else:
            self._train_partition = []
            self._tlen = 0
        if len(evals) > 0:
            el = np.asarray([int(e[0]) * int(e[1]) for e in evals], dtype=np.int64)
            self._eval_partition = np.cumsum(np.concatenate([[self._tlen], el]))
        else:
            self._eval_partition = []
        if len(prefills) > 0:
            cs = np.concatenate([[0], np.cumsum(np.asarray(prefills, dtype=np.int64))])
            self._indptr = torch.tensor(cs, dtype=indptr_dtype, device=indptr_device)
            self._doff = cs[-1] + self._tlen
        else:
            self._indptr = None
            self._doff = self._tlen

    train_batches = property(lambda self: self._train_batches)
    train_partition = property(lambda self: self._train_partition)
    eval_batches = property(lambda self: self._eval_batches)
    eval_partition = property(lambda self: self._eval_partition)
    prefills = property(lambda self: self._prefills)
    decode = property(lambda self: self._decode)
    tlen = property(lambda self: self._tlen)
    doff = property(lambda self: self._doff)
    indptr = property(lambda self: self._indptr)


def _ptr_table(tensors: Sequence[torch.Tensor], device) -> torch.Tensor:
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=device)


class add_lora(Function):
    """``add_lora.apply(y_shape, x, wa_ptr, wb_ptr, s, lora_rank, train_len,
    train_partition, *trainable)`` with ``trainable`` = (A_0, B_0, A_1, B_1, ...),
    one pair per train partition, in the PEFT layout."""

    # Set by a caller that has already planned the batch and consumed by the next forward whose ``s`` is
    # the very same tensor object.  The plan describes the CONTENTS of ``s`` at the time it was built:
    # a caller that rewrites ``s`` in place must drop the shared plan (set it to None) or build a new one.
    _shared_plan: Optional[ops.Plan] = None

    @staticmethod
    def forward(ctx: FunctionCtx, y_shape, x, wa_ptr, wb_ptr, s, lora_rank, train_len, train_partition, *args):
        # The reference splits this into forward + setup_context (kernel_utils.py:102-127); the combined
        # form is used here because the backward needs ``v``, which is not an output: it goes straight
        # into ``ctx`` instead of through any state shared between calls or threads.
        y = torch.empty(y_shape, dtype=x.dtype, device=x.device)
        v = torch.empty((x.size(0), lora_rank), dtype=x.dtype, device=x.device)
        plan = add_lora._shared_plan
        if plan is None or plan.indptr is not s or plan.T != x.size(0):
            plan = ops.Plan(s, x.size(0))
        if x.size(0) > 0 and s.numel() > 1:
            ops.fwd(y, x, v, wa_ptr, wb_ptr, plan, lora_rank, is_row_major=False)
        ctx.tp = train_partition
        ctx.rank = lora_rank
        tl = int(train_len)
        ctx.save_for_backward(x[:tl, ...], v[:tl, ...], *args)
        return y

    @staticmethod
    def backward(ctx: FunctionCtx, grad_output: torch.Tensor):
        x, v, *weight_list = ctx.saved_tensors
        tp = ctx.tp
        if len(weight_list) == 0:
            return None, None, None, None, None, None, None, None
        assert len(weight_list) % 2 == 0
        # one (A, B) pair per train partition, as the reference zips them
        npart = min(len(weight_list) // 2, len(tp) - 1)
        dev = grad_output.device
        go = grad_output.contiguous()
        grad_x = torch.zeros((go.size(0), x.size(1)), dtype=go.dtype, device=dev)
        tl = int(tp[npart])
        if tl == 0:
            return (None, grad_x, None, None, None, None, None, None,
                    *[torch.zeros_like(w) for w in weight_list])
        part = torch.tensor([int(t) for t in tp[:npart + 1]], dtype=torch.int32, device=dev)
        plan = ops.Plan(part, tl)
        was, wbs = weight_list[0:2 * npart:2], weight_list[1:2 * npart:2]
        grads = [torch.empty_like(w) for w in weight_list[:2 * npart]]
        dv = torch.empty((tl, ctx.rank), dtype=go.dtype, device=dev)
        ops.bwd(grad_x, _ptr_table(grads[::2], dev), _ptr_table(grads[1::2], dev), dv, go,
                x.contiguous(), v.contiguous(), _ptr_table(was, dev), _ptr_table(wbs, dev), plan, ctx.rank,
                is_row_major=False)
        grads += [None] * (len(weight_list) - 2 * npart)
        return None, grad_x, None, None, None, None, None, None, *grads


class rms_norm(Function):
    """RMSNorm with the call signature of the reference's autograd function
    (src/loquetier_src/kernel_utils.py:149-176): ``rms_norm.apply(x, w, eps)`` on a 2-D ``x``.
    The backward is one native pass instead of the reference's torch expressions; dW is summed in
    fp32 and returned in the weight's dtype (autograd casts the reference's fp32 sum the same way)."""

    @staticmethod
    def forward(ctx: FunctionCtx, x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6):
        from . import kernels
        m = torch.empty((x.size(0), 1), dtype=torch.float32, device=x.device)
        o = torch.empty_like(x)
        kernels.rms_norm(o, m, x, w, eps)
        ctx.save_for_backward(x, w, m)
        return o

    @staticmethod
    def backward(ctx: FunctionCtx, grad_output: torch.Tensor):
        x, w, rms_1 = ctx.saved_tensors
        go = grad_output.contiguous()
        dx = torch.empty_like(x)
        dw = torch.empty_like(w)
        if x.size(0) == 0:
            return dx, dw.zero_(), None
        ops.rms_norm_bwd(dx, dw, go, x, w, rms_1)
        return dx, dw, None


class MixedLlamaRMSNorm(torch.nn.Module):
    """The module of src/loquetier_src/models/mixed_llama.py:53-66: same constructor, parameter name
    and forward (cast to the module dtype, normalise, cast back)."""

    def __init__(self, hidden_size: int, eps: float = 1e-6, dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self.dtype = dtype
        self.weight = torch.nn.Parameter(torch.ones(hidden_size, dtype=self.dtype))
        self.variance_epsilon = eps

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        input_dtype = hidden_states.dtype
        hidden_states = hidden_states.to(self.dtype)
        return rms_norm.apply(hidden_states, self.weight, self.variance_epsilon).to(input_dtype)
