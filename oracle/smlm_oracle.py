"""CPU oracle for the Segmented Multi-LoRA Multiplication (SMLM) path.

TEST INFRASTRUCTURE ONLY.  This module is the checker the CUDA path is compared
against; nothing in the product package imports it.  Only tests, the smoke check
and the CPU-baseline leg of the benchmark may call it.

It restates, per segment and in fp32 on the host, what the reference computes:

* ``smlm_gemm``           - one reference ``smlm_forward_cutlass`` call
                            (kernel_src/csrc/smlm_forward/smlm_forward_cutlass.cuh:31-46
                            for the segment -> row-range / weight-pointer mapping,
                            :107,:140,:152 for fp32 accumulation with alpha=1, beta=0,
                            kernel_src/csrc/loquetier_ops.cc:294-303 for the weight
                            leading dimension of the two layouts).
* ``add_lora_forward``    - src/loquetier_src/kernel_utils.py:102-120 (shrink into a
                            16-bit ``v``, then expand).
* ``add_lora_backward``   - src/loquetier_src/kernel_utils.py:129-147.  The formulas
                            there are written for the math layout A[h_in,r], B[r,h_out]
                            (``is_row_major=True``); for the PEFT layout A[r,h_in],
                            B[h_out,r] that the released forward uses, the same
                            gradients are the transposed statement
                            dV = gO.B, dX = dV.A, dA = dV^T.X, dB = gO^T.(X.A^T).
* ``lora_linear_forward`` - src/loquetier_src/models/mixed_lora.py:173-218 (base
                            linear, per-token scale in the module dtype, add).
* ``BatchLenInfoOracle``  - src/loquetier_src/kernel_utils.py:11-53.
* ``order_requests`` / ``merge_segments``
                          - src/loquetier_src/model_generation.py:176-226 (row order)
                            and :267-283 (run-length merge into segments).

Parity pin: the reference ships no golden vectors for this path, so the oracle is
pinned against outputs of the reference's own Python code (``MixedLoraLinear``,
``add_lora``, ``BatchLenInfo``, the segment merge) executed with its native module
stubbed per segment; ``oracle/make_golden.py`` generates those vectors and
``tests/test_oracle_golden.py`` checks this file against them.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch


# ----------------------------------------------------------------------------
# arithmetic
# ----------------------------------------------------------------------------

def _as_math(w: torch.Tensor, is_row_major: bool) -> torch.Tensor:
    """Return the weight as a [d_in, d_out] fp32 matrix.

    ``is_row_major=True`` stores W as [d_in, d_out]; ``False`` (what the released
    forward passes, kernel_utils.py:118-119) stores it column-major, i.e. the
    tensor is [d_out, d_in] with d_in contiguous."""
    w32 = w.to(torch.float32)
    return w32 if is_row_major else w32.t()


def smlm_gemm(
    y: torch.Tensor,
    x: torch.Tensor,
    weights: Sequence[torch.Tensor],
    s: Sequence[int],
    is_row_major: bool = False,
) -> torch.Tensor:
    """Y[s_i:s_{i+1}] = X[s_i:s_{i+1}] . W_i, fp32 accumulate, rounded to y.dtype.

    Rows of ``y`` outside [s[0], s[-1]) are left untouched; zero-length segments
    are legal (smlm_forward_cutlass.cuh:37-45)."""
    s = [int(v) for v in s]
    assert len(weights) == len(s) - 1
    x32 = x.to(torch.float32)
    for i, w in enumerate(weights):
        a, b = s[i], s[i + 1]
        if b <= a:
            continue
        y[a:b] = (x32[a:b] @ _as_math(w, is_row_major)).to(y.dtype)
    return y


def add_lora_forward(
    y_shape: Tuple[int, int],
    x: torch.Tensor,
    wa: Sequence[torch.Tensor],
    wb: Sequence[torch.Tensor],
    s: Sequence[int],
    rank: int,
    is_row_major: bool = False,
    round_v: bool = True,
    fill: float = 0.0,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Shrink then expand (kernel_utils.py:114-120).  Returns (y, v).

    ``round_v`` keeps the intermediate in the input dtype like the reference does
    (kernel_utils.py:117); with ``round_v=False`` it stays fp32, which is the
    "ideal" answer used to report how much that rounding costs.  The reference
    allocates y with ``torch.empty``; rows no segment covers are undefined there
    and hold ``fill`` here."""
    T = x.shape[0]
    vdt = x.dtype if round_v else torch.float32
    v = torch.zeros((T, rank), dtype=vdt)
    smlm_gemm(v, x, wa, s, is_row_major)
    y = torch.full(tuple(y_shape), fill, dtype=x.dtype)
    smlm_gemm(y, v, wb, s, is_row_major)
    return y, v


def add_lora_backward(
    grad_out: torch.Tensor,
    x: torch.Tensor,
    wa: Sequence[torch.Tensor],
    wb: Sequence[torch.Tensor],
    train_partition: Sequence[int],
    is_row_major: bool = False,
    round_mid: bool = True,
):
    """Gradients of add_lora for the train partitions (kernel_utils.py:136-147).

    Returns (grad_x [T, h_in] with zeros outside the train rows, [dA_0, dB_0, ...]).
    ``round_mid`` rounds the two rank-r intermediates (dV and the recomputed V) to
    the input dtype as the reference's chain of 16-bit matmuls does."""
    tp = [int(v) for v in train_partition]
    dt = grad_out.dtype
    mid_dt = dt if round_mid else torch.float32
    h_in = x.shape[1]
    grad_x = torch.zeros((grad_out.shape[0], h_in), dtype=dt)
    grads: List[torch.Tensor] = []
    for pi in range(len(tp) - 1):
        a, b = tp[pi], tp[pi + 1]
        A = _as_math(wa[pi], is_row_major)          # [h_in, r]
        B = _as_math(wb[pi], is_row_major)          # [r, h_out]
        go = grad_out[a:b].to(torch.float32)
        xs = x[a:b].to(torch.float32)
        dv = (go @ B.t()).to(mid_dt).to(torch.float32)      # "mid"
        v = (xs @ A).to(mid_dt).to(torch.float32)           # recomputed x.A
        grad_x[a:b] = (dv @ A.t()).to(dt)
        dA_math = xs.t() @ dv                               # [h_in, r]
        dB_math = v.t() @ go                                # [r, h_out]
        if is_row_major:
            grads += [dA_math.to(dt), dB_math.to(dt)]
        else:
            grads += [dA_math.t().contiguous().to(dt), dB_math.t().contiguous().to(dt)]
    return grad_x, grads


def lora_linear_forward(
    x: torch.Tensor,
    w_base: torch.Tensor,
    wa_all: Sequence[torch.Tensor],
    wb_all: Sequence[torch.Tensor],
    scaling: Optional[Sequence[float]],
    lora_ids: Sequence[int],
    lora_len: Sequence[int],
    rank: int,
    dtype: torch.dtype,
) -> torch.Tensor:
    """MixedLoraLinear.forward without dropout (mixed_lora.py:173-218).

    ``scaling=None`` is the pre-scaled (``is_scaled``) branch."""
    result = torch.nn.functional.linear(x, w_base)
    seg = np.concatenate([[0], np.cumsum(np.asarray(lora_len, dtype=np.int64))])
    xs = x.to(dtype)
    y, _ = add_lora_forward(
        result.shape, xs, [wa_all[i] for i in lora_ids], [wb_all[i] for i in lora_ids],
        seg, rank, is_row_major=False, round_v=True)
    if scaling is not None:
        sc = torch.tensor([scaling[i] for i in lora_ids], dtype=dtype)
        per_tok = torch.repeat_interleave(sc, torch.as_tensor(list(lora_len), dtype=torch.long))
        y = y * per_tok.unsqueeze(-1)
    return (result + y).to(result.dtype)


# ----------------------------------------------------------------------------
# bookkeeping (integer, bit-exact)
# ----------------------------------------------------------------------------

class BatchLenInfoOracle:
    """Row-range bookkeeping of one flattened batch (kernel_utils.py:11-53).

    Row order is train | eval+prefill | decode."""

    def __init__(self, trains, prefills, decode, evals):
        tl = [int(b) * int(l) for b, l in trains]
        self.train_partition = [0]
        for n in tl:
            self.train_partition.append(self.train_partition[-1] + n)
        if not tl:
            self.train_partition = []
        self.tlen = sum(tl)
        self.eval_partition = []
        if len(evals) > 0:
            acc = self.tlen
            self.eval_partition = [acc]
            for b, l in evals:
                acc += int(b) * int(l)
                self.eval_partition.append(acc)
        self.prefills = list(prefills)
        self.decode = decode
        if len(prefills) > 0:
            ind = [0]
            for n in prefills:
                ind.append(ind[-1] + int(n))
            self.indptr = ind
            self.doff = ind[-1] + self.tlen
        else:
            self.indptr = None
            self.doff = self.tlen


def order_requests(trains, evals, prefills, decodes):
    """Batch row order of one step (model_generation.py:186-205).

    Every argument is a list of (lora_id, n_tokens) in arrival order.  Decode
    requests are stably sorted by adapter, prefill requests likewise, eval
    requests go before the prefill ones, train requests before everything."""
    dec = sorted(decodes, key=lambda r: r[0])
    pre = list(evals) + sorted(prefills, key=lambda r: r[0])
    return list(trains) + pre + dec


def merge_segments(ordered):
    """Run-length merge of equal adjacent adapter ids (model_generation.py:267-273).

    Returns (lora_ids, lora_lens, segment) with segment = [0] + cumsum(lora_lens)."""
    if not ordered:
        return [], [], [0]
    ids, lens = [ordered[0][0]], [0]
    for lid, n in ordered:
        if ids[-1] == lid:
            lens[-1] += int(n)
        else:
            ids.append(lid)
            lens.append(int(n))
    seg = [0]
    for n in lens:
        seg.append(seg[-1] + n)
    return ids, lens, seg


def smlm_tmp_size(num_problems: int) -> int:
    """Scratch bytes the reference asks its caller for: three pointer arrays, three
    int64 leading-dimension arrays and one 3-int problem size per segment
    (smlm_forward_cutlass.cuh:48-52)."""
    return (3 * 8 + 3 * 8 + 12) * int(num_problems)


# ----------------------------------------------------------------------------
# RMSNorm (the caller on either side of the projections)
# ----------------------------------------------------------------------------

def rms_norm_forward(x: torch.Tensor, w: torch.Tensor, eps: float):
    """Restates rmsnorm_twoPassAlgo_e8 (kernel_src/csrc/rms_norm/rms_norm_cutlass.cu:80-156): the sum
    of squares and ``s = rsqrt(sum / n + eps)`` in fp32 (:100-117), then every element as
    ``T(float(x) * s * float(w))`` (:141-155).  Returns (out in x's dtype, s as fp32 [rows, 1])."""
    x32 = x.to(torch.float32)
    s = torch.rsqrt((x32 * x32).sum(dim=1, keepdim=True) / x.size(1) + eps)
    out = (x32 * s * w.to(torch.float32)).to(x.dtype)
    return out, s


def rms_norm_backward(go: torch.Tensor, x: torch.Tensor, w: torch.Tensor, rms_1: torch.Tensor):
    """The formulas of rms_norm.backward (src/loquetier_src/kernel_utils.py:166-176) evaluated in fp32
    from the stored 16-bit operands: dW = sum_rows(x * rms * gO); dX = (gO * w - x * dot * rms^2 / n) * rms
    with dot = sum_cols(gO * w * x).  Returns (dx, dw) in fp32."""
    g32, x32, w32 = go.to(torch.float32), x.to(torch.float32), w.to(torch.float32)
    dw = (x32 * rms_1 * g32).sum(dim=0)
    dxh = g32 * w32
    dot = (dxh * x32).sum(dim=1, keepdim=True)
    dx = (dxh - (x32 * dot * rms_1 ** 2) / x.size(1)) * rms_1
    return dx, dw


# ----------------------------------------------------------------------------
# seeded synthetic workloads shared by tests and the benchmark's CPU leg
# ----------------------------------------------------------------------------

def make_case(seed, lens, ids, n_adapters, h_in, h_out, rank, dtype,
              is_row_major=False, a_std=None, b_std=0.02):
    """x ~ N(0,1), A ~ N(0, 1/sqrt(h_in)), B ~ N(0, 0.02), gO ~ N(0,1); generated in
    fp32 and rounded to ``dtype``."""
    g = torch.Generator().manual_seed(int(seed))
    T = int(sum(lens))
    a_std = (1.0 / float(np.sqrt(h_in))) if a_std is None else a_std
    x = torch.randn((T, h_in), generator=g).to(dtype)
    if is_row_major:
        wa = [(torch.randn((h_in, rank), generator=g) * a_std).to(dtype) for _ in range(n_adapters)]
        wb = [(torch.randn((rank, h_out), generator=g) * b_std).to(dtype) for _ in range(n_adapters)]
    else:
        wa = [(torch.randn((rank, h_in), generator=g) * a_std).to(dtype) for _ in range(n_adapters)]
        wb = [(torch.randn((h_out, rank), generator=g) * b_std).to(dtype) for _ in range(n_adapters)]
    go = torch.randn((T, h_out), generator=g).to(dtype)
    seg = [0]
    for n in lens:
        seg.append(seg[-1] + int(n))
    return dict(x=x, wa=wa, wb=wb, go=go, seg=seg, ids=list(ids), lens=list(lens),
                h_in=h_in, h_out=h_out, rank=rank, dtype=dtype, is_row_major=is_row_major)
