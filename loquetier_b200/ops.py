"""Torch-facing wrappers of the C ABI: they only translate tensors into pointers,
sizes and the current CUDA stream.  Device memory (outputs, the plan buffer) is
allocated by torch; the library itself never allocates and never synchronises."""
from __future__ import annotations

from typing import Optional

import torch

from . import cabi
from .cabi import check, lib

_DT = {torch.float16: cabi.SMLM_F16, torch.bfloat16: cabi.SMLM_BF16}


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        # same wording as the reference's dispatcher (loquetier_ops.cc:318)
        raise RuntimeError(f"No suitable kernel. dtype={t.dtype}") from None


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _chk_cuda_contig(t: torch.Tensor, name: str, dim: int):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if t.dim() != dim:
        raise RuntimeError(f"{name} must be a {dim}D tensor")


class Plan:
    """Work list of one batch: built on the device from the segment index pointer,
    shared by every SMLM call of the batch (all projections, shrink and expand)."""

    __slots__ = ("buf", "indptr", "nseg", "T", "seg_ids", "n_table", "nbytes")

    def __init__(self, indptr: torch.Tensor, T: int, seg_ids: Optional[torch.Tensor] = None, n_table: int = 0,
                 launch: bool = True):
        """``seg_ids`` (int32 per segment) and ``n_table`` make it a grouped plan: short segments
        (decode tokens) are grouped by adapter for the forward calls that pass the same ``seg_ids``
        and an adapter table of ``n_table`` entries.  Weight gradients need a plan without them.
        ``launch=False`` only allocates the buffer (for ``plan_pair``)."""
        _chk_cuda_contig(indptr, "s", 1)
        if indptr.dtype != torch.int32:
            raise RuntimeError("s must be int32")
        self.indptr = indptr
        self.nseg = int(indptr.numel()) - 1
        self.T = int(T)
        self.seg_ids = seg_ids
        self.n_table = int(n_table) if seg_ids is not None else 0
        if seg_ids is not None:
            _chk_cuda_contig(seg_ids, "seg_ids", 1)
            if seg_ids.dtype != torch.int32 or seg_ids.numel() < self.nseg:
                raise RuntimeError("seg_ids must hold one int32 adapter index per segment")
        nbytes = lib.smlm_b200_plan_bytes(self.T, max(self.nseg, 0))
        self.buf = torch.empty((nbytes + 3) // 4, dtype=torch.int32, device=indptr.device)
        self.nbytes = nbytes
        if not launch:
            return
        with torch.cuda.device(indptr.device):
            check(lib.smlm_b200_plan_grouped(self.buf.data_ptr(), nbytes, indptr.data_ptr(), _p(seg_ids), self.nseg,
                                             self.n_table, self.T, _stream(indptr)), "smlm_b200_plan")

    def status(self):
        """Synchronises.  Returns (n_pieces, status code)."""
        import ctypes
        n = ctypes.c_int(0)
        with torch.cuda.device(self.buf.device):
            rc = lib.smlm_b200_plan_status(self.buf.data_ptr(), ctypes.byref(n), _stream(self.buf))
        return n.value, rc

    def raise_if_failed(self):
        _, rc = self.status()
        check(rc, "smlm plan")


def plan_pair(indptr_a: torch.Tensor, T_a: int, indptr_b: torch.Tensor, T_b: int,
              seg_ids_a: Optional[torch.Tensor] = None, n_table_a: int = 0):
    """The two plans of a step - all segments (grouped when ``seg_ids_a`` is given) and the train
    partitions - built by one launch.  Returns (plan_a, plan_b)."""
    a = Plan(indptr_a, T_a, seg_ids=seg_ids_a, n_table=n_table_a, launch=False)
    b = Plan(indptr_b, T_b, launch=False)
    with torch.cuda.device(indptr_a.device):
        check(lib.smlm_b200_plan_pair(a.buf.data_ptr(), a.nbytes, indptr_a.data_ptr(), _p(seg_ids_a), a.nseg,
                                      a.n_table, a.T, b.buf.data_ptr(), b.nbytes, indptr_b.data_ptr(), b.nseg, b.T,
                                      _stream(indptr_a)), "smlm_b200_plan_pair")
    return a, b


def set_tensor_core_mode(mode: int) -> int:
    """Kernel choice for ranks above 32: 0 by shape (default), 1 the tcgen05 kernel wherever it
    applies, -1 never.  Returns the previous mode."""
    return int(lib.smlm_b200_set_tensor_core_mode(int(mode)))


def set_cluster_split(split: int) -> int:
    """Measurement knob of the mma.sync fused kernel: 0 lets the library choose how many CTAs share a
    piece, 1..4 forces it.  Returns the previous setting."""
    return int(lib.smlm_b200_set_cluster_split(int(split)))


def gemm(y, x, w_table, plan: Plan, is_row_major=False, seg_ids=None, seg_scale=None, accumulate=False):
    """One segmented GEMM (one reference operator call)."""
    with torch.cuda.device(x.device):
        check(lib.smlm_b200_gemm(y.data_ptr(), x.data_ptr(), w_table.data_ptr(), _p(seg_ids), _p(seg_scale),
                                 plan.buf.data_ptr(), int(w_table.numel()), int(x.size(0)), plan.nseg,
                                 int(x.size(1)), int(y.size(1)), _dtype_code(x), int(bool(is_row_major)),
                                 int(bool(accumulate)), int(plan.n_table > 0), _stream(x)), "smlm_b200_gemm")
    return y


def fwd(y, x, v, wa_table, wb_table, plan: Plan, rank: int, is_row_major=False, seg_ids=None, seg_scale=None,
        accumulate=False, independent=False):
    """Fused shrink + expand (+ scale, + accumulate into y); writes v [T, rank].

    ``independent=True`` is a promise about every kernel enqueued on the stream since, and including,
    the most recent launch with ``independent=False``: this call neither reads nor writes anything
    those kernels write, and writes nothing they read.  The launch then does not wait at its start
    and may run alongside all of them (its read phase overlaps their write phases); it still
    completes after them.  A call that consumes the output of an earlier launch must therefore pass
    ``independent=False`` even when unrelated independent launches sit between the two."""
    with torch.cuda.device(x.device):
        check(lib.smlm_b200_fwd(y.data_ptr(), x.data_ptr(), v.data_ptr(), wa_table.data_ptr(),
                                wb_table.data_ptr(), _p(seg_ids), _p(seg_scale), plan.buf.data_ptr(),
                                int(wa_table.numel()), int(x.size(0)), plan.nseg, int(x.size(1)),
                                int(y.size(1)), int(rank), _dtype_code(x), int(bool(is_row_major)),
                                int(bool(accumulate)), int(bool(independent)), int(plan.n_table > 0), _stream(x)),
              "smlm_b200_fwd")
    return y


def bwd_dx(dx, dv, go, wa_table, wb_table, plan: Plan, rank: int, is_row_major=False, part_ids=None,
           part_scale=None, independent=False):
    """dV = scale * gO . B and dX = dV . A over the train partitions of ``plan``."""
    with torch.cuda.device(go.device):
        check(lib.smlm_b200_bwd_dx(dx.data_ptr(), dv.data_ptr(), go.data_ptr(), wa_table.data_ptr(),
                                   wb_table.data_ptr(), _p(part_ids), _p(part_scale), plan.buf.data_ptr(),
                                   int(wa_table.numel()), plan.T, plan.nseg, int(dx.size(1)), int(go.size(1)),
                                   int(rank), _dtype_code(go), int(bool(is_row_major)), int(bool(independent)),
                                   int(plan.n_table > 0), _stream(go)), "smlm_b200_bwd_dx")
    return dx


_WORKSPACES = {}


_WS_SHAPE = {}   # (device, slot) -> the shape the cached workspace was last handed out for


def _cached_workspace(device, slot, need: int, shape, ticket_bytes: int) -> torch.Tensor:
    """One buffer per (device, slot), grown on demand and zero-filled when (re)allocated.  The kernels leave
    the tickets at its head zeroed, but a different shape moves the boundary between tickets and parked sums,
    so the head is cleared again (a few KB, on the current stream) whenever the shape differs from the one the
    buffer was last handed out for."""
    key = (device, slot)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    elif _WS_SHAPE.get(key) != shape and ticket_bytes > 0:
        with torch.cuda.device(device):
            ws[:ticket_bytes].zero_()
    _WS_SHAPE[key] = shape
    return ws


def wgrad_workspace(device, T: int, npart: int, rank: int, h0: int, h1: int = 0, slot: int = 0) -> torch.Tensor:
    """Scratch of the weight-gradient kernels with its tickets zeroed, cached per device and ``slot``.  Ask for
    it right before the launch that uses it (on the stream of that launch); calls that may overlap on different
    streams need workspaces of their own: different slots."""
    shape = (int(T), int(npart), int(rank), int(h0), int(h1))
    need = int(lib.smlm_b200_wgrad_workspace_bytes(*shape))
    return _cached_workspace(device, slot, need, shape, int(lib.smlm_b200_wgrad_ticket_bytes(*shape)))


def wgrad(g_table, p, q, part_indptr, plan: Plan, transposed: bool, part_scale=None, accumulate=False,
          grad_fp32=False, workspace=None):
    ws = workspace if workspace is not None else wgrad_workspace(p.device, plan.T, plan.nseg, p.size(1), q.size(1))
    with torch.cuda.device(p.device):
        check(lib.smlm_b200_wgrad(g_table.data_ptr(), p.data_ptr(), q.data_ptr(), part_indptr.data_ptr(),
                                  _p(part_scale), plan.buf.data_ptr(), ws.data_ptr(), ws.numel(),
                                  int(part_indptr.numel()) - 1, plan.T, int(p.size(1)), int(q.size(1)),
                                  _dtype_code(p), int(bool(transposed)), int(bool(accumulate)),
                                  int(bool(grad_fp32)), _stream(p)), "smlm_b200_wgrad")


def wgrad_pair(dA_table, dB_table, dv, x, v, go, part_indptr, plan: Plan, rank: int, is_row_major=False,
               part_ids=None, part_scale=None, n_table=0, accumulate=False, grad_fp32=False, workspace=None,
               independent=False):
    """dA and dB of every train partition in one launch.  ``independent=True``: the promise of
    ``fwd``, and in addition the call shares its ``workspace`` with none of those kernels."""
    ws = workspace if workspace is not None else wgrad_workspace(go.device, plan.T, plan.nseg, rank, go.size(1),
                                                                 x.size(1))
    with torch.cuda.device(go.device):
        check(lib.smlm_b200_wgrad_pair(dA_table.data_ptr(), dB_table.data_ptr(), dv.data_ptr(), x.data_ptr(),
                                       v.data_ptr(), go.data_ptr(), part_indptr.data_ptr(), _p(part_ids),
                                       _p(part_scale), plan.buf.data_ptr(), ws.data_ptr(), ws.numel(), int(n_table),
                                       int(part_indptr.numel()) - 1, plan.T, int(x.size(1)), int(go.size(1)),
                                       int(rank), _dtype_code(go), int(bool(is_row_major)), int(bool(accumulate)),
                                       int(bool(grad_fp32)), int(bool(independent)), _stream(go)),
              "smlm_b200_wgrad_pair")


def bwd(dx, dA_table, dB_table, dv, go, x, v, wa_table, wb_table, plan: Plan, rank: int, is_row_major=False,
        part_ids=None, part_scale=None, accumulate_grads=False, grad_fp32=False, workspace=None):
    """Backward over the train partitions ``plan.indptr``; rows = go.size(0)."""
    ws = workspace if workspace is not None else wgrad_workspace(go.device, plan.T, plan.nseg, rank, go.size(1),
                                                                 x.size(1))
    with torch.cuda.device(go.device):
        check(lib.smlm_b200_bwd(dx.data_ptr(), dA_table.data_ptr(), dB_table.data_ptr(), dv.data_ptr(),
                                go.data_ptr(), x.data_ptr(), v.data_ptr(), wa_table.data_ptr(),
                                wb_table.data_ptr(), _p(part_ids), _p(part_scale), plan.indptr.data_ptr(),
                                plan.buf.data_ptr(), ws.data_ptr(), ws.numel(), int(wa_table.numel()), plan.T,
                                plan.nseg, int(x.size(1)), int(go.size(1)), int(rank), _dtype_code(go),
                                int(bool(is_row_major)), int(bool(accumulate_grads)), int(bool(grad_fp32)),
                                _stream(go)), "smlm_b200_bwd")


# ---------------------------------------------------------------------------
# several projections per launch
# ---------------------------------------------------------------------------

class ProjSet:
    """Host-side descriptor array (``smlm_b200_proj``) of up to ``cabi.SMLM_MAX_PROJ`` projections that share a
    batch: the same segment plan, adapter ids, rank and scales, different tensors.  ``projs`` is a list of
    dicts with the tensors the entry points to be called need: ``x, y, v, wa, wb`` for the forward;
    ``go, dx, dv, wa, wb`` for dV/dX; ``dv, x, v, go, dA_t, dB_t`` for the weight gradients (``wa``/``wb``/
    ``dA_t``/``dB_t`` are int64 pointer tables on the device).  The set keeps the tensors alive."""

    def __init__(self, projs):
        import ctypes
        n = len(projs)
        if not 1 <= n <= cabi.SMLM_MAX_PROJ:
            raise RuntimeError(f"a projection set holds 1..{cabi.SMLM_MAX_PROJ} projections")
        self.keep = list(projs)
        self.n = n
        self.arr = (cabi.SmlmProj * n)()
        ref = None
        for i, p in enumerate(projs):
            d = self.arr[i]
            for f, k in (("x", "x"), ("y", "y"), ("v", "v"), ("go", "go"), ("dx", "dx"), ("dv", "dv"),
                         ("wa_table", "wa"), ("wb_table", "wb"), ("dA_table", "dA_t"), ("dB_table", "dB_t")):
                t = p.get(k)
                if t is not None:
                    if not t.is_cuda or not t.is_contiguous():
                        raise RuntimeError(f"{k} must be a contiguous CUDA tensor")
                    setattr(d, f, t.data_ptr())
                    ref = ref if ref is not None else t
            if "h_in" in p:
                d.h_in, d.h_out = int(p["h_in"]), int(p["h_out"])
            else:
                d.h_in = int((p["x"] if p.get("x") is not None else p["dx"]).size(1))
                d.h_out = int((p["y"] if p.get("y") is not None else p["go"]).size(1))
        self.ref = ref
        self.ptr = ctypes.cast(self.arr, ctypes.c_void_p)

    def _dt(self, key):
        return _dtype_code(self.keep[0][key])


def fwd_multi(ps: ProjSet, plan: Plan, rank: int, is_row_major=False, seg_ids=None, seg_scale=None,
              accumulate=False, independent=False):
    """``fwd`` for every projection of the set in one launch."""
    with torch.cuda.device(ps.ref.device):
        check(lib.smlm_b200_fwd_multi(ps.ptr, ps.n, _p(seg_ids), _p(seg_scale), plan.buf.data_ptr(),
                                      int(ps.keep[0]["wa"].numel()), plan.T, plan.nseg, int(rank), ps._dt("x"),
                                      int(bool(is_row_major)), int(bool(accumulate)), int(bool(independent)),
                                      int(plan.n_table > 0), _stream(ps.ref)), "smlm_b200_fwd_multi")


def bwd_dx_multi(ps: ProjSet, plan: Plan, rank: int, is_row_major=False, part_ids=None, part_scale=None,
                 independent=False):
    """``bwd_dx`` for every projection of the set in one launch."""
    with torch.cuda.device(ps.ref.device):
        check(lib.smlm_b200_bwd_dx_multi(ps.ptr, ps.n, _p(part_ids), _p(part_scale), plan.buf.data_ptr(),
                                         int(ps.keep[0]["wa"].numel()), plan.T, plan.nseg, int(rank), ps._dt("go"),
                                         int(bool(is_row_major)), int(bool(independent)), _stream(ps.ref)),
              "smlm_b200_bwd_dx_multi")


def wgrad_multi_workspace(ps: ProjSet, T: int, npart: int, rank: int, slot: str = "multi", which: int = 3) -> torch.Tensor:
    """Workspace of ``wgrad_pair_multi`` for this set with its tickets zeroed, cached per device and slot (see
    ``wgrad_workspace``); ``which`` is the kinds the launch will select."""
    need = int(lib.smlm_b200_wgrad_multi_workspace_bytes(ps.ptr, ps.n, int(T), int(npart), int(rank)))
    tickets = int(lib.smlm_b200_wgrad_multi_ticket_bytes(ps.ptr, ps.n, int(T), int(npart), int(rank)))
    shape = (int(T), int(npart), int(rank), tuple((int(ps.arr[i].h_in), int(ps.arr[i].h_out)) for i in range(ps.n)),
             int(which))
    return _cached_workspace(ps.ref.device, slot, need, shape, tickets)


WGRAD_DB, WGRAD_DA = 1, 2


def wgrad_pair_multi(ps: ProjSet, part_indptr, plan: Plan, rank: int, is_row_major=False, part_ids=None,
                     part_scale=None, n_table=0, accumulate=False, grad_fp32=False, workspace=None,
                     independent=False, which=WGRAD_DB | WGRAD_DA):
    """``wgrad_pair`` for every projection of the set in one launch; ``which`` restricts it to dB (reads v, go)
    or dA (reads dv, x)."""
    ws = workspace if workspace is not None else wgrad_multi_workspace(ps, plan.T, plan.nseg, rank, which=which)
    with torch.cuda.device(ps.ref.device):
        check(lib.smlm_b200_wgrad_select_multi(ps.ptr, ps.n, int(which), part_indptr.data_ptr(), _p(part_ids),
                                               _p(part_scale), plan.buf.data_ptr(), ws.data_ptr(), ws.numel(),
                                               int(n_table), int(part_indptr.numel()) - 1, plan.T, int(rank),
                                               ps._dt("go"), int(bool(is_row_major)), int(bool(accumulate)),
                                               int(bool(grad_fp32)), int(bool(independent)), _stream(ps.ref)),
              "smlm_b200_wgrad_select_multi")


# ---------------------------------------------------------------------------
# RMSNorm (the caller on either side of the projections)
# ---------------------------------------------------------------------------

def rms_norm(out: torch.Tensor, rms_out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, eps: float):
    """out = x * rsqrt(mean(x^2) + eps) * w per row, rms_out [rows, 1] fp32 gets the rsqrt."""
    with torch.cuda.device(x.device):
        check(lib.smlm_b200_rms_norm(out.data_ptr(), rms_out.data_ptr(), x.data_ptr(), w.data_ptr(), int(x.size(0)),
                                     int(x.size(1)), float(eps), _dtype_code(x), _stream(x)), "smlm_b200_rms_norm")
    return out


def rms_norm_bwd(dx: torch.Tensor, dw: torch.Tensor, go: torch.Tensor, x: torch.Tensor, w: torch.Tensor,
                 rms: torch.Tensor, workspace: Optional[torch.Tensor] = None):
    """dX and dW of ``rms_norm``; ``dw`` in the storage type or fp32."""
    rows, cols = int(x.size(0)), int(x.size(1))
    need = int(lib.smlm_b200_rms_norm_bwd_workspace_bytes(rows, cols))
    ws = workspace if workspace is not None else torch.empty(max(need, 16), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.smlm_b200_rms_norm_bwd(dx.data_ptr(), dw.data_ptr(), go.data_ptr(), x.data_ptr(), w.data_ptr(),
                                         rms.data_ptr(), ws.data_ptr(), ws.numel(), rows, cols, _dtype_code(x),
                                         int(dw.dtype == torch.float32), _stream(x)), "smlm_b200_rms_norm_bwd")
    return dx, dw
