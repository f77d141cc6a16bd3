"""ctypes binding of ``libsmlm_b200.so`` (declared in ``include/smlm_b200.h``).

The library is the product: there is no fallback.  If it has not been built the
import fails with the command that builds it."""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsmlm_b200.so")

SMLM_OK = 0
SMLM_F16 = 0
SMLM_BF16 = 1

STATUS_NAMES = {
    0: "SMLM_OK", 1: "SMLM_ERR_INVALID_ARGUMENT", 2: "SMLM_ERR_DTYPE", 3: "SMLM_ERR_NO_KERNEL",
    4: "SMLM_ERR_MISALIGNED", 5: "SMLM_ERR_WORKSPACE", 6: "SMLM_ERR_CUDA", 7: "SMLM_ERR_BAD_INDPTR",
    8: "SMLM_ERR_BAD_POINTER", 9: "SMLM_ERR_BAD_INDEX", 10: "SMLM_ERR_TIMEOUT", 11: "SMLM_ERR_STATIC_LIMIT",
    12: "SMLM_ERR_GROUPED_PLAN",
}

SMLM_MAX_PROJ = 8


class SmlmProj(ctypes.Structure):
    """``smlm_b200_proj`` of include/smlm_b200.h: the tensors of one projection for the entry points
    that serve several projections per launch."""
    _fields_ = [("x", c_void_p), ("y", c_void_p), ("v", c_void_p), ("go", c_void_p), ("dx", c_void_p),
                ("dv", c_void_p), ("wa_table", c_void_p), ("wb_table", c_void_p), ("dA_table", c_void_p),
                ("dB_table", c_void_p), ("h_in", c_int), ("h_out", c_int)]


# name -> (restype, argtypes); mirrors include/smlm_b200.h and include/smlm_b200_kv.h one to one
SIGNATURES = {
    "smlm_b200_version": (c_int, []),
    "smlm_b200_status_string": (c_char_p, [c_int]),
    "smlm_b200_tmp_size": (c_size_t, [c_int]),
    "smlm_b200_group_ids_from_pointers": (c_int, [c_void_p, c_int, c_void_p, c_void_p]),
    "smlm_b200_merge_segments": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "smlm_b200_piece_rows": (c_int, [c_int]),
    "smlm_b200_set_tensor_core_mode": (c_int, [c_int]),
    "smlm_b200_set_cluster_split": (c_int, [c_int]),
    "smlm_b200_plan_bytes": (c_size_t, [c_int, c_int]),
    "smlm_b200_plan": (c_int, [c_void_p, c_size_t, c_void_p, c_int, c_int, c_void_p]),
    "smlm_b200_plan_grouped": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "smlm_b200_plan_pair": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_int, c_int, c_int,
                                    c_void_p, c_size_t, c_void_p, c_int, c_int, c_void_p]),
    "smlm_b200_plan_status": (c_int, [c_void_p, ctypes.POINTER(c_int), c_void_p]),
    "smlm_b200_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "smlm_b200_fwd": (c_int, [c_void_p] * 8 + [c_int] * 11 + [c_void_p]),
    "smlm_b200_bwd_dx": (c_int, [c_void_p] * 8 + [c_int] * 10 + [c_void_p]),
    "smlm_b200_wgrad_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "smlm_b200_wgrad_ticket_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "smlm_b200_wgrad": (c_int, [c_void_p] * 7 + [c_size_t] + [c_int] * 8 + [c_void_p]),
    "smlm_b200_wgrad_static": (c_int, [c_void_p] * 6 + [c_int] * 8 + [c_void_p]),
    "smlm_b200_wgrad_pair": (c_int, [c_void_p] * 11 + [c_size_t] + [c_int] * 11 + [c_void_p]),
    "smlm_b200_bwd": (c_int, [c_void_p] * 14 + [c_size_t] + [c_int] * 10 + [c_void_p]),
    "smlm_b200_fwd_multi": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p] + [c_int] * 9 + [c_void_p]),
    "smlm_b200_bwd_dx_multi": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p] + [c_int] * 7 + [c_void_p]),
    "smlm_b200_wgrad_multi_workspace_bytes": (c_size_t, [c_void_p, c_int, c_int, c_int, c_int]),
    "smlm_b200_wgrad_multi_ticket_bytes": (c_size_t, [c_void_p, c_int, c_int, c_int, c_int]),
    "smlm_b200_wgrad_pair_multi": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_size_t] + [c_int] * 9 + [c_void_p]),
    "smlm_b200_wgrad_select_multi": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_size_t] + [c_int] * 9 + [c_void_p]),
    "smlm_b200_batch_decode_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "smlm_b200_batch_decode_ticket_bytes": (c_size_t, [c_int, c_int]),
    "smlm_b200_batch_prefill_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "smlm_b200_batch_prefill": (c_int, [c_void_p] * 7 + [c_size_t, c_void_p] + [c_int] * 9 + [c_float, c_int, c_void_p]),
    "smlm_b200_batch_decode": (c_int, [c_void_p] * 6 + [c_size_t, c_void_p] + [c_int] * 8 + [c_float, c_int, c_void_p]),
    "smlm_b200_append_kv": (c_int, [c_void_p] * 6 + [c_int] * 8 + [c_void_p]),
    "smlm_b200_init_kv": (c_int, [c_void_p] * 7 + [c_int] * 9 + [c_void_p]),
    "smlm_b200_rms_norm": (c_int, [c_void_p] * 4 + [c_int, c_int, c_float, c_int, c_void_p]),
    "smlm_b200_rms_norm_bwd_workspace_bytes": (c_size_t, [c_int, c_int]),
    "smlm_b200_rms_norm_bwd": (c_int, [c_void_p] * 7 + [c_size_t] + [c_int] * 4 + [c_void_p]),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA library of the SMLM path has not been built. "
            "Build it with `python -m loquetier_b200.build` (needs nvcc); there is no CPU fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


class SmlmError(RuntimeError):
    """Raised for a non-zero status; the reference surfaces its failures as
    RuntimeError through TORCH_CHECK (kernel_src/csrc/loquetier_ops.cc:318)."""

    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib.smlm_b200_status_string(status).decode()
        super().__init__(f"{where}: {msg} [{STATUS_NAMES.get(status, status)}]")


def check(status: int, where: str) -> None:
    if status != SMLM_OK:
        raise SmlmError(status, where)
