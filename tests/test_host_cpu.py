"""CPU-only checks of the host side: bookkeeping against the reference's vectors,
property tests against the oracle, and the C-ABI library's exported symbols."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from helpers import load_bookkeeping
from oracle import smlm_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_loads_and_exports_every_declared_symbol():
    hdr = "".join(open(os.path.join(ROOT, "include", f)).read() for f in sorted(os.listdir(os.path.join(ROOT, "include")))
                  if f.endswith(".h"))
    declared = sorted(set(re.findall(r"\b(smlm_b200_\w+)\s*\(", hdr)))
    assert len(declared) >= 9
    from loquetier_b200 import cabi
    for name in declared:
        assert hasattr(cabi.lib, name), name
        assert name in cabi.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(cabi.SIGNATURES) == declared
    # pure host entry points can be called without a GPU
    assert cabi.lib.smlm_b200_version() >= 1
    assert cabi.lib.smlm_b200_tmp_size(70) == O.smlm_tmp_size(70) == 4200
    assert cabi.lib.smlm_b200_tmp_size(0) == 0
    bm = cabi.lib.smlm_b200_piece_rows(8192)
    assert 16 <= bm <= 64 and bm % 8 == 0
    assert cabi.lib.smlm_b200_plan_bytes(8192, 100) == (16 + 16 * (8192 // bm + 100 + 1)
                                                        + 16 + 16 * (8192 // 128 + 100 + 1)
                                                        + 4 * (8192 + 4))
    assert cabi.lib.smlm_b200_status_string(3) == b"No suitable kernel."


def test_argument_validation_needs_no_gpu():
    from loquetier_b200 import cabi
    L = cabi.lib
    # dtype, shapes and alignment are rejected before any CUDA call
    assert L.smlm_b200_gemm(16, 16, 16, None, None, 16, 1, 8, 1, 64, 16, 5, 0, 0, 0, None) == 2
    assert L.smlm_b200_gemm(16, 16, 16, None, None, 16, 1, 8, 1, 256, 256, 1, 0, 0, 0, None) == 3
    assert L.smlm_b200_gemm(16, 16, 16, None, None, 16, 1, 8, 1, 64, 12, 1, 0, 0, 0, None) == 3
    assert L.smlm_b200_gemm(16, 24, 16, None, None, 16, 1, 8, 1, 64, 16, 1, 0, 0, 0, None) == 4
    assert L.smlm_b200_gemm(None, 16, 16, None, None, 16, 1, 8, 1, 64, 16, 1, 0, 0, 0, None) == 1
    assert L.smlm_b200_gemm(None, None, None, None, None, None, 0, 0, 0, 64, 16, 1, 0, 0, 0, None) == 0
    assert L.smlm_b200_plan(16, 8, 16, 4, 100, None) == 5
    assert L.smlm_b200_fwd(16, 16, 16, 16, 16, None, None, 16, 1, 8, 1, 64, 64, 130, 1, 0, 0, 0, 0, None) == 3
    with pytest.raises(cabi.SmlmError, match="No suitable kernel"):
        cabi.check(3, "x")


def test_attention_entry_points_validate_before_any_cuda_call():
    """The paged-cache entry points reject bad arguments before any CUDA call (no GPU needed)."""
    from loquetier_b200 import cabi
    L = cabi.lib
    # workspace sizes follow the batch shape
    assert L.smlm_b200_batch_prefill_workspace_bytes(10, 16, 8) == 10 * 16 * 2 * 8 * 128 * 2
    assert L.smlm_b200_batch_prefill_workspace_bytes(0, 16, 8) == 0
    assert L.smlm_b200_batch_decode_workspace_bytes(0, 32, 8) == 0
    ws = L.smlm_b200_batch_prefill_workspace_bytes(4, 16, 8)

    def pre(o=256, wsp=1 << 20, ws_bytes=ws, pages=4, nq=32, hd=128, layer=0, P=16, theta=10000.0, dt=1):
        return L.smlm_b200_batch_prefill(o, 256, 256, 256, 256, 256, wsp, ws_bytes, None, 2, 64, pages, nq, 8, hd, 1,
                                         layer, P, theta, dt, None)

    assert pre(dt=5) == 2                      # dtype
    assert pre(hd=64) == 3                     # head dim outside the path: "No suitable kernel."
    assert pre(P=12) == 3                      # page size
    assert pre(nq=24) == 3                     # 24 query heads on 8 kv heads: a group of 3
    assert pre(layer=1) == 1                   # layer index past the layers
    assert pre(theta=0.0) == 1
    assert pre(o=264) == 4                     # o not 16-byte aligned
    assert pre(wsp=None) == 5 and pre(ws_bytes=ws - 1) == 5   # workspace missing / too small
    assert pre(wsp=(1 << 20) + 16) == 4        # workspace not 128-byte aligned
    assert pre(pages=0) == 1                   # queries without a single page of keys

    def dec(nq=32, hd=128, P=16, dt=1):
        return L.smlm_b200_batch_decode(256, 256, 256, 256, 256, None, 0, None, 2, 4, nq, 8, hd, 1, 0, P, 10000.0, dt,
                                        None)

    assert dec(dt=7) == 2 and dec(hd=96) == 3 and dec(P=128) == 3 and dec(nq=40) == 3
    assert dec() == 5                          # 2 requests x 8 heads are cut into page ranges: a workspace is needed

    def app(k=256, hd=128, dt=0):
        return L.smlm_b200_append_kv(256, 256, 256, k, 256, None, 2, 4, 1, 0, 8, hd, 16, dt, None)

    assert app(dt=9) == 2 and app(hd=256) == 3 and app(k=264) == 4
    # the weight gradients of one kind: `which` must name dB, dA or both
    assert L.smlm_b200_wgrad_select_multi(None, 0, 0, None, None, None, None, None, 0, 0, 0, 0, 16, 1, 0, 0, 0, 0,
                                          None) == 1


def test_batch_len_info_matches_reference():
    from loquetier_b200.kernel_utils import BatchLenInfo
    for row in load_bookkeeping()["batch_len_info"]:
        c = row["case"]
        b = BatchLenInfo([tuple(t) for t in c["trains"]], c["prefills"], c["decode"],
                         [tuple(t) for t in c["evals"]], torch.device("cpu"))
        assert [int(v) for v in b.train_partition] == row["train_partition"]
        assert int(b.tlen) == row["tlen"] and int(b.doff) == row["doff"] and b.decode == row["decode"]
        assert [int(v) for v in b.eval_partition] == row["eval_partition"]
        assert [int(v) for v in b.prefills] == row["prefills"]
        if row["indptr"] is None:
            assert b.indptr is None
        else:
            assert b.indptr.tolist() == row["indptr"] and str(b.indptr.dtype) == row["indptr_dtype"]


def test_segment_builder_matches_reference():
    from loquetier_b200.enums import InferStatus
    from loquetier_b200.segments import SegmentRequest, build_segment_batch, order_requests
    for row in load_bookkeeping()["segments"]:
        groups = {"train": [], "eval": [], "prefill": [], "decode": []}
        for kind, lid, n in row["spec"]:
            st = {"train": InferStatus.Train, "eval": InferStatus.Prefill, "prefill": InferStatus.Prefill,
                  "decode": InferStatus.Decode}[kind]
            groups[kind].append(SegmentRequest(st, lid, n, is_eval=(kind == "eval")))
        ordered = order_requests(groups["train"], groups["eval"], groups["prefill"], groups["decode"])
        sb = build_segment_batch(ordered, "cpu")
        assert sb.lora_ids == row["lora_ids"]
        assert sb.lora_len.tolist() == row["lora_len"] and str(sb.lora_len.dtype) == row["lora_len_dtype"]
        assert sb.segment.tolist() == row["segment"] and str(sb.segment.dtype) == row["segment_dtype"]
        assert sb.train_idx == row["train_idx"] and sb.n_tokens == row["n_tokens"]


def test_segment_builder_properties():
    hyp = pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as st
    from loquetier_b200.enums import InferStatus
    from loquetier_b200.segments import SegmentRequest, merge_segments, order_requests

    req = st.tuples(st.sampled_from(["train", "eval", "prefill", "decode"]), st.integers(0, 5), st.integers(1, 40))

    @settings(max_examples=200, deadline=None)
    @given(st.lists(req, min_size=0, max_size=40))
    def prop(spec):
        groups = {"train": [], "eval": [], "prefill": [], "decode": []}
        og = {"train": [], "eval": [], "prefill": [], "decode": []}
        for kind, lid, n in spec:
            n = 1 if kind == "decode" else n
            stt = {"train": InferStatus.Train, "eval": InferStatus.Prefill, "prefill": InferStatus.Prefill,
                   "decode": InferStatus.Decode}[kind]
            groups[kind].append(SegmentRequest(stt, lid, n))
            og[kind].append((lid, n))
        ordered = order_requests(groups["train"], groups["eval"], groups["prefill"], groups["decode"])
        ids, lens = merge_segments(ordered)
        oids, olens, oseg = O.merge_segments(O.order_requests(og["train"], og["eval"], og["prefill"], og["decode"]))
        assert ids == oids and lens == olens
        assert sum(lens) == sum(r.n_tokens for r in ordered)
        assert all(a != b for a, b in zip(ids, ids[1:])) and all(n > 0 for n in lens)

    prop()


def test_prepare_weight_pads_rank_and_bakes_scale():
    from loquetier_b200.mixed_lora import prepare_weight
    w = torch.arange(12, dtype=torch.float32).reshape(3, 4)
    p = prepare_weight(w, 8, torch.float32, "cpu", rank_dim=0, scaling=2.0)
    assert p.shape == (8, 4) and torch.equal(p[:3], w * 2) and (p[3:] == 0).all()
    q = prepare_weight(w.t().contiguous(), 8, torch.bfloat16, "cpu", rank_dim=1)
    assert q.shape == (4, 8) and q.dtype == torch.bfloat16 and (q[:, 3:] == 0).all()
    same = prepare_weight(w, 3, torch.float16, "cpu")
    assert same.shape == (3, 4) and same.is_contiguous()


def test_grouped_plan_is_requested_only_when_it_changes_something():
    from loquetier_b200.segments import wants_grouped_plan
    assert not wants_grouped_plan([], [])
    assert not wants_grouped_plan([100, 1, 1, 9], [0, 1, 2, 1])      # no adapter has two short segments
    assert wants_grouped_plan([100, 1, 50, 8], [0, 1, 2, 1])        # adapter 1: rows 100 and 151..158
    assert not wants_grouped_plan([0, 0, 4], [3, 3, 3])             # empty segments do not count
    assert wants_grouped_plan([1] * 4, [7, 2, 5, 7])


@pytest.mark.parametrize("name", ["prepare_weight_bf16", "prepare_weight_fp16"])
def test_prepare_weight_matches_the_reference_bit_for_bit(name):
    """Against MixedLoraModel._prepare_weight of the reference (mixed_lora.py:501-521) run on the same inputs:
    padding along either dimension, the scale baked in before the cast."""
    from helpers import load_npz
    from loquetier_b200.mixed_lora import prepare_weight
    z = load_npz(name)
    dt = z["dtype"]
    for key, rank_dim, scaling in (("a_small", 0, 2.0), ("b_small", 1, None), ("a_full", 0, 0.3)):
        got = prepare_weight(z[key], 16, dt, "cpu", rank_dim=rank_dim, scaling=scaling)
        want = z[key + "_out"]
        assert got.dtype == dt and got.is_contiguous() and got.shape == want.shape
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), key


def test_install_as_loquetier_kernels_resolves_the_reference_import():
    """`from loquetier.ops import _kernels` (src/loquetier_src/kernel_utils.py:8 of the reference) must find the
    three names its pybind module registers for this path (kernel_src/csrc/loquetier_ops.cc:371-373)."""
    import sys
    saved = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "loquetier" or k.startswith("loquetier.")}
    try:
        from loquetier_b200 import kernels
        me = kernels.install_as_loquetier_kernels()
        from loquetier.ops import _kernels as kernel
        assert kernel is me is kernels
        import loquetier.ops._kernels as again
        assert again is kernels
        for name in ("smlm_forward_cutlass", "smlm_forward_cutlass_tmp_size", "rms_norm"):
            assert callable(getattr(kernel, name)), name
        assert kernel.smlm_forward_cutlass_tmp_size(70) == 4200
        # the argument checks of the dispatcher run before any device work
        t = torch.zeros((4, 8))
        with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
            kernel.smlm_forward_cutlass(t, t, torch.zeros(1, dtype=torch.int64), torch.zeros(2, dtype=torch.int32),
                                        torch.zeros(60, dtype=torch.uint8), False)
    finally:
        for k in [k for k in sys.modules if k == "loquetier" or k.startswith("loquetier.")]:
            del sys.modules[k]
        sys.modules.update(saved)
