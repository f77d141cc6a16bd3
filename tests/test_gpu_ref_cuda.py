"""The reference's own CUDA kernels as a second witness on the GPU: the CUTLASS grouped GEMM behind
``smlm_forward_cutlass`` and the RMSNorm kernel, compiled from the reference checkout by
``oracle/build_ref.py`` into ``oracle/_ref/libref.so``.  Three-way agreement: reference kernel, this
library's kernels, CPU oracle.  Skipped when the reference library has not been built."""
import numpy as np
import pytest
import torch

import ref_cuda
from gpu_util import dev, ptr_table, to_dev
from helpers import assert_close, load_npz
from oracle import smlm_oracle as O

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref/libref.so not built")]


def _mismatch(a, b):
    return float((a.view(torch.int16) != b.view(torch.int16)).float().mean())


@pytest.mark.parametrize("name", ["rmsnorm_bf16", "rmsnorm_fp16"])
def test_rms_norm_forward_reference_kernel_pins_oracle_and_library(name):
    from loquetier_b200 import kernels
    z = load_npz(name)
    dt = z["dtype"]
    rows, cols, eps = int(z["meta"][0]), int(z["meta"][1]), float(z["meta"][2])
    x, w = z["x"].to(dev()), z["w"].to(dev())
    o_ref = torch.empty_like(x)
    m_ref = torch.empty((rows, 1), dtype=torch.float32, device=dev())
    ref_cuda.rms_norm(o_ref, m_ref, x, w, eps)
    o_or, m_or = O.rms_norm_forward(z["x"], z["w"], eps)
    # the reference kernel against the CPU restatement of it: the same value up to the order of the fp32 sum
    assert torch.allclose(m_ref.cpu(), m_or, rtol=2e-6, atol=0)
    assert _mismatch(o_ref.cpu(), o_or) < 2e-3
    assert_close(o_ref, o_or, what="reference kernel vs oracle")
    o = torch.empty_like(x)
    m = torch.empty_like(m_ref)
    kernels.rms_norm(o, m, x, w, eps)
    torch.cuda.synchronize()
    assert torch.allclose(m, m_ref, rtol=2e-6, atol=0)
    assert _mismatch(o, o_ref) < 2e-3
    assert_close(o, o_ref, what="library vs reference kernel")


@pytest.mark.parametrize("rows,cols", [(1, 8), (3, 4096), (64, 8192), (130, 11008)])
def test_rms_norm_forward_matches_reference_kernel_on_model_shapes(rows, cols):
    from loquetier_b200 import kernels
    g = torch.Generator().manual_seed(rows * 7 + cols)
    x = (torch.randn((rows, cols), generator=g) * 1.5).to(torch.bfloat16).to(dev())
    w = (1.0 + 0.1 * torch.randn((cols,), generator=g)).to(torch.bfloat16).to(dev())
    o_ref, o = torch.empty_like(x), torch.empty_like(x)
    m_ref = torch.empty((rows, 1), dtype=torch.float32, device=dev())
    m = torch.empty_like(m_ref)
    ref_cuda.rms_norm(o_ref, m_ref, x, w, 1e-5)
    kernels.rms_norm(o, m, x, w, 1e-5)
    torch.cuda.synchronize()
    assert torch.allclose(m, m_ref, rtol=2e-6, atol=0)
    assert _mismatch(o, o_ref) < 2e-3
    assert_close(o, o_ref, what="library vs reference kernel")


def _three_way(case, what):
    """shrink then expand as add_lora.forward issues them (kernel_utils.py:117-119), on the reference's
    kernel, on this library behind the same operator name, and fused; then the oracle."""
    from loquetier_b200 import kernels, ops
    c = to_dev(case)
    T, r = c["x"].shape[0], c["rank"]
    dt = c["dtype"]
    wa = ptr_table([c["wa_d"][i] for i in c["ids"]])
    wb = ptr_table([c["wb_d"][i] for i in c["ids"]])
    rm = c["is_row_major"]
    a, b = c["seg"][0], c["seg"][-1]
    v_ref = torch.zeros((T, r), dtype=dt, device=dev())
    y_ref = torch.zeros((T, c["h_out"]), dtype=dt, device=dev())
    torch.cuda.synchronize()
    ref_cuda.smlm_forward_cutlass(v_ref, c["x"], wa, c["seg_d"], rm)
    ref_cuda.smlm_forward_cutlass(y_ref, v_ref, wb, c["seg_d"], rm)
    torch.cuda.synchronize()
    v_lib, y_lib = torch.zeros_like(v_ref), torch.zeros_like(y_ref)
    tmp = torch.empty(kernels.smlm_forward_cutlass_tmp_size(len(c["ids"])), dtype=torch.uint8, device=dev())
    kernels.smlm_forward_cutlass(v_lib, c["x"], wa, c["seg_d"], tmp, rm)
    kernels.smlm_forward_cutlass(y_lib, v_lib, wb, c["seg_d"], tmp, rm)
    v_f, y_f = torch.zeros_like(v_ref), torch.zeros_like(y_ref)
    plan = ops.Plan(c["seg_d"], T)
    ops.fwd(y_f, c["x"], v_f, wa, wb, plan, r, is_row_major=rm)
    torch.cuda.synchronize()
    plan.raise_if_failed()
    y_or, v_or = O.add_lora_forward((T, c["h_out"]), case["x"], [case["wa"][i] for i in case["ids"]],
                                    [case["wb"][i] for i in case["ids"]], case["seg"], r, is_row_major=rm)
    assert_close(v_ref[a:b], v_or[a:b], what=f"{what}: reference kernel v vs oracle")
    assert_close(y_ref[a:b], y_or[a:b], what=f"{what}: reference kernel y vs oracle")
    for nm, vv, yy in (("operator", v_lib, y_lib), ("fused", v_f, y_f)):
        assert_close(vv[a:b], v_ref[a:b], what=f"{what}: {nm} v vs reference kernel")
        assert_close(yy[a:b], y_ref[a:b], what=f"{what}: {nm} y vs reference kernel")
    # rows no segment covers stay as they were in every implementation
    for t in (v_ref, y_ref, v_lib, y_lib, v_f, y_f):
        assert bool((t[:a] == 0).all()) and bool((t[b:] == 0).all())
    return _mismatch(y_f[a:b].cpu(), y_ref[a:b].cpu())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_smlm_forward_c1_against_reference_kernel(dtype):
    c = O.make_case(1000, [7, 33, 1, 64], [0, 2, 1, 0], 3, 256, 256, 8, dtype)
    _three_way(c, "c1")


def test_smlm_forward_c2_against_reference_kernel():
    rng = np.random.default_rng(2000)
    lens = [1024, 1024] + [512] * 4 + [1] * 64
    ids = [int(v) for v in rng.integers(0, 32, size=len(lens))]
    c = O.make_case(2000, lens, ids, 32, 4096, 4096, 16, torch.float16)
    _three_way(c, "c2")


@pytest.mark.parametrize("h_in,h_out", [(4096, 11008), (11008, 4096)])
def test_smlm_forward_c4_decode_against_reference_kernel(h_in, h_out):
    rng = np.random.default_rng(4000)
    ids = [int(v) for v in rng.integers(0, 256, size=1024)]
    c = O.make_case(4000, [1] * 1024, ids, 256, h_in, h_out, 32, torch.bfloat16)
    _three_way(c, "c4")


@pytest.mark.parametrize("rm", [False, True])
def test_smlm_forward_edge_lengths_and_layouts_against_reference_kernel(rm):
    lens = [0, 1, 15, 16, 17, 31, 33, 0, 64, 65, 1, 1, 127, 2]
    rng = np.random.default_rng(5)
    ids = [int(v) for v in rng.integers(0, 4, size=len(lens))]
    c = O.make_case(5 + rm, lens, ids, 4, 320, 192, 16, torch.bfloat16, is_row_major=rm)
    _three_way(c, f"edges rm={rm}")
