"""GPU parity of the tcgen05 kernel (ranks above 32, 128-row tiles) against the CPU oracle and
against the mma.sync kernel, through the C ABI.  The kernel is forced on so that small and
ragged batches reach it.  Tolerance as for the other kernels: rtol 1e-2, atol 1e-2."""
import numpy as np
import pytest
import torch

from helpers import assert_close
from oracle import smlm_oracle as O

pytestmark = pytest.mark.gpu

TALL_LENS = [0, 1, 127, 128, 129, 0, 300, 64, 15, 1, 256]


@pytest.fixture(autouse=True)
def forced_tensor_core_kernel():
    from loquetier_b200 import ops
    prev = ops.set_tensor_core_mode(1)
    yield
    ops.set_tensor_core_mode(prev)


def _case(seed, lens, n_ad, h_in, h_out, rank, dtype, rm=False, ids=None):
    rng = np.random.default_rng(seed)
    ids = list(rng.integers(0, n_ad, size=len(lens))) if ids is None else ids
    return O.make_case(seed, lens, [int(i) for i in ids], n_ad, h_in, h_out, rank, dtype, is_row_major=rm)


def test_first_light_rank64():
    from gpu_util import check_forward
    check_forward(_case(1, [128], 1, 256, 128, 64, torch.bfloat16, False, ids=[0]))
    check_forward(_case(2, [128, 40], 2, 512, 256, 64, torch.bfloat16, False))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rm", [False, True])
@pytest.mark.parametrize("rank", [40, 64, 96, 128])
def test_forward_edge_lengths(dtype, rm, rank):
    from gpu_util import check_forward
    check_forward(_case(400 + rank, TALL_LENS, 5, 200, 328, rank, dtype, rm))


@pytest.mark.parametrize("h_in,h_out", [(4096, 1024), (1000, 264), (14336, 4096), (4096, 14336)])
@pytest.mark.parametrize("rm", [False, True])
def test_forward_shapes(h_in, h_out, rm):
    from gpu_util import check_forward
    c = _case(17, [200, 1, 3, 130, 128], 4, h_in, h_out, 64, torch.bfloat16, rm)
    check_forward(c)
    check_forward(c, indexed=True)


def test_forward_scale_and_accumulate():
    from gpu_util import check_forward
    c = _case(18, [140, 1, 290, 17], 3, 512, 776, 64, torch.bfloat16)
    g = torch.Generator().manual_seed(1)
    y0 = torch.randn((sum(c["lens"]), 776), generator=g).to(torch.bfloat16)
    check_forward(c, scale=[2.0, 0.5, 1.25])
    check_forward(c, scale=[2.0, 0.5, 1.25], indexed=True, accumulate=True, y_init=y0)


def test_rows_outside_segments_untouched_and_deterministic():
    from gpu_util import dev, ptr_table, to_dev
    from loquetier_b200 import ops
    c = to_dev(_case(19, [133, 1, 164], 3, 256, 384, 64, torch.float16))
    T = 310
    x = torch.randn((T, 256), device=dev(), dtype=torch.float16)
    seg = torch.tensor([4, 137, 138, 302], dtype=torch.int32, device=dev())
    plan = ops.Plan(seg, T)
    wa = ptr_table([c["wa_d"][i] for i in c["ids"]])
    wb = ptr_table([c["wb_d"][i] for i in c["ids"]])
    outs = []
    for _ in range(2):
        y = torch.full((T, 384), 7.0, dtype=torch.float16, device=dev())
        v = torch.full((T, 64), 3.0, dtype=torch.float16, device=dev())
        ops.fwd(y, x, v, wa, wb, plan, 64)
        outs.append((y.clone(), v.clone()))
    torch.cuda.synchronize()
    plan.raise_if_failed()
    y, v = outs[0]
    assert (y[:4] == 7).all() and (y[302:] == 7).all() and (v[:4] == 3).all() and (v[302:] == 3).all()
    assert not (y[4:302] == 7).all()
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


def test_matches_the_mma_sync_kernel():
    from gpu_util import run_forward
    from loquetier_b200 import ops
    c = _case(20, [300, 128, 77], 3, 1024, 640, 64, torch.bfloat16)
    y_tc, v_tc = run_forward(c)
    ops.set_tensor_core_mode(-1)
    y_mma, v_mma = run_forward(c)
    assert_close(v_tc, v_mma.to(torch.float32), rtol=1e-2, atol=1e-2, what="v")
    assert_close(y_tc, y_mma.to(torch.float32), rtol=1e-2, atol=1e-2, what="y")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rm", [False, True])
@pytest.mark.parametrize("rank", [16, 32, 40, 64, 128])
def test_backward_vs_oracle(dtype, rm, rank):
    # ranks up to 32: the forced mode sends only the weight gradients to the tcgen05 kernel (rank padded to 32)
    from test_gpu_parity import _grad_close, _oracle_bwd, _run_bwd
    part = [0, 133, 133, 330, 331, 600]
    c = _case(500 + rank, [610], 5, 264, 200, rank, dtype, rm, ids=[0])
    dx, dA, dB = _run_bwd(c, part)
    gx, gA, gB = _oracle_bwd(c, part)
    _grad_close(dx[:600], gx[:600], "dX")
    assert (dx[600:] == 0).all()
    for p in range(5):
        _grad_close(dA[p], gA[p], f"dA{p}")
        _grad_close(dB[p], gB[p], f"dB{p}")


def test_backward_scale_fp32_accumulate():
    from test_gpu_parity import _grad_close, _oracle_bwd, _run_bwd
    part = [0, 100, 457]
    c = _case(600, [457], 2, 512, 320, 64, torch.bfloat16, False, ids=[0])
    dx, dA, dB = _run_bwd(c, part, scale=[2.0, 0.5], grad_fp32=True, accumulate=True)
    gx, gA, gB = _oracle_bwd(c, part, scale=[2.0, 0.5])
    _grad_close(dx, gx, "dX")
    for p in range(2):
        assert dA[p].dtype == torch.float32
        _grad_close(dA[p] - 1.0, gA[p], f"dA{p}")
        _grad_close(dB[p] - 1.0, gB[p], f"dB{p}")


@pytest.mark.parametrize("rm", [False, True])
def test_backward_many_partitions_per_group(rm):
    """Enough pieces that a CTA of the weight-gradient kernel owns several of them: runs that end
    inside a CTA, runs that straddle CTAs, and more than two runs per CTA."""
    from test_gpu_parity import _grad_close, _oracle_bwd, _run_bwd
    rng = np.random.default_rng(5)
    lens = [int(v) for v in rng.integers(0, 200, size=100)]
    part = [0] + [int(v) for v in np.cumsum(lens)]
    c = _case(601, [part[-1] + 7], 100, 512, 1024, 64, torch.bfloat16, rm, ids=[0])
    dx, dA, dB = _run_bwd(c, part)
    gx, gA, gB = _oracle_bwd(c, part)
    _grad_close(dx[:part[-1]], gx[:part[-1]], "dX")
    for p in range(100):
        _grad_close(dA[p], gA[p], f"dA{p}")
        _grad_close(dB[p], gB[p], f"dB{p}")
    # the ticketed sum runs in a fixed order: a second launch gives the same bits
    dx2, dA2, dB2 = _run_bwd(c, part)
    assert all(torch.equal(a, b) for a, b in zip(dA, dA2)) and all(torch.equal(a, b) for a, b in zip(dB, dB2))


def test_bad_adapter_pointer_is_reported_not_dereferenced():
    from gpu_util import dev, ptr_table, to_dev
    from loquetier_b200 import cabi, ops
    c = to_dev(_case(21, [150, 20], 2, 256, 256, 64, torch.bfloat16))
    T = 170
    plan = ops.Plan(c["seg_d"], T)
    wa = ptr_table([c["wa_d"][i] for i in c["ids"]])
    wb = ptr_table([c["wb_d"][i] for i in c["ids"]])
    wb[1] = 0
    y = torch.zeros((T, 256), dtype=torch.bfloat16, device=dev())
    v = torch.zeros((T, 64), dtype=torch.bfloat16, device=dev())
    ops.fwd(y, c["x"], v, wa, wb, plan, 64)
    torch.cuda.synchronize()
    with pytest.raises(cabi.SmlmError):
        plan.raise_if_failed()
    assert (y[150:] == 0).all()


def test_c5_full_size_both_kernels_and_oracle_slices():
    """The fine-tune-heavy configuration at full size (16 x 2048 tokens, rank 64, 4096 -> 14336): the
    kernel choice left to the library (long segments: tcgen05), against the mma.sync kernels on the
    same tensors, and against the CPU oracle on slices of rows (rows are independent of each other)."""
    from gpu_util import dev, ptr_table
    from loquetier_b200 import ops
    ops.set_tensor_core_mode(0)
    T, nseg, h_in, h_out, r = 32768, 16, 4096, 14336, 64
    g = torch.Generator(device=dev()).manual_seed(55)
    dt = torch.bfloat16
    x = torch.randn((T, h_in), generator=g, device=dev(), dtype=torch.float32).to(dt)
    go = torch.randn((T, h_out), generator=g, device=dev(), dtype=torch.float32).to(dt)
    wa = [(torch.randn((r, h_in), generator=g, device=dev()) / h_in ** 0.5).to(dt) for _ in range(nseg)]
    wb = [(torch.randn((h_out, r), generator=g, device=dev()) * 0.02).to(dt) for _ in range(nseg)]
    seg = torch.arange(0, T + 1, T // nseg, dtype=torch.int32, device=dev())
    wa_t, wb_t = ptr_table(wa), ptr_table(wb)

    def run():
        plan = ops.Plan(seg, T)
        y = torch.zeros((T, h_out), dtype=dt, device=dev())
        v = torch.zeros((T, r), dtype=dt, device=dev())
        ops.fwd(y, x, v, wa_t, wb_t, plan, r)
        dx = torch.zeros((T, h_in), dtype=dt, device=dev())
        dv = torch.zeros((T, r), dtype=dt, device=dev())
        dA = [torch.zeros_like(w) for w in wa]
        dB = [torch.zeros_like(w) for w in wb]
        ops.bwd(dx, ptr_table(dA), ptr_table(dB), dv, go, x, v, wa_t, wb_t, plan, r)
        torch.cuda.synchronize()
        plan.raise_if_failed()
        return y, v, dx, dA, dB

    y, v, dx, dA, dB = run()
    ops.set_tensor_core_mode(-1)
    y2, v2, dx2, dA2, dB2 = run()

    def close(a, b, what):
        a32, b32 = a.float(), b.float()
        tol = 1e-2 * max(1.0, float(b32.abs().max()))
        bad = (a32 - b32).abs() > tol + 1e-2 * b32.abs()
        assert not bool(bad.any()), f"{what}: {int(bad.sum())} elements differ"

    close(v, v2, "v")
    close(y, y2, "y")
    close(dx, dx2, "dX")
    for p in (0, 7, 15):
        close(dA[p], dA2[p], f"dA{p}")
        close(dB[p], dB2[p], f"dB{p}")
    # oracle on row slices: fp32 on the host from the same 16-bit inputs
    for s, off, n in ((0, 0, 40), (5, 1000, 64), (15, 2047, 1)):
        a, b = s * 2048 + off, s * 2048 + off + n
        xs = x[a:b].cpu().float()
        vs = (xs @ wa[s].cpu().float().T).to(dt).float()
        ys = vs @ wb[s].cpu().float().T
        assert_close(v[a:b].cpu(), vs, what=f"v rows of segment {s}")
        assert_close(y[a:b].cpu(), ys, what=f"y rows of segment {s}")
        gs = go[a:b].cpu().float()
        dvs = gs @ wb[s].cpu().float()
        dxs = dvs @ wa[s].cpu().float()
        assert_close(dx[a:b].cpu(), dxs, rtol=2e-2, atol=2e-2, what=f"dX rows of segment {s}")
    # one adapter's gradients against the oracle formulas (dB = gO^T v, dA = dV^T x), fp32 on the device
    s = 9
    a, b = s * 2048, (s + 1) * 2048
    vs = (x[a:b].float() @ wa[s].float().T).to(dt).float()
    dB_ref = go[a:b].float().T @ vs
    dvs = (go[a:b].float() @ wb[s].float())
    dA_ref = dvs.T @ x[a:b].float()
    close(dB[s], dB_ref, "dB vs fp32")
    close(dA[s], dA_ref, "dA vs fp32")


# ---- either product alone (one reference operator call each) on the tcgen05 kernel ----

def _check_halves(case, scale=None, accumulate=False, y_init=None):
    """v = x . W1 by one shrink-only call, y (+)= scale * v . W2 by one expand-only call, against the oracle's
    two-call forward (v rounded to the storage type in between)."""
    from gpu_util import dev, oracle_forward, ptr_table, to_dev
    from loquetier_b200 import ops
    c = to_dev(case)
    T = c["x"].shape[0]
    plan = ops.Plan(c["seg_d"], T)
    wa_t = ptr_table([c["wa_d"][i] for i in c["ids"]])
    wb_t = ptr_table([c["wb_d"][i] for i in c["ids"]])
    v = torch.full((T, c["rank"]), 7.0, dtype=c["dtype"], device=dev())
    y = (torch.zeros((T, c["h_out"]), dtype=c["dtype"], device=dev()) if y_init is None else y_init.to(dev()).clone())
    sc = None if scale is None else torch.tensor([scale[i] for i in c["ids"]], dtype=torch.float32, device=dev())
    ops.gemm(v, c["x"], wa_t, plan, is_row_major=c["is_row_major"])
    ops.gemm(y, v, wb_t, plan, is_row_major=c["is_row_major"], seg_scale=sc, accumulate=accumulate)
    torch.cuda.synchronize()
    plan.raise_if_failed()
    y_ref, v_ref = oracle_forward(case, scale=scale, y_init=y_init)
    a, b = case["seg"][0], case["seg"][-1]
    assert_close(v.cpu()[a:b], v_ref[a:b], what="v (shrink alone)")
    assert_close(y.cpu()[a:b], y_ref[a:b], what="y (expand alone)")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rm", [False, True])
@pytest.mark.parametrize("rank", [40, 64, 128])
def test_halves_edge_lengths(dtype, rm, rank):
    _check_halves(_case(600 + rank, TALL_LENS, 5, 200, 328, rank, dtype, rm))


@pytest.mark.parametrize("h_in,h_out", [(4096, 1024), (14336, 4096), (4096, 14336)])
@pytest.mark.parametrize("rm", [False, True])
def test_halves_shapes(h_in, h_out, rm):
    _check_halves(_case(27, [200, 1, 3, 130, 128], 4, h_in, h_out, 64, torch.bfloat16, rm))


def test_halves_scale_and_accumulate():
    c = _case(28, [140, 1, 290, 17], 3, 512, 776, 64, torch.bfloat16)
    g = torch.Generator().manual_seed(2)
    y0 = torch.randn((sum(c["lens"]), 776), generator=g).to(torch.bfloat16)
    _check_halves(c, scale=[2.0, 0.5, 1.25])
    _check_halves(c, scale=[2.0, 0.5, 1.25], accumulate=True, y_init=y0)
