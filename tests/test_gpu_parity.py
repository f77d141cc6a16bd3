"""GPU parity of the SMLM path against the CPU oracle, through the C ABI.
Tolerance for 16-bit storage with fp32 accumulation: rtol 1e-2, atol 1e-2;
bookkeeping (plans, untouched rows, determinism) is bit-exact."""
import numpy as np
import pytest
import torch

from helpers import assert_close, load_npz
from oracle import smlm_oracle as O

pytestmark = pytest.mark.gpu

EDGE_LENS = [0, 1, 15, 16, 17, 31, 33, 0, 64, 65, 1, 1, 127, 2]


def _case(seed, lens, n_ad, h_in, h_out, rank, dtype, rm=False, ids=None):
    rng = np.random.default_rng(seed)
    ids = list(rng.integers(0, n_ad, size=len(lens))) if ids is None else ids
    return O.make_case(seed, lens, [int(i) for i in ids], n_ad, h_in, h_out, rank, dtype, is_row_major=rm)


# ---------------------------------------------------------------------------
# plan
# ---------------------------------------------------------------------------

def test_plan_pieces_bit_exact():
    from loquetier_b200 import ops
    rng = np.random.default_rng(0)
    for trial in range(6):
        nseg = [1, 5, 70, 1024, 1500, 3000][trial]
        lens = rng.integers(0, 200, size=nseg)
        if trial == 2:
            lens[:3] = [2048, 1024, 777]
        seg = np.concatenate([[3], 3 + np.cumsum(lens)]).astype(np.int32)
        T = int(seg[-1]) + 5
        s = torch.tensor(seg, device="cuda")
        plan = ops.Plan(s, T)
        n, rc = plan.status()
        assert rc == 0
        from loquetier_b200 import cabi
        bm = cabi.lib.smlm_b200_piece_rows(T)
        assert 16 <= bm <= 64 and bm % 8 == 0
        want = []
        for i in range(nseg):
            a, b = int(seg[i]), int(seg[i + 1])
            for r0 in range(a, b, bm):
                want.append((r0, min(bm, b - r0), i, 0))
        assert n == len(want)
        got = plan.buf[4:4 + 4 * n].cpu().view(-1, 4).tolist()
        assert [tuple(g) for g in got] == want
        # the second list: the same segments cut at the height its header records (96..128 rows)
        off = 4 + 4 * (T // bm + nseg + 1)
        hdr = plan.buf[off:off + 4].tolist()
        bm2 = hdr[3]
        assert 96 <= bm2 <= 128 and bm2 % 8 == 0
        want2 = []
        for i in range(nseg):
            a, b = int(seg[i]), int(seg[i + 1])
            for r0 in range(a, b, bm2):
                want2.append((r0, min(bm2, b - r0), i, 0))
        assert hdr[0] == len(want2) and hdr[0] <= hdr[2]
        got2 = plan.buf[off + 4:off + 4 + 4 * hdr[0]].cpu().view(-1, 4).tolist()
        assert [tuple(g) for g in got2] == want2


@pytest.mark.parametrize("seg", [[0, 5, 3], [-1, 4], [0, 4, 11]])
def test_plan_rejects_bad_indptr(seg):
    from loquetier_b200 import ops
    plan = ops.Plan(torch.tensor(seg, dtype=torch.int32, device="cuda"), 10)
    n, rc = plan.status()
    assert n == 0 and rc == 7


# ---------------------------------------------------------------------------
# forward
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rm", [False, True])
@pytest.mark.parametrize("rank", [8, 16, 24, 32, 64, 128])
def test_forward_edge_lengths(dtype, rm, rank):
    from gpu_util import check_forward
    c = _case(100 + rank, EDGE_LENS, 5, 200, 328, rank, dtype, rm)
    check_forward(c)


@pytest.mark.parametrize("h_in,h_out", [(64, 64), (4096, 1024), (1000, 264), (14336, 4096), (4096, 14336)])
def test_forward_shapes(h_in, h_out):
    from gpu_util import check_forward
    c = _case(7, [70, 1, 3, 130, 1, 1, 64], 4, h_in, h_out, 16, torch.bfloat16)
    check_forward(c)
    check_forward(c, indexed=True)


def test_forward_scale_and_accumulate():
    from gpu_util import check_forward
    c = _case(8, [40, 1, 90, 17], 3, 512, 768, 16, torch.bfloat16)
    g = torch.Generator().manual_seed(1)
    y0 = torch.randn((sum(c["lens"]), 768), generator=g).to(torch.bfloat16)
    check_forward(c, scale=[2.0, 0.5, 1.25])
    check_forward(c, scale=[2.0, 0.5, 1.25], indexed=True, accumulate=True, y_init=y0)


def test_rows_outside_segments_untouched_and_deterministic():
    from gpu_util import dev, ptr_table, to_dev
    from loquetier_b200 import ops
    c = to_dev(_case(9, [33, 1, 64], 3, 256, 384, 16, torch.float16))
    T = 110
    x = torch.randn((T, 256), device=dev(), dtype=torch.float16)
    seg = torch.tensor([4, 37, 38, 102], dtype=torch.int32, device=dev())
    plan = ops.Plan(seg, T)
    wa = ptr_table([c["wa_d"][i] for i in c["ids"]])
    wb = ptr_table([c["wb_d"][i] for i in c["ids"]])
    outs = []
    for _ in range(2):
        y = torch.full((T, 384), 7.0, dtype=torch.float16, device=dev())
        v = torch.full((T, 16), 3.0, dtype=torch.float16, device=dev())
        ops.fwd(y, x, v, wa, wb, plan, 16)
        outs.append((y.clone(), v.clone()))
    torch.cuda.synchronize()
    y, v = outs[0]
    assert (y[:4] == 7).all() and (y[102:] == 7).all() and (v[:4] == 3).all() and (v[102:] == 3).all()
    assert not (y[4:102] == 7).all()
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


def test_bad_adapter_pointer_is_reported_not_dereferenced():
    from gpu_util import dev
    from loquetier_b200 import ops
    T = 20
    x = torch.randn((T, 64), device=dev(), dtype=torch.bfloat16)
    y = torch.zeros((T, 16), device=dev(), dtype=torch.bfloat16)
    seg = torch.tensor([0, 20], dtype=torch.int32, device=dev())
    plan = ops.Plan(seg, T)
    ops.gemm(y, x, torch.tensor([0], dtype=torch.int64, device=dev()), plan)
    n, rc = plan.status()
    assert rc == 8 and (y == 0).all()
    plan2 = ops.Plan(seg, T)
    w = torch.randn((16, 64), device=dev(), dtype=torch.bfloat16)
    ops.gemm(y, x, torch.tensor([w.data_ptr()], dtype=torch.int64, device=dev()), plan2,
             seg_ids=torch.tensor([3], dtype=torch.int32, device=dev()))
    assert plan2.status()[1] == 9


def test_unsupported_shapes_raise():
    from gpu_util import dev
    from loquetier_b200 import ops
    from loquetier_b200.cabi import SmlmError
    x = torch.zeros((8, 256), device=dev(), dtype=torch.bfloat16)
    y = torch.zeros((8, 256), device=dev(), dtype=torch.bfloat16)
    seg = torch.tensor([0, 8], dtype=torch.int32, device=dev())
    plan = ops.Plan(seg, 8)
    w = torch.zeros(1, dtype=torch.int64, device=dev())
    with pytest.raises(SmlmError, match="No suitable kernel"):
        ops.gemm(y, x, w, plan)
    with pytest.raises(RuntimeError, match="No suitable kernel"):
        ops.gemm(y.float(), x.float(), w, plan)


# ---------------------------------------------------------------------------
# the reference's operator names
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("name", ["addlora_edges_bf16", "addlora_edges_fp16"])
def test_reference_named_op_matches_golden(name):
    from gpu_util import dev, ptr_table
    from loquetier_b200 import kernels
    z = load_npz(name)
    h_in, h_out, r, n_ad, T = (int(v) for v in z["meta"])
    ids, seg = z["ids"].tolist(), z["seg"].tolist()
    wa = [z[f"wa{i}"].to(dev()) for i in range(n_ad)]
    wb = [z[f"wb{i}"].to(dev()) for i in range(n_ad)]
    x = z["x"].to(dev())
    s = torch.tensor(seg, dtype=torch.int32, device=dev())
    tmp = torch.empty(kernels.smlm_forward_cutlass_tmp_size(len(ids)), dtype=torch.uint8, device=dev())
    v = torch.zeros((T, r), dtype=x.dtype, device=dev())
    y = torch.zeros((T, h_out), dtype=x.dtype, device=dev())
    kernels.smlm_forward_cutlass(v, x, ptr_table([wa[i] for i in ids]), s, tmp, False)
    kernels.smlm_forward_cutlass(y, v, ptr_table([wb[i] for i in ids]), s, tmp, False)
    assert_close(y[seg[0]:seg[-1]], z["y"], what="y vs reference golden")
    assert (y[:seg[0]] == 0).all() and (y[seg[-1]:] == 0).all()
    with pytest.raises(RuntimeError, match="CHECK_EQ"):
        kernels.smlm_forward_cutlass(v, x, ptr_table([wa[i] for i in ids]), s, tmp[:-1], False)
    with pytest.raises(RuntimeError, match="must be contiguous"):
        kernels.smlm_forward_cutlass(v, x.t(), ptr_table([wa[i] for i in ids]), s, tmp, False)


# ---------------------------------------------------------------------------
# backward
# ---------------------------------------------------------------------------

def _run_bwd(c, part, scale=None, grad_fp32=False, accumulate=False):
    from gpu_util import dev, ptr_table, to_dev
    from loquetier_b200 import ops
    d = to_dev(c)
    npart = len(part) - 1
    tl = part[-1]
    rm = c["is_row_major"]
    pd = torch.tensor(part, dtype=torch.int32, device=dev())
    plan = ops.Plan(pd, tl)
    # v from the forward over the partitions
    wa_t, wb_t = ptr_table(d["wa_d"][:npart]), ptr_table(d["wb_d"][:npart])
    T = d["x"].shape[0]
    y = torch.zeros((T, c["h_out"]), dtype=c["dtype"], device=dev())
    v = torch.zeros((T, c["rank"]), dtype=c["dtype"], device=dev())
    ops.fwd(y, d["x"], v, wa_t, wb_t, plan, c["rank"], is_row_major=rm)
    gdt = torch.float32 if grad_fp32 else c["dtype"]
    init = 1.0 if accumulate else 0.0
    dA = [torch.full_like(w, init, dtype=gdt) for w in d["wa_d"][:npart]]
    dB = [torch.full_like(w, init, dtype=gdt) for w in d["wb_d"][:npart]]
    dx = torch.zeros((T, c["h_in"]), dtype=c["dtype"], device=dev())
    dv = torch.zeros((tl, c["rank"]), dtype=c["dtype"], device=dev())
    sc = None if scale is None else torch.tensor(scale, dtype=torch.float32, device=dev())
    ops.bwd(dx, ptr_table(dA), ptr_table(dB), dv, d["go"], d["x"], v, wa_t, wb_t, plan, c["rank"],
            is_row_major=rm, part_scale=sc, accumulate_grads=accumulate, grad_fp32=grad_fp32)
    torch.cuda.synchronize()
    plan.raise_if_failed()
    return dx.cpu(), [g.cpu() for g in dA], [g.cpu() for g in dB]


def _oracle_bwd(c, part, scale=None):
    npart = len(part) - 1
    go = c["go"].to(torch.float32).clone()
    if scale is not None:
        for p in range(npart):
            go[part[p]:part[p + 1]] *= scale[p]
    gx, grads = O.add_lora_backward(go.to(torch.float32), c["x"].to(torch.float32),
                                    [w.to(torch.float32) for w in c["wa"][:npart]],
                                    [w.to(torch.float32) for w in c["wb"][:npart]], part,
                                    is_row_major=c["is_row_major"], round_mid=False)
    return gx, grads[0::2], grads[1::2]


def _grad_close(got, want, what):
    # gradients are sums over up to thousands of tokens: scale the absolute
    # tolerance with the magnitude of the result
    s = max(1.0, float(want.abs().max()))
    assert_close(got, want, rtol=1e-2, atol=1e-2 * s, what=what)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rm", [False, True])
@pytest.mark.parametrize("rank", [8, 16, 64])
def test_backward_vs_oracle(dtype, rm, rank):
    part = [0, 33, 33, 130, 131, 300]
    c = _case(200 + rank, [310], 5, 264, 200, rank, dtype, rm, ids=[0])
    dx, dA, dB = _run_bwd(c, part)
    gx, gA, gB = _oracle_bwd(c, part)
    _grad_close(dx[:300], gx[:300], "dX")
    assert (dx[300:] == 0).all()
    for p in range(5):
        _grad_close(dA[p], gA[p], f"dA{p}")
        _grad_close(dB[p], gB[p], f"dB{p}")


def test_backward_scale_fp32_accumulate():
    part = [0, 100, 257]
    c = _case(300, [257], 2, 512, 320, 16, torch.bfloat16, False, ids=[0])
    dx, dA, dB = _run_bwd(c, part, scale=[2.0, 0.5], grad_fp32=True, accumulate=True)
    gx, gA, gB = _oracle_bwd(c, part, scale=[2.0, 0.5])
    _grad_close(dx, gx, "dX")
    for p in range(2):
        assert dA[p].dtype == torch.float32
        _grad_close(dA[p] - 1.0, gA[p], f"dA{p}")
        _grad_close(dB[p] - 1.0, gB[p], f"dB{p}")


@pytest.mark.parametrize("name", ["bwd_math_bf16", "bwd_math_fp16"])
def test_backward_matches_reference_golden(name):
    """The reference's own backward (math layout) on its own inputs."""
    z = load_npz(name)
    h_in, h_out, r, npart, T = (int(v) for v in z["meta"])
    part = z["part"].tolist()
    c = dict(x=z["x"], go=z["go"], wa=[z[f"wa{p}"] for p in range(npart)],
             wb=[z[f"wb{p}"] for p in range(npart)], seg=[0, T], ids=[0], lens=[T], h_in=h_in, h_out=h_out,
             rank=r, dtype=z["dtype"], is_row_major=True)
    dx, dA, dB = _run_bwd(c, part)
    _grad_close(dx, z["gx"], "dX")
    for p in range(npart):
        _grad_close(dA[p], z[f"dA{p}"], f"dA{p}")
        _grad_close(dB[p], z[f"dB{p}"], f"dB{p}")


def test_backward_deterministic():
    part = [0, 700, 1500]
    c = _case(301, [1500], 2, 1024, 512, 16, torch.bfloat16, False, ids=[0])
    a = _run_bwd(c, part)
    b = _run_bwd(c, part)
    assert torch.equal(a[0], b[0])
    for g1, g2 in zip(a[1] + a[2], b[1] + b[2]):
        assert torch.equal(g1, g2)


def test_independent_launches_match_serial_ones():
    """Launches marked independent may overlap with their predecessor; results must be
    the same bits as when every launch waits for the one before."""
    from gpu_util import dev, ptr_table, to_dev
    from loquetier_b200 import ops
    cases = [to_dev(_case(400 + i, [700, 64, 3, 1, 1200, 33], 6, 1024, 2048 if i % 2 else 512, 16, torch.bfloat16))
             for i in range(4)]
    T = cases[0]["x"].shape[0]
    plan = ops.Plan(cases[0]["seg_d"], T)
    part = torch.tensor([0, 700, 764], dtype=torch.int32, device=dev())
    pplan = ops.Plan(part, 764)
    tabs = [(ptr_table(c["wa_d"]), ptr_table(c["wb_d"])) for c in cases]
    outs = {}
    for mode in (False, True):
        ys, vs, dxs, dvs = [], [], [], []
        for i, c in enumerate(cases):
            y = torch.zeros((T, c["h_out"]), dtype=torch.bfloat16, device=dev())
            v = torch.zeros((T, 16), dtype=torch.bfloat16, device=dev())
            ops.fwd(y, c["x"], v, tabs[i][0], tabs[i][1], plan, 16, seg_ids=c["ids_d"], independent=mode and i > 0)
            ys.append(y); vs.append(v)
        for i, c in enumerate(cases):
            dx = torch.zeros((T, c["h_in"]), dtype=torch.bfloat16, device=dev())
            dv = torch.zeros((764, 16), dtype=torch.bfloat16, device=dev())
            ops.bwd_dx(dx, dv, c["go"], tabs[i][0], tabs[i][1], pplan, 16, part_ids=c["ids_d"][:2].contiguous(),
                       independent=mode)
            dxs.append(dx); dvs.append(dv)
        torch.cuda.synchronize()
        plan.raise_if_failed(); pplan.raise_if_failed()
        outs[mode] = ys + vs + dxs + dvs
    for a, b in zip(outs[False], outs[True]):
        assert torch.equal(a, b)
    assert float(outs[True][0].abs().max()) > 0


def test_device_segment_merge_is_bit_exact():
    """Integer bookkeeping on the device against the oracle's merge (and through it the reference's)."""
    from loquetier_b200.segments import merge_segments_device
    rng = np.random.default_rng(5)
    for n in (1, 2, 37, 1024, 1025, 3000):
        ids = rng.integers(0, 6, size=n)
        if n > 40:
            ids = np.sort(ids) if n % 2 else ids       # long runs and short runs
        lens = rng.integers(1, 50, size=n)
        want_ids, want_lens, want_seg = O.merge_segments(list(zip(ids.tolist(), lens.tolist())))
        si, sl, sp, ns = merge_segments_device(torch.tensor(ids, dtype=torch.int32, device="cuda"),
                                               torch.tensor(lens, dtype=torch.int32, device="cuda"))
        k = int(ns.item())
        assert k == len(want_ids)
        assert si[:k].tolist() == want_ids and sl[:k].tolist() == want_lens and sp[:k + 1].tolist() == want_seg
        # the padding is made of empty segments
        assert (sl[k:] == 0).all() and (sp[k:] == want_seg[-1]).all()
    # the padded arrays drive the kernels directly
    from gpu_util import dev, ptr_table, to_dev
    from loquetier_b200 import ops
    c = _case(9, [5, 40, 3, 70], 3, 256, 384, 16, torch.bfloat16, ids=[1, 1, 0, 2])
    d = to_dev(c)
    si, sl, sp, ns = merge_segments_device(torch.tensor([1, 1, 0, 2], dtype=torch.int32, device="cuda"),
                                           torch.tensor([5, 40, 3, 70], dtype=torch.int32, device="cuda"))
    T = 118
    plan = ops.Plan(sp, T)
    y = torch.zeros((T, 384), dtype=torch.bfloat16, device=dev())
    v = torch.zeros((T, 16), dtype=torch.bfloat16, device=dev())
    ops.fwd(y, d["x"], v, ptr_table(d["wa_d"]), ptr_table(d["wb_d"]), plan, 16, seg_ids=si)
    torch.cuda.synchronize()
    plan.raise_if_failed()
    from gpu_util import oracle_forward
    y_ref, _ = oracle_forward(c)
    assert_close(y, y_ref, what="y through device-merged segments")


def test_independent_promise_covers_every_open_kernel():
    """A chain D (dependent), I (independent, unrelated), C: C consumes D's output, so C has to be
    launched with independent = 0 although an unrelated independent launch sits between the two - an
    independent launch may run alongside ALL kernels since the last dependent one.  Launched that way
    the chain gives the oracle's answer."""
    from gpu_util import dev, ptr_table, to_dev
    from loquetier_b200 import ops
    lens, ids = [200, 3, 130, 64], [1, 0, 2, 1]
    c = to_dev(O.make_case(77, lens, ids, 3, 512, 512, 16, torch.bfloat16))
    T = sum(lens)
    wa = ptr_table([c["wa_d"][i] for i in ids])
    wb = ptr_table([c["wb_d"][i] for i in ids])
    plan = ops.Plan(c["seg_d"], T)
    y_d = torch.zeros((T, 512), dtype=torch.bfloat16, device=dev())
    y_i = torch.zeros_like(y_d)
    y_c = torch.zeros_like(y_d)
    v = [torch.zeros((T, 16), dtype=torch.bfloat16, device=dev()) for _ in range(3)]
    other = torch.randn((T, 512), device=dev()).to(torch.bfloat16)
    ops.fwd(y_d, c["x"], v[0], wa, wb, plan, 16)                              # D: writes y_d
    ops.fwd(y_i, other, v[1], wa, wb, plan, 16, independent=True)             # I: touches nothing of D or C
    ops.fwd(y_c, y_d, v[2], wa, wb, plan, 16, independent=False)              # C: reads y_d
    torch.cuda.synchronize()
    plan.raise_if_failed()
    want_d, _ = O.add_lora_forward((T, 512), c["x"].cpu(), [c["wa"][i] for i in ids], [c["wb"][i] for i in ids],
                                   c["seg"], 16)
    want_c, _ = O.add_lora_forward((T, 512), y_d.cpu(), [c["wa"][i] for i in ids], [c["wb"][i] for i in ids],
                                   c["seg"], 16)
    assert_close(y_d, want_d, what="D")
    assert_close(y_c, want_c, what="C reads D's output")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rank", [16, 64])
def test_backward_literal_tolerance_at_reference_rounding_points(dtype, rank):
    """dX, dA and dB against the oracle evaluated the way the reference evaluates them - dV and the
    recomputed v rounded to the storage type (round_mid=True).  dX and the gradients of short partitions
    meet the literal rtol = atol = 1e-2 element by element.  A long partition's dA / dB are sums over its
    tokens of products with an intermediate that both sides round on their own; where the two roundings
    differ by one unit a gradient element moves by ulp(intermediate) * |other operand|, which is more than
    0.01 for small elements: those are held to atol * max|want| and at most 1 % of the elements may lie
    outside the literal tolerance.  The observed figures are printed."""
    part = [0, 1, 18, 1518, 1519, 1627]
    c = _case(500 + rank, [1700], 5, 512, 384, rank, dtype, False, ids=[0])
    dx, dA, dB = _run_bwd(c, part)
    npart = len(part) - 1
    gx, grads = O.add_lora_backward(c["go"], c["x"], c["wa"][:npart], c["wb"][:npart], part, round_mid=True)
    assert_close(dx[:part[-1]], gx[:part[-1]], rtol=1e-2, atol=1e-2, what="dX")
    worst, share = 0.0, 0.0
    for p in range(npart):
        n = part[p + 1] - part[p]
        for got, want, nm in ((dA[p], grads[2 * p], "dA"), (dB[p], grads[2 * p + 1], "dB")):
            g, w = got.float(), want.float()
            err = (g - w).abs()
            if n <= 32:
                assert_close(got, want, rtol=1e-2, atol=1e-2, what=f"{nm}{p} ({n} rows)")
            else:
                assert_close(got, want, rtol=1e-2, atol=1e-2 * max(1.0, float(w.abs().max())), what=f"{nm}{p}")
                out = float((err > 1e-2 + 1e-2 * w.abs()).float().mean())
                assert out < 1e-2, f"{nm}{p}: {out:.2%} outside the literal tolerance"
                share = max(share, out)
            worst = max(worst, float(err.max()) / max(float(w.abs().max()), 1e-30))
    assert worst < 1e-2
    print(f"observed max|err|/max|ref| over dA, dB: {worst:.3e}; largest share outside the literal tolerance: {share:.3e}")


def test_plan_pair_builds_the_same_two_plans_in_one_launch():
    from loquetier_b200 import ops
    rng = np.random.default_rng(3)
    lens = [int(v) for v in rng.integers(0, 90, size=200)]
    ids = torch.tensor(rng.integers(0, 16, size=200), dtype=torch.int32, device="cuda")
    seg = torch.tensor(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32), device="cuda")
    T = int(seg[-1])
    part = seg[:9].contiguous()
    tl = int(part[-1])
    a0 = ops.Plan(seg, T, seg_ids=ids, n_table=16)
    b0 = ops.Plan(part, tl)
    a1, b1 = ops.plan_pair(seg, T, part, tl, seg_ids_a=ids, n_table_a=16)
    torch.cuda.synchronize()
    assert a1.status() == a0.status() and b1.status() == b0.status() and a0.status()[1] == 0

    def used(p):   # header + the pieces that were written
        n = p.status()[0]
        return p.buf[:4 + 4 * n]
    assert torch.equal(used(a0), used(a1)) and torch.equal(used(b0), used(b1))


@pytest.mark.parametrize("n", [1, 17, 256, 257, 1000, 4096])
def test_adapter_groups_from_pointers_are_first_occurrences(n):
    """ids[i] = first j with w[j] == w[i]: integer work, bit-exact against the host loop; several tiles and CTAs."""
    from loquetier_b200.cabi import check, lib
    rng = np.random.default_rng(n)
    vals = rng.integers(1, max(2, n // 3 + 1), size=n).astype(np.int64) * 4096   # many repeats
    w = torch.tensor(vals, dtype=torch.int64, device="cuda:0")
    ids = torch.full((n,), -1, dtype=torch.int32, device="cuda:0")
    check(lib.smlm_b200_group_ids_from_pointers(w.data_ptr(), n, ids.data_ptr(),
                                                torch.cuda.current_stream().cuda_stream), "group ids")
    torch.cuda.synchronize()
    first = {}
    want = [first.setdefault(int(v), i) for i, v in enumerate(vals)]
    assert ids.cpu().tolist() == want


def test_cached_workspace_survives_alternating_shapes():
    """The cached weight-gradient workspace is used for one shape, then another whose tickets reach into what the
    first one parked, then the first again: every result must still match.  Long partitions, so that partial
    sums really are parked (a partition spread over several CTAs)."""
    shapes = [(1600, [0, 900, 1600], 2048, 256, 16), (1900, [0, 100, 1900], 256, 4096, 16),
              (1600, [0, 900, 1600], 2048, 256, 16), (700, [0, 700], 512, 512, 64)]
    for k, (T, part, h_in, h_out, rank) in enumerate(shapes * 2):
        c = _case(500 + k % len(shapes), [T], len(part) - 1, h_in, h_out, rank, torch.bfloat16, False, ids=[0])
        dx, dA, dB = _run_bwd(c, part)
        gx, gA, gB = _oracle_bwd(c, part)
        _grad_close(dx, gx, f"dX, call {k}")
        for p in range(len(part) - 1):
            _grad_close(dA[p], gA[p], f"dA{p}, call {k}")
            _grad_close(dB[p], gB[p], f"dB{p}, call {k}")


@pytest.mark.parametrize("seed", list(range(16)))
def test_forward_and_backward_random_shapes(seed):
    """Seeded random batches: segment lengths (empty, single-token, long), ranks 8..128, hidden sizes that are
    multiples of 8 but of nothing larger, both layouts, both storage types, pointer-per-segment and adapter-table
    calls; forward and backward against the oracle."""
    from gpu_util import check_forward
    rng = np.random.default_rng(7000 + seed)
    rank = int(rng.choice([8, 16, 24, 32, 40, 64, 96, 128]))
    h_in = int(rng.integers(4, 300)) * 8
    h_out = int(rng.integers(4, 300)) * 8
    dtype = torch.bfloat16 if seed % 2 == 0 else torch.float16
    rm = bool(rng.integers(0, 2))
    nseg = int(rng.integers(1, 24))
    kinds = rng.integers(0, 4, size=nseg)
    lens = [0 if k == 0 else 1 if k == 1 else int(rng.integers(2, 40)) if k == 2 else int(rng.integers(40, 400))
            for k in kinds]
    if sum(lens) == 0:
        lens[0] = 77
    n_ad = int(rng.integers(1, 7))
    c = _case(7100 + seed, lens, n_ad, h_in, h_out, rank, dtype, rm)
    check_forward(c)
    check_forward(c, indexed=True)
    # backward over the first few segments as train partitions (pointer tables per partition)
    npart = int(rng.integers(1, min(nseg, n_ad) + 1))
    part = [0]
    for n in lens[:npart]:
        part.append(part[-1] + n)
    if part[-1] == 0:
        return
    cb = _case(7200 + seed, [sum(lens)], max(npart, 1), h_in, h_out, rank, dtype, rm, ids=[0])
    dx, dA, dB = _run_bwd(cb, part)
    gx, gA, gB = _oracle_bwd(cb, part)
    _grad_close(dx[:part[-1]], gx[:part[-1]], f"dX seed {seed}")
    for p in range(npart):
        _grad_close(dA[p], gA[p], f"dA{p} seed {seed}")
        _grad_close(dB[p], gB[p], f"dB{p} seed {seed}")


@pytest.mark.parametrize("rank,rm", [(8, False), (16, True), (16, False), (32, True)])
def test_grouped_plan_hidden_size_ending_in_half_a_step(rank, rm):
    """Gathered rows of short segments with a hidden size of 16k + 8 and more column steps than ring
    stages: the last 16-column step of a row reads 8 columns past the hidden size, which must be zeros
    although the stage held a full step before."""
    from gpu_util import check_forward
    lens = [1, 3, 1, 2, 1, 1, 5, 1, 40, 1, 1, 2]
    c = _case(812, lens, 3, 2056 + 1024, 136, rank, torch.bfloat16, rm)
    check_forward(c, indexed=True)
    check_forward(c)
