"""Grouped plans: short segments (decode tokens) gathered by adapter wherever they sit in the batch.
The plan is bit-exact against a host statement of the same rule; the forward through it matches the CPU
oracle and the forward through an ordinary plan (to rounding: how the warps split the contraction depends
on how many rows a piece has, so the fp32 sums are formed in a different order)."""
import numpy as np
import pytest
import torch

from oracle import smlm_oracle as O

pytestmark = pytest.mark.gpu

SHORT = 8    # segments of at most this many rows are grouped, if their adapter has at least two of them
GROWS = 48   # rows of a gather piece at most


def _case(seed, lens, n_ad, h_in, h_out, rank, dtype, rm=False, ids=None):
    rng = np.random.default_rng(seed)
    ids = list(rng.integers(0, n_ad, size=len(lens))) if ids is None else ids
    return O.make_case(seed, lens, [int(i) for i in ids], n_ad, h_in, h_out, rank, dtype, is_row_major=rm)


def _expected_plan(seg, ids, n_table, bm):
    pieces, rows = [], []
    nseg = len(seg) - 1
    short = [0 < seg[i + 1] - seg[i] <= SHORT and 0 <= ids[i] < n_table for i in range(nseg)]
    per_adapter = {}
    for i in range(nseg):
        if short[i]:
            per_adapter[ids[i]] = per_adapter.get(ids[i], 0) + 1
    short = [short[i] and per_adapter[ids[i]] >= 2 for i in range(nseg)]
    for i in range(nseg):
        if not short[i]:
            for r0 in range(seg[i], seg[i + 1], bm):
                pieces.append((r0, min(bm, seg[i + 1] - r0), i, 0))
    for a in range(n_table):
        mine = [r for i in range(nseg) if short[i] and ids[i] == a for r in range(seg[i], seg[i + 1])]
        for r0 in range(0, len(mine), GROWS):
            pieces.append((len(rows) + r0, min(GROWS, len(mine) - r0), a, 1))
        rows += mine
    return pieces, rows


def test_grouped_plan_is_bit_exact():
    from loquetier_b200 import cabi, ops
    rng = np.random.default_rng(1)
    for trial, (nseg, n_table) in enumerate([(1, 3), (40, 4), (1024, 256), (3000, 64), (2500, 4096), (300, 1)]):
        lens = rng.integers(0, 4, size=nseg)
        big = rng.random(nseg) < 0.05
        lens[big] = rng.integers(5, 300, size=int(big.sum()))
        if trial == 2:
            lens[:] = 1
        seg = np.concatenate([[2], 2 + np.cumsum(lens)]).astype(np.int32)
        ids = rng.integers(0, n_table, size=nseg).astype(np.int32)
        if trial == 1:
            ids[5] = 9  # outside the table: stays an ordinary piece (and the consumer reports it)
        T = int(seg[-1]) + 3
        plan = ops.Plan(torch.tensor(seg, device="cuda"), T, seg_ids=torch.tensor(ids, device="cuda"), n_table=n_table)
        n, rc = plan.status()
        assert rc == 0
        bm = cabi.lib.smlm_b200_piece_rows(T)
        want, rows = _expected_plan([int(v) for v in seg], [int(v) for v in ids], n_table, bm)
        assert n == len(want)
        got = plan.buf[4:4 + 4 * n].cpu().view(-1, 4).tolist()
        assert [tuple(g) for g in got] == want
        cap, tall_cap = int(plan.buf[2]), int(plan.buf[4 + 4 * (int(plan.buf[2]) + 1) + 2])
        off = 4 + 4 * (cap + 1) + 4 + 4 * (tall_cap + 1)
        assert plan.buf[off:off + len(rows)].cpu().tolist() == rows


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rm", [False, True])
@pytest.mark.parametrize("rank", [8, 16, 32, 64])
def test_forward_unsorted_decode_tokens(dtype, rm, rank):
    from gpu_util import check_forward, run_forward
    rng = np.random.default_rng(rank)
    lens = [1] * 150 + [3, 70, 1, 8, 9, 2, 0, 1, 1, 130]
    order = rng.permutation(len(lens))
    lens = [lens[i] for i in order]
    c = _case(700 + rank, lens, 6, 200, 328, rank, dtype, rm)
    y, v = check_forward(c, indexed=True)
    y2, v2 = run_forward(c, indexed=True, grouped=False)
    from helpers import assert_close
    assert_close(v, v2.float(), rtol=4e-3, atol=4e-3, what="v grouped vs ordinary")
    assert_close(y, y2.float(), rtol=4e-3, atol=4e-3, what="y grouped vs ordinary")


def test_forward_c4_like_scale_accumulate_and_single_operator():
    from gpu_util import check_forward, dev, ptr_table, to_dev
    from loquetier_b200 import ops
    c = _case(710, [1] * 300, 40, 1024, 1408, 32, torch.bfloat16)
    g = torch.Generator().manual_seed(3)
    y0 = torch.randn((300, 1408), generator=g).to(torch.bfloat16)
    sc = [float(1 + 0.25 * (i % 4)) for i in range(40)]
    check_forward(c, indexed=True, scale=sc)
    check_forward(c, indexed=True, scale=sc, accumulate=True, y_init=y0)
    # one operator call at a time (shrink alone, expand alone) through the same grouped plan
    d = to_dev(c)
    plan = ops.Plan(d["seg_d"], 300, seg_ids=d["ids_d"], n_table=40)
    v = torch.zeros((300, 32), dtype=torch.bfloat16, device=dev())
    y = torch.zeros((300, 1408), dtype=torch.bfloat16, device=dev())
    ops.gemm(v, d["x"], ptr_table(d["wa_d"]), plan, seg_ids=d["ids_d"])
    ops.gemm(y, v, ptr_table(d["wb_d"]), plan, seg_ids=d["ids_d"])
    torch.cuda.synchronize()
    plan.raise_if_failed()
    y_ref, v_ref = O.add_lora_forward((300, 1408), c["x"], [c["wa"][i] for i in c["ids"]],
                                      [c["wb"][i] for i in c["ids"]], c["seg"], 32, round_v=True)
    from helpers import assert_close
    assert_close(v, v_ref, what="v")
    assert_close(y, y_ref, what="y")


def test_grouped_plan_needs_the_adapter_table_and_is_refused_by_weight_gradients():
    from gpu_util import dev, ptr_table, to_dev
    from loquetier_b200 import cabi, ops
    c = to_dev(_case(720, [1, 1, 40, 1], 3, 256, 256, 16, torch.bfloat16, ids=[0, 0, 1, 0]))
    T = 43
    plan = ops.Plan(c["seg_d"], T, seg_ids=c["ids_d"], n_table=3)
    y = torch.zeros((T, 256), dtype=torch.bfloat16, device=dev())
    v = torch.zeros((T, 16), dtype=torch.bfloat16, device=dev())
    # per-segment pointer tables cannot serve gather pieces: reported, rows of short segments untouched
    ops.fwd(y, c["x"], v, ptr_table([c["wa_d"][i] for i in c["ids"]]), ptr_table([c["wb_d"][i] for i in c["ids"]]),
            plan, 16)
    torch.cuda.synchronize()
    assert plan.status()[1] == 9
    assert (y[:2] == 0).all() and (y[42:] == 0).all() and not (y[2:42] == 0).all()
    # weight gradients on a grouped plan
    plan = ops.Plan(c["seg_d"], T, seg_ids=c["ids_d"], n_table=3)
    dA = [torch.zeros_like(c["wa_d"][0]) for _ in range(4)]
    dB = [torch.zeros_like(c["wb_d"][0]) for _ in range(4)]
    ops.wgrad_pair(ptr_table(dA), ptr_table(dB), v, c["x"], v, c["go"], c["seg_d"], plan, 16)
    torch.cuda.synchronize()
    assert plan.status()[1] == 12
    with pytest.raises(cabi.SmlmError):
        plan.raise_if_failed()


def test_grouped_plan_without_the_flag_is_refused_not_misread():
    from gpu_util import dev, ptr_table, to_dev
    from loquetier_b200 import cabi, ops
    c = to_dev(_case(721, [1, 1, 40, 1], 3, 256, 256, 16, torch.bfloat16, ids=[0, 0, 1, 0]))
    T = 43
    plan = ops.Plan(c["seg_d"], T, seg_ids=c["ids_d"], n_table=3)
    y = torch.zeros((T, 256), dtype=torch.bfloat16, device=dev())
    v = torch.zeros((T, 16), dtype=torch.bfloat16, device=dev())
    wa, wb = ptr_table(c["wa_d"]), ptr_table(c["wb_d"])
    rc = cabi.lib.smlm_b200_fwd(y.data_ptr(), c["x"].data_ptr(), v.data_ptr(), wa.data_ptr(), wb.data_ptr(),
                                c["ids_d"].data_ptr(), None, plan.buf.data_ptr(), 3, T, 4, 256, 256, 16, cabi.SMLM_BF16,
                                0, 0, 0, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert plan.status()[1] == 12
    # the long segment is an ordinary piece and was computed; the gathered rows were left alone
    assert not (y[2:42] == 0).all() and (y[:2] == 0).all() and (y[42:] == 0).all()
