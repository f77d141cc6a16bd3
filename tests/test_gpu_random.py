"""Seeded random batches through every entry point of the path, each against its CPU oracle: the fused
forward with its options (scale, accumulate, adapter table, grouped plan, rows outside the segments),
the backward with its options (partition scale, fp32 gradients, accumulation), the single operator
call in both directions (including decode batches with duplicated weight pointers, which take the
grouped plan), several projections per launch, RMSNorm, and the key-value cache writers.  The shapes
are drawn, not chosen: hidden sizes are multiples of 8 and of nothing larger, segments are empty,
one token, short or long side by side.  SMLM_RANDOM_SEEDS=k runs k times as many seeds."""
import os

import numpy as np
import pytest
import torch

from helpers import assert_close
from oracle import attention_oracle as A
from oracle import smlm_oracle as O

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
RANKS = [8, 16, 24, 32, 40, 64, 96, 128]
MORE = max(1, int(os.environ.get("SMLM_RANDOM_SEEDS", "1")))   # multiplies the number of seeds of every test


def _lens(rng, nseg, long_max=400):
    kinds = rng.integers(0, 4, size=nseg)
    lens = [0 if k == 0 else 1 if k == 1 else int(rng.integers(2, 40)) if k == 2 else int(rng.integers(40, long_max))
            for k in kinds]
    if sum(lens) == 0:
        lens[int(rng.integers(0, nseg))] = int(rng.integers(1, 100))
    return lens


def _draw(seed, nseg_max=24, h_max=300):
    rng = np.random.default_rng(seed)
    rank = int(rng.choice(RANKS))
    h_in = int(rng.integers(4, h_max)) * 8
    h_out = int(rng.integers(4, h_max)) * 8
    dtype = torch.bfloat16 if rng.integers(0, 2) else torch.float16
    rm = bool(rng.integers(0, 2))
    nseg = int(rng.integers(1, nseg_max))
    lens = _lens(rng, nseg)
    n_ad = int(rng.integers(1, 7))
    ids = [int(i) for i in rng.integers(0, n_ad, size=nseg)]
    return rng, rank, h_in, h_out, dtype, rm, lens, n_ad, ids


def _grad_close(got, want, what):
    s = max(1.0, float(want.abs().max()))
    assert_close(got, want, rtol=1e-2, atol=1e-2 * s, what=what)


@pytest.mark.parametrize("seed", list(range(16 * MORE)))
def test_forward_options(seed):
    from gpu_util import check_forward, oracle_forward, run_forward
    rng, rank, h_in, h_out, dtype, rm, lens, n_ad, ids = _draw(9000 + seed)
    c = O.make_case(9000 + seed, lens, ids, n_ad, h_in, h_out, rank, dtype, is_row_major=rm)
    # scales: powers of two (folded into the intermediate for bf16), others, and one.  (Larger ones only
    # multiply the one-ulp differences of the rounded intermediate past the absolute tolerance.)
    scale = [float(rng.choice([1.0, 2.0, 0.5, 1.25, 4.0, 3.0])) for _ in range(n_ad)]
    g = torch.Generator().manual_seed(seed)
    y0 = torch.randn((sum(lens), h_out), generator=g).to(dtype)
    check_forward(c, scale=scale)
    check_forward(c, scale=scale, indexed=True)
    # y += product: the product is rounded to the storage type before it meets y, as in the reference
    # (y += scale * lora_out on 16-bit tensors), so where the two cancel the sum carries the operands'
    # rounding: the bound adds one ulp of the larger operand to the literal tolerance
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    for kw in (dict(scale=scale, indexed=True, grouped=False), dict(), dict(indexed=True)):
        y, v = run_forward(c, accumulate=True, y_init=y0, **kw)
        y_ref, v_ref = oracle_forward(c, scale=kw.get("scale"), y_init=y0)
        assert_close(v, v_ref, what="v")
        y, y_ref, y032 = y.float(), y_ref.float(), y0.float()
        bound = 1e-2 + 1e-2 * y_ref.abs() + ulp * torch.maximum(y032.abs(), (y_ref - y032).abs())
        bad = (y - y_ref).abs() > bound
        assert not bool(bad.any()), f"y (accumulate, {kw}): {int(bad.sum())} outside, max err {float((y - y_ref).abs().max())}"


@pytest.mark.parametrize("seed", list(range(12 * MORE)))
def test_forward_rows_outside_the_segments(seed):
    """The segments cover a window of the batch: rows before and after keep what they held, in y and v."""
    from gpu_util import ptr_table, to_dev
    from loquetier_b200 import ops
    rng, rank, h_in, h_out, dtype, rm, lens, n_ad, ids = _draw(9100 + seed)
    lead, trail = int(rng.integers(0, 70)), int(rng.integers(0, 70))
    c = O.make_case(9100 + seed, [lead] + lens + [trail], [0] + ids + [0], n_ad, h_in, h_out, rank, dtype,
                    is_row_major=rm)
    d = to_dev(c)
    T = sum(lens) + lead + trail
    seg = c["seg"][1:-1]
    plan = ops.Plan(torch.tensor(seg, dtype=torch.int32, device=DEV), T)
    y = torch.full((T, h_out), 7.0, dtype=dtype, device=DEV)
    v = torch.full((T, rank), 3.0, dtype=dtype, device=DEV)
    ops.fwd(y, d["x"], v, ptr_table([d["wa_d"][i] for i in ids]), ptr_table([d["wb_d"][i] for i in ids]), plan, rank,
            is_row_major=rm)
    torch.cuda.synchronize()
    plan.raise_if_failed()
    y_ref, v_ref = O.add_lora_forward((T, h_out), c["x"], [c["wa"][i] for i in [0] + ids + [0]],
                                      [c["wb"][i] for i in [0] + ids + [0]], c["seg"], rank, is_row_major=rm,
                                      round_v=True)
    a, b = lead, T - trail
    assert bool((y[:a] == 7).all()) and bool((y[b:] == 7).all()) and bool((v[:a] == 3).all()) and bool((v[b:] == 3).all())
    assert_close(v[a:b].cpu(), v_ref[a:b], what="v")
    assert_close(y[a:b].cpu(), y_ref[a:b].to(torch.float32), what="y")


@pytest.mark.parametrize("seed", list(range(16 * MORE)))
def test_backward_options(seed):
    from gpu_util import ptr_table, to_dev
    from loquetier_b200 import ops
    rng, rank, h_in, h_out, dtype, rm, lens, n_ad, ids = _draw(9200 + seed, nseg_max=8)
    npart = len(lens)
    part = [0] + [int(s) for s in np.cumsum(lens)]
    tl = part[-1]
    extra = int(rng.integers(0, 50))       # inference rows after the train partitions
    c = O.make_case(9200 + seed, [tl + extra], [0], npart, h_in, h_out, rank, dtype, is_row_major=rm)
    scale = None if rng.integers(0, 3) == 0 else [float(rng.choice([1.0, 2.0, 0.5, 1.5])) for _ in range(npart)]
    fp32 = bool(rng.integers(0, 2))
    acc = bool(rng.integers(0, 2))
    d = to_dev(c)
    plan = ops.Plan(torch.tensor(part, dtype=torch.int32, device=DEV), tl)
    wa_t, wb_t = ptr_table(d["wa_d"]), ptr_table(d["wb_d"])
    T = tl + extra
    y = torch.zeros((T, h_out), dtype=dtype, device=DEV)
    v = torch.zeros((T, rank), dtype=dtype, device=DEV)
    ops.fwd(y, d["x"], v, wa_t, wb_t, plan, rank, is_row_major=rm)
    gdt = torch.float32 if fp32 else dtype
    init = 1.0 if acc else float("nan")      # without accumulation nothing of the old content may survive
    dA = [torch.full_like(w, init, dtype=gdt) for w in d["wa_d"]]
    dB = [torch.full_like(w, init, dtype=gdt) for w in d["wb_d"]]
    dx = torch.full((T, h_in), 5.0, dtype=dtype, device=DEV)
    dv = torch.zeros((tl, rank), dtype=dtype, device=DEV)
    sc = None if scale is None else torch.tensor(scale, dtype=torch.float32, device=DEV)
    ops.bwd(dx, ptr_table(dA), ptr_table(dB), dv, d["go"], d["x"], v, wa_t, wb_t, plan, rank, is_row_major=rm,
            part_scale=sc, accumulate_grads=acc, grad_fp32=fp32)
    torch.cuda.synchronize()
    plan.raise_if_failed()
    go = c["go"].to(torch.float32).clone()
    if scale is not None:
        for p in range(npart):
            go[part[p]:part[p + 1]] *= scale[p]
    gx, grads = O.add_lora_backward(go, c["x"].to(torch.float32), [w.to(torch.float32) for w in c["wa"]],
                                    [w.to(torch.float32) for w in c["wb"]], part, is_row_major=rm, round_mid=False)
    _grad_close(dx[:tl].cpu(), gx[:tl], "dX")
    assert bool((dx[tl:] == 5).all()), "dX rows past the train partitions were written"
    for p in range(npart):
        ga, gb = dA[p].cpu().float(), dB[p].cpu().float()
        if lens[p] == 0 and not acc:
            # an empty partition has a zero gradient, written as such
            assert bool((ga == 0).all()) and bool((gb == 0).all()), f"empty partition {p}"
            continue
        off = 1.0 if acc else 0.0
        _grad_close(ga - off, grads[2 * p], f"dA{p}")
        _grad_close(gb - off, grads[2 * p + 1], f"dB{p}")


def _operator_case(seed, decode):
    rng = np.random.default_rng(seed)
    rank = int(rng.choice(RANKS))
    H = int(rng.integers(4, 300)) * 8
    dtype = torch.bfloat16 if rng.integers(0, 2) else torch.float16
    rm = bool(rng.integers(0, 2))
    if decode:
        nseg = int(rng.integers(16, 200))
        lens = [int(x) for x in rng.choice([0, 1, 1, 1, 2, 3, 9], size=nseg)]
        if sum(lens) == 0:
            lens[0] = 1
    else:
        nseg = int(rng.integers(1, 20))
        lens = _lens(rng, nseg)
    n_ad = int(rng.integers(1, 9))
    ids = [int(i) for i in rng.integers(0, n_ad, size=nseg)]
    return rank, H, dtype, rm, lens, n_ad, ids


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("seed", list(range(12 * MORE)))
def test_single_operator_calls(seed, decode):
    """The reference operator, one call per direction: shrink (hidden -> rank), then expand (rank -> hidden) of
    what the shrink wrote.  Decode batches repeat weight pointers in no order."""
    from gpu_util import ptr_table, to_dev
    from loquetier_b200 import kernels
    rank, H, dtype, rm, lens, n_ad, ids = _operator_case(9300 + seed + (100 if decode else 0), decode)
    c = O.make_case(9300 + seed, lens, ids, n_ad, H, H, rank, dtype, is_row_major=rm)
    d = to_dev(c)
    T = sum(lens)
    s = torch.tensor(c["seg"], dtype=torch.int32, device=DEV)
    tmp = torch.empty(kernels.smlm_forward_cutlass_tmp_size(len(lens)), dtype=torch.uint8, device=DEV)
    v = torch.full((T, rank), float("nan"), dtype=dtype, device=DEV)
    y = torch.full((T, H), float("nan"), dtype=dtype, device=DEV)
    kernels.smlm_forward_cutlass(v, d["x"], ptr_table([d["wa_d"][i] for i in ids]), s, tmp, rm)
    kernels.smlm_forward_cutlass(y, v, ptr_table([d["wb_d"][i] for i in ids]), s, tmp, rm)
    torch.cuda.synchronize()
    y_ref, v_ref = O.add_lora_forward((T, H), c["x"], [c["wa"][i] for i in ids], [c["wb"][i] for i in ids], c["seg"],
                                      rank, is_row_major=rm, round_v=True)
    assert_close(v.cpu(), v_ref, what="v")
    assert_close(y.cpu(), y_ref.to(torch.float32), what="y")


@pytest.mark.parametrize("seed", list(range(10 * MORE)))
def test_several_projections_per_launch(seed):
    """One launch per kernel class over projections of different sizes equals the oracle per projection."""
    from gpu_util import ptr_table
    from loquetier_b200 import ops
    rng = np.random.default_rng(9400 + seed)
    rank = int(rng.choice(RANKS))
    dtype = torch.bfloat16 if rng.integers(0, 2) else torch.float16
    rm = bool(rng.integers(0, 2))
    nproj = int(rng.integers(2, 6))
    npart = int(rng.integers(1, 5))
    lens = _lens(rng, npart, long_max=300)
    part = [0] + [int(s) for s in np.cumsum(lens)]
    tl = part[-1]
    plan = ops.Plan(torch.tensor(part, dtype=torch.int32, device=DEV), tl)
    cases, projs, keep = [], [], []
    for j in range(nproj):
        h_in, h_out = int(rng.integers(4, 200)) * 8, int(rng.integers(4, 200)) * 8
        c = O.make_case(9400 + 31 * seed + j, [tl], [0], npart, h_in, h_out, rank, dtype, is_row_major=rm)
        x, go = c["x"].to(DEV), c["go"].to(DEV)
        wa = [w.to(DEV).contiguous() for w in c["wa"]]
        wb = [w.to(DEV).contiguous() for w in c["wb"]]
        p = dict(x=x, go=go, y=torch.zeros((tl, h_out), dtype=dtype, device=DEV),
                 v=torch.zeros((tl, rank), dtype=dtype, device=DEV),
                 dx=torch.zeros((tl, h_in), dtype=dtype, device=DEV),
                 dv=torch.zeros((tl, rank), dtype=dtype, device=DEV),
                 dA=[torch.full_like(w, float("nan")) for w in wa], dB=[torch.full_like(w, float("nan")) for w in wb])
        p["wa_t"], p["wb_t"] = ptr_table(wa), ptr_table(wb)
        p["dA_t"], p["dB_t"] = ptr_table(p["dA"]), ptr_table(p["dB"])
        keep.append((wa, wb))
        cases.append(c)
        projs.append(p)
    mp = ops.ProjSet([dict(x=p["x"], y=p["y"], v=p["v"], go=p["go"], dx=p["dx"], dv=p["dv"], wa=p["wa_t"],
                           wb=p["wb_t"], dA_t=p["dA_t"], dB_t=p["dB_t"]) for p in projs])
    pd = torch.tensor(part, dtype=torch.int32, device=DEV)
    ops.fwd_multi(mp, plan, rank, is_row_major=rm)
    ops.bwd_dx_multi(mp, plan, rank, is_row_major=rm)
    ops.wgrad_pair_multi(mp, pd, plan, rank, is_row_major=rm)
    torch.cuda.synchronize()
    plan.raise_if_failed()
    for c, p in zip(cases, projs):
        y_ref, v_ref = O.add_lora_forward((tl, c["h_out"]), c["x"], c["wa"], c["wb"], part, rank, is_row_major=rm,
                                          round_v=True)
        assert_close(p["v"].cpu(), v_ref, what="v")
        assert_close(p["y"].cpu(), y_ref.to(torch.float32), what="y")
        gx, grads = O.add_lora_backward(c["go"].to(torch.float32), c["x"].to(torch.float32),
                                        [w.to(torch.float32) for w in c["wa"]],
                                        [w.to(torch.float32) for w in c["wb"]], part, is_row_major=rm, round_mid=False)
        _grad_close(p["dx"].cpu(), gx, "dX")
        for q in range(npart):
            if lens[q] == 0:
                assert bool((p["dA"][q] == 0).all()) and bool((p["dB"][q] == 0).all())
                continue
            _grad_close(p["dA"][q].cpu().float(), grads[2 * q], f"dA{q}")
            _grad_close(p["dB"][q].cpu().float(), grads[2 * q + 1], f"dB{q}")


@pytest.mark.parametrize("seed", list(range(12 * MORE)))
def test_rms_norm_random_shapes(seed):
    from loquetier_b200 import ops
    rng = np.random.default_rng(9500 + seed)
    rows = int(rng.choice([1, 2, 7, 33, 150, 1000, 3000]))
    cols = int(rng.integers(1, 2100)) * 8
    dtype = torch.bfloat16 if rng.integers(0, 2) else torch.float16
    g = torch.Generator().manual_seed(9500 + seed)
    x = (torch.randn((rows, cols), generator=g) * 1.5).to(dtype)
    w = (1.0 + 0.1 * torch.randn((cols,), generator=g)).to(dtype)
    go = torch.randn((rows, cols), generator=g).to(dtype)
    xd, wd, gd = x.to(DEV), w.to(DEV), go.to(DEV)
    o = torch.empty_like(xd)
    m = torch.empty((rows, 1), dtype=torch.float32, device=DEV)
    ops.rms_norm(o, m, xd, wd, 1e-6)
    o_ref, m_ref = O.rms_norm_forward(x, w, 1e-6)
    assert torch.allclose(m.cpu(), m_ref, rtol=1e-5, atol=0)
    assert_close(o.cpu(), o_ref, what="out")
    dx = torch.empty_like(xd)
    dw = torch.empty((cols,), dtype=torch.float32, device=DEV)
    ops.rms_norm_bwd(dx, dw, gd, xd, wd, m)
    dx_ref, dw_ref = O.rms_norm_backward(go, x, w, m_ref)
    assert_close(dx.cpu(), dx_ref, what="dx")
    s = max(1.0, float(dw_ref.abs().max()))
    assert_close(dw.cpu(), dw_ref, rtol=1e-2, atol=1e-2 * s, what="dw")


@pytest.mark.parametrize("seed", list(range(10 * MORE)))
def test_cache_writers_random_shapes(seed):
    """append_kv and init_kv over random page tables: every page bit-exact against the oracle, so nothing
    else was touched either."""
    from loquetier_b200 import kvcache
    rng = np.random.default_rng(9600 + seed)
    P = int(rng.choice([8, 16, 32]))
    N = int(rng.choice([1, 2, 4, 8]))
    Lyr = int(rng.integers(1, 4))
    dt = torch.bfloat16 if rng.integers(0, 2) else torch.float16
    B = int(rng.integers(1, 40))
    seqlens = [int(x) for x in rng.integers(1, 6 * P, size=B)]
    pages, indptr, last = A.make_cache(9600 + seed, seqlens, Lyr, N, P, 128, dt)
    pd = [p.to(DEV) for p in pages]
    ptrs = torch.tensor([p.data_ptr() for p in pd], dtype=torch.int64, device=DEV)
    ind = torch.tensor(indptr, dtype=torch.int32, device=DEV)
    lst = torch.tensor(last, dtype=torch.int32, device=DEV)
    g = torch.Generator().manual_seed(seed)
    word = torch.zeros(1, dtype=torch.int32, device=DEV)
    layer = int(rng.integers(0, Lyr))
    k, v = torch.randn((B, N, 128), generator=g).to(dt), torch.randn((B, N, 128), generator=g).to(dt)
    kvcache.append_kv_raw(ptrs, ind, lst, k.to(DEV), v.to(DEV), Lyr, layer, N, P, status_word=word)
    A.append_kv(pages, indptr, last, k, v, layer)
    runs = [int(rng.integers(0, s + 1)) for s in seqlens]
    sind = [0] + [int(s) for s in np.cumsum(runs)]
    n = max(sind[-1], 1)
    k2, v2 = torch.randn((n, N, 128), generator=g).to(dt), torch.randn((n, N, 128), generator=g).to(dt)
    layer2 = int(rng.integers(0, Lyr))
    kvcache.init_kv_raw(ptrs, ind, lst, k2.to(DEV), v2.to(DEV), torch.tensor(sind, dtype=torch.int32, device=DEV), Lyr,
                        layer2, N, P, status_word=word)
    A.init_kv(pages, indptr, last, k2, v2, sind, layer2)
    torch.cuda.synchronize()
    assert int(word.item()) == 0
    for got, want in zip(pd, pages):
        assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("rank", [8, 16, 32, 64, 128])
@pytest.mark.parametrize("h_in,h_out", [(8, 8), (16, 72), (24, 8), (40, 56), (72, 24), (8, 4096), (4096, 8)])
def test_smallest_hidden_sizes(rank, h_in, h_out):
    """Hidden sizes below one column step, one 64-column chunk or one slab, in either direction."""
    from gpu_util import check_forward
    lens = [1, 70, 0, 9, 130]
    part = [0, 1, 71, 71, 80]
    for rm in (False, True):
        c = O.make_case(500 + rank + h_in, lens, [0, 1, 2, 1, 0], 3, h_in, h_out, rank, torch.bfloat16,
                        is_row_major=rm, a_std=1.0 / np.sqrt(max(h_in, 64)))
        check_forward(c)
        check_forward(c, indexed=True)
        from test_gpu_parity import _grad_close as gc, _oracle_bwd, _run_bwd
        cb = O.make_case(600 + rank + h_in, [80], [0], 4, h_in, h_out, rank, torch.bfloat16, is_row_major=rm,
                         a_std=1.0 / np.sqrt(max(h_in, 64)))
        dx, dA, dB = _run_bwd(cb, part)
        gx, gA, gB = _oracle_bwd(cb, part)
        gc(dx, gx, "dX")
        for p in (0, 1, 3):
            gc(dA[p], gA[p], f"dA{p}")
            gc(dB[p], gB[p], f"dB{p}")


@pytest.mark.parametrize("rank", [16, 64])
def test_thousands_of_segments_and_a_long_batch(rank):
    """6000 segments of 0-3 rows (more pieces than any launch of the other tests holds), then 150 000 rows in a
    handful of segments."""
    from gpu_util import check_forward
    rng = np.random.default_rng(77 + rank)
    lens = [int(x) for x in rng.integers(0, 4, size=6000)]
    ids = [int(i) for i in rng.integers(0, 5, size=6000)]
    c = O.make_case(78, lens, ids, 5, 264, 136, rank, torch.bfloat16)
    check_forward(c)
    check_forward(c, indexed=True)
    lens = [70000, 1, 50000, 29999]
    c = O.make_case(79, lens, [0, 1, 1, 0], 2, 72, 64, rank, torch.float16, is_row_major=True)
    check_forward(c)
