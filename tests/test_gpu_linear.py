"""The LoRA linear and the add_lora autograd function on the GPU, against the
vectors the reference's own MixedLoraLinear produced and against the oracle."""
import numpy as np
import pytest
import torch
from torch import nn

from helpers import assert_close, load_npz
from oracle import smlm_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _build_linear(z, scale_mode, dtype):
    from loquetier_b200.kernel_utils import BatchLenInfo
    from loquetier_b200.mixed_lora import MixedLoraContext, MixedLoraLinear, NamedLoraLayer
    h_in, h_out, r, n_ad, scale = z["meta"]
    h_in, h_out, r, n_ad = int(h_in), int(h_out), int(r), int(n_ad)
    base = nn.Linear(h_in, h_out, bias=False, dtype=dtype, device=DEV)
    with torch.no_grad():
        base.weight.copy_(z["w_base"].to(dtype))
    ads = [NamedLoraLayer(f"a{i}", z[f"wa{i}"].to(DEV).to(dtype).contiguous(),
                          z[f"wb{i}"].to(DEV).to(dtype).contiguous(), nn.Identity(),
                          None if scale < 0 else float(scale)) for i in range(n_ad)]
    ctx = MixedLoraContext()
    lin = MixedLoraLinear(ctx, base, ads, r, dtype, is_scaled=scale < 0)
    lens, ids = z["lens"].tolist(), z["ids"].tolist()
    seg = torch.cumsum(torch.tensor([0] + lens, dtype=torch.int32, device=DEV), 0, dtype=torch.int32)
    blen = BatchLenInfo([], [], 0, [], torch.device(DEV))
    ctx.update(blen, ids, torch.tensor(lens, dtype=torch.int32, device=DEV), seg, [])
    return lin, ctx


@pytest.mark.parametrize("name", ["linear_c1_bf16", "linear_c1_fp16_prescaled", "linear_ragged_bf16"])
@pytest.mark.parametrize("path", ["fused", "reference_ops"])
def test_linear_matches_reference_golden(name, path):
    z = load_npz(name)
    lin, _ = _build_linear(z, None, z["dtype"])
    x = z["x"].to(DEV)
    with torch.no_grad():
        y = lin(x) if path == "fused" else lin.forward_reference_ops(x)
    assert_close(y, z["y"], what=f"{name}/{path}")


def test_linear_c1_fp32_answer_in_16bit():
    """The CPU plumbing configuration (fp32 on the CPU in the reference) run in
    bf16 and fp16 on the GPU against the fp32 answer."""
    z = load_npz("linear_c1_fp32")
    for dt in (torch.bfloat16, torch.float16):
        lin, _ = _build_linear(z, None, dt)
        with torch.no_grad():
            y = lin(z["x"].to(DEV).to(dt))
        assert_close(y, z["y"], rtol=2e-2, atol=2e-2, what=f"c1 {dt}")


@pytest.mark.parametrize("path", ["fused", "reference_ops"])
def test_linear_training_step_vs_oracle(path):
    from loquetier_b200.kernel_utils import BatchLenInfo
    from loquetier_b200.mixed_lora import MixedLoraContext, MixedLoraLinear, NamedLoraLayer
    dt = torch.bfloat16
    h_in, h_out, r, n_ad = 256, 320, 16, 4
    g = torch.Generator().manual_seed(11)
    # rows: two train requests (adapters 2 and 0), one prefill (adapter 1), three decodes
    trains = [(1, 40), (2, 24)]
    lens, ids = [40, 48, 17, 1, 2], [2, 0, 1, 0, 3]
    T = sum(lens)
    x = torch.randn((T, h_in), generator=g).to(dt)
    wbase = (torch.randn((h_out, h_in), generator=g) * 0.02).to(dt)
    was = [(torch.randn((r, h_in), generator=g) / 16).to(dt) for _ in range(n_ad)]
    wbs = [(torch.randn((h_out, r), generator=g) * 0.02).to(dt) for _ in range(n_ad)]
    go = torch.randn((T, h_out), generator=g).to(dt)
    scale = [2.0, 0.5, 1.0, 4.0]

    base = nn.Linear(h_in, h_out, bias=False, dtype=dt, device=DEV)
    with torch.no_grad():
        base.weight.copy_(wbase)
    base.weight.requires_grad_(False)
    ads = [NamedLoraLayer(f"a{i}", was[i].to(DEV).contiguous(), wbs[i].to(DEV).contiguous(), nn.Identity(),
                          scale[i]) for i in range(n_ad)]
    ctx = MixedLoraContext()
    lin = MixedLoraLinear(ctx, base, ads, r, dt)
    lin.set_trainable([2, 0])
    blen = BatchLenInfo(trains, [17], 3, [], torch.device(DEV))
    seg = torch.cumsum(torch.tensor([0] + lens, dtype=torch.int32, device=DEV), 0, dtype=torch.int32)
    ctx.update(blen, ids, torch.tensor(lens, dtype=torch.int32, device=DEV), seg, [2, 0])
    xd = x.to(DEV).requires_grad_(True)
    y = lin(xd) if path == "fused" else lin.forward_reference_ops(xd)
    y.backward(go.to(DEV))
    torch.cuda.synchronize()

    # oracle: fp32 autograd of the same function on the rounded inputs
    x32 = x.float().requires_grad_(True)
    A = [w.float().requires_grad_(True) for w in was]
    B = [w.float().requires_grad_(True) for w in wbs]
    seg_h = np.concatenate([[0], np.cumsum(lens)])
    outs = []
    for i, a in enumerate(ids):
        xs = x32[seg_h[i]:seg_h[i + 1]]
        outs.append(xs @ wbase.float().t() + scale[a] * ((xs @ A[a].t()) @ B[a].t()))
    y32 = torch.cat(outs)
    # only the train rows carry gradient in the reference (grad_x is zero elsewhere,
    # weights of non-train rows are not parameters)
    tl = 88
    (y32[:tl] * go.float()[:tl]).sum().backward()
    assert_close(y, y32.detach(), what="y")
    gx = xd.grad.float().cpu()
    lora_gx = x32.grad[:tl] - go.float()[:tl] @ wbase.float()
    base_gx = (go.float() @ wbase.float())
    want_gx = base_gx.clone()
    want_gx[:tl] += lora_gx
    s = float(want_gx.abs().max())
    assert_close(gx, want_gx, rtol=1e-2, atol=1e-2 * s, what="grad_x")
    for idx in (2, 0):
        ga = lin.get_parameter(f"lora-{idx}-A").grad
        gb = lin.get_parameter(f"lora-{idx}-B").grad
        assert_close(ga, A[idx].grad, rtol=1e-2, atol=1e-2 * float(A[idx].grad.abs().max()), what=f"dA{idx}")
        assert_close(gb, B[idx].grad, rtol=1e-2, atol=1e-2 * float(B[idx].grad.abs().max()), what=f"dB{idx}")


def test_add_lora_signature_and_return_structure():
    from loquetier_b200.kernel_utils import add_lora
    dt = torch.float16
    g = torch.Generator().manual_seed(3)
    T, h_in, h_out, r = 50, 64, 72, 8
    x = torch.randn((T, h_in), generator=g).to(dt).to(DEV).requires_grad_(True)
    wa = [nn.Parameter((torch.randn((r, h_in), generator=g) / 8).to(dt).to(DEV)) for _ in range(2)]
    wb = [nn.Parameter((torch.randn((h_out, r), generator=g) * 0.1).to(dt).to(DEV)) for _ in range(2)]
    s = torch.tensor([0, 20, 50], dtype=torch.int32, device=DEV)
    wa_ptr = torch.tensor([w.data_ptr() for w in wa], dtype=torch.int64, device=DEV)
    wb_ptr = torch.tensor([w.data_ptr() for w in wb], dtype=torch.int64, device=DEV)
    y = add_lora.apply((T, h_out), x, wa_ptr, wb_ptr, s, r, 20, [0, 20], wa[0], wb[0])
    go = torch.randn((T, h_out), generator=g).to(dt).to(DEV)
    y.backward(go)
    torch.cuda.synchronize()
    assert x.grad.shape == x.shape and (x.grad[20:] == 0).all() and not (x.grad[:20] == 0).all()
    assert wa[0].grad is not None and wb[0].grad is not None and wa[1].grad is None
    gx, grads = O.add_lora_backward(go.cpu(), x.detach().cpu(), [wa[0].detach().cpu()], [wb[0].detach().cpu()],
                                    [0, 20], is_row_major=False)
    assert_close(x.grad, gx, what="grad_x")
    assert_close(wa[0].grad, grads[0], rtol=1e-2, atol=1e-2 * float(grads[0].abs().max()) + 1e-2, what="dA")
    assert_close(wb[0].grad, grads[1], rtol=1e-2, atol=1e-2 * float(grads[1].abs().max()) + 1e-2, what="dB")
    # no trainable weights: backward returns None for every input
    x2 = x.detach().clone().requires_grad_(True)
    y2 = add_lora.apply((T, h_out), x2, wa_ptr, wb_ptr, s, r, 0, [])
    y2.sum().backward()
    assert x2.grad is None or (x2.grad == 0).all()


def test_linear_forward_replays_inside_a_cuda_graph():
    """The inference path allocates through torch and launches stream-ordered kernels only, so the
    whole LoRA linear can be captured once and replayed on new inputs."""
    z = load_npz("linear_ragged_bf16")
    lin, _ = _build_linear(z, None, z["dtype"])
    x_static = z["x"].to(DEV).clone()
    with torch.no_grad():
        lin(x_static)                                    # builds the per-step device state
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            lin(x_static)
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            y_static = lin(x_static)
        g.replay()
        torch.cuda.synchronize()
        assert_close(y_static, z["y"], what="replay 1")
        x2 = (z["x"].float() * 0.5).to(z["dtype"])
        x_static.copy_(x2.to(DEV))
        g.replay()
        torch.cuda.synchronize()
        want = lin(x2.to(DEV))
        assert torch.equal(y_static, want)


def test_linear_with_unsorted_decode_tokens_uses_a_grouped_plan():
    """A batch whose decode tokens of one adapter are scattered: the module asks for a grouped plan, and its
    result equals the reference's operator sequence (per-segment pointers, ordinary plan) and the oracle."""
    from loquetier_b200.kernel_utils import BatchLenInfo
    from loquetier_b200.mixed_lora import MixedLoraContext, MixedLoraLinear, NamedLoraLayer
    dt = torch.bfloat16
    h_in, h_out, r, n_ad = 512, 384, 16, 5
    g = torch.Generator().manual_seed(12)
    rng = np.random.default_rng(12)
    lens = [70] + [1] * 40 + [3, 1, 9]
    ids = [4] + [int(v) for v in rng.integers(0, n_ad, size=40)] + [1, 2, 0]
    T = sum(lens)
    x = torch.randn((T, h_in), generator=g).to(dt)
    wbase = (torch.randn((h_out, h_in), generator=g) * 0.02).to(dt)
    was = [(torch.randn((r, h_in), generator=g) / 22).to(dt) for _ in range(n_ad)]
    wbs = [(torch.randn((h_out, r), generator=g) * 0.02).to(dt) for _ in range(n_ad)]
    scale = [2.0, 0.5, 1.0, 4.0, 1.5]
    base = nn.Linear(h_in, h_out, bias=False, dtype=dt, device=DEV)
    with torch.no_grad():
        base.weight.copy_(wbase)
    ads = [NamedLoraLayer(f"a{i}", was[i].to(DEV).contiguous(), wbs[i].to(DEV).contiguous(), nn.Identity(),
                          scale[i]) for i in range(n_ad)]
    ctx = MixedLoraContext()
    lin = MixedLoraLinear(ctx, base, ads, r, dt)
    seg = torch.cumsum(torch.tensor([0] + lens, dtype=torch.int32, device=DEV), 0, dtype=torch.int32)
    ctx.update(BatchLenInfo([], [], 0, [], torch.device(DEV)), ids, torch.tensor(lens, dtype=torch.int32, device=DEV),
               seg, [])
    with torch.no_grad():
        y = lin(x.to(DEV))
        y_ops = lin.forward_reference_ops(x.to(DEV))
    st = ctx.device_state(torch.device(DEV), T)
    assert st["plan"].n_table == max(ids) + 1          # the grouped plan was requested
    y_ref = O.lora_linear_forward(x, wbase, was, wbs, scale, ids, lens, r, dt)
    assert_close(y, y_ref, what="fused, grouped plan")
    assert_close(y_ops, y_ref, what="reference operator sequence")
    assert_close(y, y_ops.float(), rtol=1e-2, atol=1e-2, what="fused vs operator sequence")


def test_add_and_del_adapter_keep_tables_and_results_in_step():
    """add_adapter / del_adapter (mixed_lora.py:106-148 of the reference) followed by a forward: the pointer and
    scale tables follow the adapter list, and a batch that uses the changed list gives the oracle's result."""
    from loquetier_b200.kernel_utils import BatchLenInfo
    from loquetier_b200.mixed_lora import MixedLoraContext, MixedLoraLinear, NamedLoraLayer
    dt = torch.bfloat16
    h_in, h_out, r = 256, 192, 16
    g = torch.Generator().manual_seed(21)
    mk = lambda i, sc: (NamedLoraLayer(f"a{i}", (torch.randn((r, h_in), generator=g) / 16).to(dt).to(DEV).contiguous(),
                                       (torch.randn((h_out, r), generator=g) * 0.02).to(dt).to(DEV).contiguous(),
                                       nn.Identity(), sc))
    ads = [mk(0, 2.0), mk(1, 0.5), mk(2, 1.0)]
    wbase = (torch.randn((h_out, h_in), generator=g) * 0.02).to(dt)
    base = nn.Linear(h_in, h_out, bias=False, dtype=dt, device=DEV)
    with torch.no_grad():
        base.weight.copy_(wbase)
    ctx = MixedLoraContext()
    lin = MixedLoraLinear(ctx, base, list(ads), r, dt)

    def run(lens, ids):
        T = sum(lens)
        x = torch.randn((T, h_in), generator=g).to(dt)
        seg = torch.cumsum(torch.tensor([0] + lens, dtype=torch.int32, device=DEV), 0, dtype=torch.int32)
        ctx.update(BatchLenInfo([], [], 0, [], torch.device(DEV)), ids,
                   torch.tensor(lens, dtype=torch.int32, device=DEV), seg, [])
        with torch.no_grad():
            y = lin(x.to(DEV))
        cur = lin.adapters
        want = O.lora_linear_forward(x, wbase, [a.wa.cpu() for a in cur], [a.wb.cpu() for a in cur],
                                     [a.scaling for a in cur], ids, lens, r, dt)
        assert_close(y, want, what=f"{len(cur)} adapters")

    run([20, 3, 40], [2, 0, 1])
    extra = mk(3, 4.0)
    lin.add_adapter(extra)
    assert lin.wa_ptrs.tolist() == [a.wa.data_ptr() for a in ads + [extra]]
    assert lin.wb_ptrs.tolist() == [a.wb.data_ptr() for a in ads + [extra]]
    assert lin.scaling.tolist() == [2.0, 0.5, 1.0, 4.0] and lin.scaling.dtype == dt
    run([5, 33, 1, 17], [3, 0, 3, 1])            # the new adapter is index 3
    lin.del_adapter(1)                           # indices above it move down by one
    assert [a.adapter_name for a in lin.adapters] == ["a0", "a2", "a3"]
    assert lin.wa_ptrs.tolist() == [ads[0].wa.data_ptr(), ads[2].wa.data_ptr(), extra.wa.data_ptr()]
    assert lin.scaling.tolist() == [2.0, 1.0, 4.0]
    run([9, 64, 2], [2, 1, 0])
    with pytest.raises(AssertionError):
        lin.del_adapter(3)


def test_segments_rebuilt_inside_a_cuda_graph_follow_new_requests():
    """merge of the requests into segments -> plan (grouped) -> fused forward, all captured in ONE graph; between
    replays only the per-request device arrays are rewritten, and each replay gives the oracle's answer for the
    batch those arrays describe."""
    from loquetier_b200 import ops
    from loquetier_b200.cabi import check, lib
    dt = torch.bfloat16
    h_in, h_out, r, n_ad, n_req, T = 256, 320, 16, 4, 12, 96
    g = torch.Generator().manual_seed(31)
    was = [(torch.randn((r, h_in), generator=g) / 16).to(dt) for _ in range(n_ad)]
    wbs = [(torch.randn((h_out, r), generator=g) * 0.02).to(dt) for _ in range(n_ad)]
    wa_d = [w.to(DEV).contiguous() for w in was]
    wb_d = [w.to(DEV).contiguous() for w in wbs]
    tab = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=DEV)
    wa_t, wb_t = tab(wa_d), tab(wb_d)
    req_ids = torch.zeros(n_req, dtype=torch.int32, device=DEV)
    req_len = torch.zeros(n_req, dtype=torch.int32, device=DEV)
    seg_ids = torch.zeros(n_req, dtype=torch.int32, device=DEV)
    seg_len = torch.zeros(n_req, dtype=torch.int32, device=DEV)
    segment = torch.zeros(n_req + 1, dtype=torch.int32, device=DEV)
    nseg = torch.zeros(1, dtype=torch.int32, device=DEV)
    x = torch.zeros((T, h_in), dtype=dt, device=DEV)
    y = torch.zeros((T, h_out), dtype=dt, device=DEV)
    v = torch.zeros((T, r), dtype=dt, device=DEV)
    nbytes = lib.smlm_b200_plan_bytes(T, n_req)
    plan_buf = torch.zeros((nbytes + 3) // 4, dtype=torch.int32, device=DEV)

    def step():
        st = torch.cuda.current_stream().cuda_stream
        check(lib.smlm_b200_merge_segments(req_ids.data_ptr(), req_len.data_ptr(), n_req, seg_ids.data_ptr(),
                                           seg_len.data_ptr(), segment.data_ptr(), nseg.data_ptr(), st), "merge")
        check(lib.smlm_b200_plan_grouped(plan_buf.data_ptr(), nbytes, segment.data_ptr(), seg_ids.data_ptr(), n_req,
                                         n_ad, T, st), "plan")
        check(lib.smlm_b200_fwd(y.data_ptr(), x.data_ptr(), v.data_ptr(), wa_t.data_ptr(), wb_t.data_ptr(),
                                seg_ids.data_ptr(), None, plan_buf.data_ptr(), n_ad, T, n_req, h_in, h_out, r, 1, 0,
                                0, 0, 1, st), "fwd")

    batches = [
        ([1, 1, 0, 2, 2, 2, 3, 0, 1, 3, 0, 0], [10, 6, 1, 20, 1, 1, 30, 1, 1, 1, 1, 1]),     # 74 rows, 9 segments
        ([0, 3, 0, 3, 0, 3, 1, 1, 2, 2, 2, 2], [1, 1, 1, 1, 1, 1, 40, 2, 8, 8, 8, 8]),      # 80 rows, scattered decode
        ([2] * 12, [8] * 12),                                                                  # one segment of 96 rows
    ]
    req_ids.copy_(torch.tensor(batches[0][0], dtype=torch.int32))
    req_len.copy_(torch.tensor(batches[0][1], dtype=torch.int32))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for ids, lens in batches:
        n = sum(lens)
        xb = torch.randn((T, h_in), generator=g).to(dt)
        req_ids.copy_(torch.tensor(ids, dtype=torch.int32))
        req_len.copy_(torch.tensor(lens, dtype=torch.int32))
        x.copy_(xb)
        y.fill_(7.0)
        graph.replay()
        torch.cuda.synchronize()
        mids, mlens, mseg = O.merge_segments(list(zip(ids, lens)))
        assert int(nseg.item()) == len(mids)
        assert seg_ids[:len(mids)].tolist() == mids and segment[:len(mids) + 1].tolist() == mseg
        want, _ = O.add_lora_forward((T, h_out), xb, [was[i] for i in mids], [wbs[i] for i in mids], mseg, r,
                                     fill=7.0)
        assert_close(y[:n], want[:n], what=f"replay with {len(mids)} segments")
        assert bool((y[n:] == 7.0).all()), "rows past the batch must stay untouched"
        hdr = plan_buf[:4].tolist()
        assert hdr[1] == 0, f"plan recorded fault bits {hdr[1]}"


@pytest.mark.parametrize("path", ["fused", "reference_ops"])
@pytest.mark.parametrize("seed", list(range(8)))
def test_linear_training_step_random_batches(seed, path):
    """Seeded random mixes of train partitions, prefill requests and decode tokens through the module and its
    autograd function, against fp32 autograd of the same function on the rounded inputs."""
    from loquetier_b200.kernel_utils import BatchLenInfo
    from loquetier_b200.mixed_lora import MixedLoraContext, MixedLoraLinear, NamedLoraLayer
    rng = np.random.default_rng(4000 + seed)
    dt = torch.bfloat16 if seed % 2 == 0 else torch.float16
    h_in, h_out = int(rng.integers(4, 120)) * 8, int(rng.integers(4, 120)) * 8
    r = int(rng.choice([8, 16, 32, 64]))
    n_ad = int(rng.integers(2, 7))
    ntrain = int(rng.integers(0, min(3, n_ad) + 1))
    train_idx = [int(i) for i in rng.permutation(n_ad)[:ntrain]]
    trains = [(int(rng.integers(1, 4)), int(rng.integers(1, 60))) for _ in range(ntrain)]
    prefills = [int(rng.integers(1, 90)) for _ in range(int(rng.integers(0, 4)))]
    dec = [(int(rng.integers(0, n_ad)), int(rng.integers(1, 6))) for _ in range(int(rng.integers(0, 5)))]
    lens = [c * n for c, n in trains] + prefills + [n for _, n in dec]
    ids = train_idx + [int(rng.integers(0, n_ad)) for _ in prefills] + [a for a, _ in dec]
    if sum(lens) == 0:
        pytest.skip("empty draw")
    T, tl = sum(lens), sum(c * n for c, n in trains)
    g = torch.Generator().manual_seed(4000 + seed)
    x = torch.randn((T, h_in), generator=g).to(dt)
    wbase = (torch.randn((h_out, h_in), generator=g) * 0.02).to(dt)
    was = [(torch.randn((r, h_in), generator=g) / np.sqrt(h_in)).to(dt) for _ in range(n_ad)]
    wbs = [(torch.randn((h_out, r), generator=g) * 0.02).to(dt) for _ in range(n_ad)]
    go = torch.randn((T, h_out), generator=g).to(dt)
    scale = [float(rng.choice([1.0, 2.0, 0.5, 1.5])) for _ in range(n_ad)]

    base = nn.Linear(h_in, h_out, bias=False, dtype=dt, device=DEV)
    with torch.no_grad():
        base.weight.copy_(wbase)
    base.weight.requires_grad_(False)
    ads = [NamedLoraLayer(f"a{i}", was[i].to(DEV).contiguous(), wbs[i].to(DEV).contiguous(), nn.Identity(),
                          scale[i]) for i in range(n_ad)]
    ctx = MixedLoraContext()
    lin = MixedLoraLinear(ctx, base, ads, r, dt)
    lin.set_trainable(train_idx)
    blen = BatchLenInfo(trains, prefills, sum(n for _, n in dec), [], torch.device(DEV))
    seg = torch.cumsum(torch.tensor([0] + lens, dtype=torch.int32, device=DEV), 0, dtype=torch.int32)
    ctx.update(blen, ids, torch.tensor(lens, dtype=torch.int32, device=DEV), seg, train_idx)
    xd = x.to(DEV).requires_grad_(True)
    y = lin(xd) if path == "fused" else lin.forward_reference_ops(xd)
    y.backward(go.to(DEV))
    torch.cuda.synchronize()

    x32 = x.float().requires_grad_(True)
    A = [w.float().requires_grad_(True) for w in was]
    B = [w.float().requires_grad_(True) for w in wbs]
    seg_h = np.concatenate([[0], np.cumsum(lens)])
    outs = []
    for i, a in enumerate(ids):
        xs = x32[seg_h[i]:seg_h[i + 1]]
        outs.append(xs @ wbase.float().t() + scale[a] * ((xs @ A[a].t()) @ B[a].t()))
    y32 = torch.cat(outs)
    assert_close(y, y32.detach(), rtol=2e-2, atol=2e-2, what="y")
    want_gx = go.float() @ wbase.float()
    if tl:
        (y32[:tl] * go.float()[:tl]).sum().backward()
        want_gx[:tl] = x32.grad[:tl]
    s = max(1.0, float(want_gx.abs().max()))
    assert_close(xd.grad.float().cpu(), want_gx, rtol=1e-2, atol=1e-2 * s, what="grad_x")
    for idx in train_idx:
        ga = lin.get_parameter(f"lora-{idx}-A").grad
        gb = lin.get_parameter(f"lora-{idx}-B").grad
        assert_close(ga, A[idx].grad, rtol=1e-2, atol=1e-2 * max(1e-3, float(A[idx].grad.abs().max())), what=f"dA{idx}")
        assert_close(gb, B[idx].grad, rtol=1e-2, atol=1e-2 * max(1e-3, float(B[idx].grad.abs().max())), what=f"dB{idx}")
