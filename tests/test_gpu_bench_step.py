"""The step that bench.py times, checked as it is timed: the same Workload object, the same schedule
(one launch per kernel class over all projections, the split variant with a second stream, and the
per-projection launches on side streams), captured into a CUDA graph and replayed, then EVERY output
of EVERY projection compared with the CPU oracle at the reference's rounding points and at the
literal tolerance rtol = atol = 1e-2 for y and v over all rows and dX over the train rows; dA and dB of
all train partitions (the c3 batch has partitions of 1, 5, 15, 17, 108 and 1900 rows side by side) at
the bound bench.check_step documents, with under 1 % of their elements outside the literal one."""
import math

import pytest
import torch

import bench

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _poison_outputs(wl):
    """What the warm-up and the capture left behind must not be what the check sees."""
    for p in wl.proj:
        for k in ("y", "v", "dx", "dv"):
            if k in p:
                p[k].fill_(float("nan"))
        if "dA" in p and not wl.accumulate_grads:
            p["dA"].fill_(float("nan"))
            p["dB"].fill_(float("nan"))


@pytest.mark.parametrize("sched", ["multi", "multi_s", "multi_f", "split", "split3", "single"])
def test_c3_timed_step_every_projection_matches_oracle(sched):
    spec = bench.workload_spec("c3")
    parts = [l for l, f in zip(spec["lens"], spec["ft"]) if f]
    assert sum(parts) == 2048 and min(parts) == 1 and max(parts) >= 1024   # ragged partitions side by side
    wl = bench.Workload(spec, DEV)
    wl.sched = sched
    wl.step()
    torch.cuda.synchronize()
    replay = bench.capture(wl.step, torch)
    _poison_outputs(wl)
    for _ in range(3):
        replay()
    torch.cuda.synchronize()
    for pl in wl.plans():
        pl.raise_if_failed()
    worst, outside = bench.check_step(wl, torch)
    assert set(worst) == {"y", "v", "dX", "dA", "dB"} and set(outside) == {"dA", "dB"}
    assert all(math.isfinite(v) and v < 1e-2 for v in worst.values()), worst
    print("max|err|/max|ref|:", worst, "share outside the literal tolerance:", outside)


def test_c3_multi_and_single_schedules_agree():
    """One launch over all projections computes what the per-projection launches compute.  The forward's
    v and the backward's dV are sums over the hidden dimension that a launch may cut over the CTAs of a
    cluster differently (the cut is chosen per launch), so the two can differ in the last bit of a sum;
    everything else follows from them."""
    spec = bench.workload_spec("c3")
    outs = {}
    for sched in ("single", "multi", "multi_f", "split"):
        wl = bench.Workload(spec, DEV)
        wl.sched = sched
        wl.step()
        torch.cuda.synchronize()
        outs[sched] = [{k: p[k].clone() for k in ("y", "v", "dx", "dv", "dA", "dB")} for p in wl.proj]
        del wl
    for sched in ("multi", "multi_f", "split"):
        for a, b in zip(outs["single"], outs[sched]):
            for k in a:
                x, y = a[k].float(), b[k].float()
                tol = 2.0 ** -6 * x.abs() + 4e-3 * float(x.abs().max())
                assert bool(((x - y).abs() <= tol).all()), f"{sched}: {k} differs from the per-projection launches"
                if k not in ("dA", "dB"):   # (a gradient element sums thousands of products with v / dV)
                    assert float((a[k] != b[k]).float().mean()) < 0.02, f"{sched}: {k}: too many elements differ"
    # the two single-launch orders run the same kernels with the same cuts: bit-identical
    for a, b in zip(outs["multi"], outs["multi_f"]):
        for k in a:
            assert torch.equal(a[k], b[k]), f"multi vs multi_f: {k}"


def test_c3_host_pipeline_matches_oracle():
    """The end-to-end step of the benchmark (row blocks through pinned host buffers) leaves the same
    results in host memory as the oracle computes."""
    spec = bench.workload_spec("c3")
    wl = bench.Workload(spec, DEV)
    hp = bench.HostPipeline(wl, torch)
    # device copies of the inputs are destroyed: the pipeline must bring them from the host buffers
    saved = [(p["x"].clone(), p["go"].clone()) for p in wl.proj]
    for p in wl.proj:
        p["x"].fill_(float("nan"))
        p["go"].fill_(float("nan"))
    _poison_outputs(wl)
    hp.step()
    torch.cuda.synchronize()
    for pl in hp.plans:
        pl.raise_if_failed()
    for p, h, (x, go) in zip(wl.proj, hp.h, saved):
        assert torch.equal(p["x"], x) and torch.equal(p["go"], go)
        for k in ("y", "dx", "dA", "dB"):
            assert torch.equal(h[k], p[k].cpu()), f"{p['name']}: host copy of {k} differs from the device result"
    worst, _ = bench.check_step(wl, torch)
    assert all(v < 1e-2 for v in worst.values()), worst


@pytest.mark.parametrize("order", ["fused", "grads_first"])
def test_c5_data_parallel_step_one_rank_matches_oracle(order):
    """Workload c5 as bench.py runs it (tcgen05 kernels, gradients written into bucket slots, the last
    projection's weight gradients in slot ranges) at full size: 16 partitions of 2048 rows, rank 64, both
    directions 4096 <-> 14336.  Both orders of a step: dV/dX fused, or dV early and dX last."""
    spec = bench.workload_spec("c5")
    wl = bench.Workload(spec, DEV)
    dp = bench.DataParallelStep(wl, torch, None, chunks=4)
    dp.order = order
    assert len(dp.ranges) == 4 and dp.bucket.n_slots == 16
    dp.step()
    torch.cuda.synchronize()
    replay = bench.capture(dp.step, torch)
    _poison_outputs(wl)
    dp.bucket.flat.fill_(float("nan"))   # every slot is written by this rank's kernels, none needs clearing
    replay()
    replay()
    torch.cuda.synchronize()
    for pl in wl.plans():
        pl.raise_if_failed()
    # gradients sit in the slots of the partitions' adapters
    for i, p in enumerate(wl.proj):
        sl = dp.bucket.slots(dp.local_ids)
        p["dA"] = dp.bucket.dA[i][sl]
        p["dB"] = dp.bucket.dB[i][sl]
    wl.accumulate_grads = False
    worst, _ = bench.check_step(wl, torch)
    assert all(v < 1e-2 for v in worst.values()), worst
