#!/usr/bin/env python
"""Benchmark of the SMLM path (segmented multi-LoRA shrink/expand forward and the
fine-tuning backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3|c2|c4|c5]
    python bench.py --impl reference ...       # the CPU path on the host cores

One "step" is one pass of the hot path over one synthetic batch: for every LoRA
target projection of one transformer layer, the fused forward over all token rows
and the backward (dV, dB, dA, dX) over the fine-tune rows.  Default workload (c3):
Llama-3-8B projection set, bf16, rank 16, 128 adapters, 8192 tokens in segments of
Zipf(1.2) lengths clipped to [1, 2048], 25 % of the tokens in fine-tune segments.
Under torchrun every rank holds its own batch (weak scaling) whose segments use
the adapters that rank owns; the path has no collective for c2/c3/c4; for c5 the dA/dB
slice of each projection is all-reduced over NCCL, started right behind that projection's
weight-gradient kernel so that it runs under the next projection's backward.

Rank 0 prints ONE JSON line.  `value` is tokens/s with inputs resident in HBM;
`e2e` is the same metric with the step's inputs copied from pinned host memory and
its results copied back inside the timed region; `roofline` describes the kernel
class that takes the largest share of the step; `cpu_baseline` is the CPU oracle
(a port of the reference's per-segment torch path) timed on the host cores.
Inputs of one step exceed the 126 MB L2 several times over, so consecutive steps
do not find their operands in cache.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SCALE = 2.0  # alpha / r of the reference's fine-tune configuration (16 / 8)


# ---------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------

def zipf_lengths(seed, total, a=1.2, lo=1, hi=2048):
    rng = np.random.default_rng(seed)
    lens, tot = [], 0
    while tot < total:
        n = int(min(hi, max(lo, rng.zipf(a))))
        n = min(n, total - tot)
        lens.append(n)
        tot += n
    return lens


def workload_spec(name, rank=0, world=1):
    """Returns dict(projections=[(name, h_in, h_out)], lens, ft (bool per segment),
    ids, n_adapters, rank, dtype).  Row order: fine-tune segments, then the rest."""
    k = {"c2": 2, "c3": 3, "c4": 4, "c4s": 4, "c5": 5}[name]
    seed = 1000 * k + rank
    rng = np.random.default_rng(seed)
    if name == "c2":
        lens = [1024, 1024] + [512] * 4 + [1] * 64
        ft = [True, True] + [False] * 68
        n_ad, r, dt = 32, 16, "fp16"
        proj = [("q_proj", 4096, 4096)]
    elif name == "c3":
        # the segment lengths are the same on every rank (weak scaling: per-GPU work is fixed);
        # adapter ids and tensor values differ per rank
        raw = zipf_lengths(1000 * k, 8192)
        # mark fine-tune segments in generation order until 2048 tokens, splitting the crossing one
        ft_lens, inf_lens, acc = [], [], 0
        for n in raw:
            if acc < 2048:
                take = min(n, 2048 - acc)
                ft_lens.append(take)
                acc += take
                if n > take:
                    inf_lens.append(n - take)
            else:
                inf_lens.append(n)
        lens = ft_lens + inf_lens
        ft = [True] * len(ft_lens) + [False] * len(inf_lens)
        n_ad, r, dt = 128, 16, "bf16"
        proj = [("q_proj", 4096, 4096), ("k_proj", 4096, 1024), ("v_proj", 4096, 1024), ("o_proj", 4096, 4096),
                ("gate_proj", 4096, 14336), ("up_proj", 4096, 14336), ("down_proj", 14336, 4096)]
    elif name in ("c4", "c4s"):
        lens = [1] * 1024
        ft = [False] * 1024
        n_ad, r, dt = 256, 32, "bf16"
        proj = [("expand_4096_11008", 4096, 11008), ("shrink_11008_4096", 11008, 4096)]
    else:  # c5
        lens = [2048] * 16
        ft = [True] * 16
        n_ad, r, dt = 64, 64, "bf16"
        proj = [("up_4096_14336", 4096, 14336), ("down_14336_4096", 14336, 4096)]
    if name == "c5":
        # the train partitions of a rank are ordered by adapter, so that a range of adapters is a range of rows
        ids = sorted(int(v) for v in rng.choice(n_ad, size=16, replace=False))
    else:
        # a rank only receives segments of the adapters it owns: a mod world == rank
        owned = np.arange(rank, n_ad, world)
        ids = [int(v) for v in owned[rng.integers(0, len(owned), size=len(lens))]]
    if name == "c4s":
        # the same decode tokens in the order the reference's batch assembler produces: decode requests
        # sorted by adapter, equal neighbours merged into one segment (model_generation.py:186, 267-273)
        ids = sorted(ids)
        merged_ids, merged_lens = [], []
        for a_ in ids:
            if merged_ids and merged_ids[-1] == a_:
                merged_lens[-1] += 1
            else:
                merged_ids.append(a_)
                merged_lens.append(1)
        ids, lens, ft = merged_ids, merged_lens, [False] * len(merged_ids)
    return dict(name=name, projections=proj, lens=lens, ft=ft, ids=ids, n_adapters=n_ad, rank=r, dtype=dt,
                seed=seed)


def algorithmic_bytes(spec):
    """Compulsory HBM traffic of one step with 2-byte elements and gradients: every
    activation row read or written once, every distinct adapter panel once; the
    rank-r intermediates of the forward are not counted."""
    e = 2
    T = sum(spec["lens"])
    n = sum(l for l, f in zip(spec["lens"], spec["ft"]) if f)
    used = len(set(spec["ids"]))
    used_ft = len(set(i for i, f in zip(spec["ids"], spec["ft"]) if f))
    r = spec["rank"]
    fwd = bwd = 0
    for _, hi, ho in spec["projections"]:
        fwd += e * (T * hi + T * ho + used * r * (hi + ho))
        if n:
            bwd += e * (n * ho + 2 * n * hi + n * r) + 2 * e * used_ft * r * (hi + ho)
    return fwd, bwd


class Workload:
    """Device-resident tensors of one rank's batch."""

    def __init__(self, spec, device):
        import torch
        from loquetier_b200 import ops
        self.spec = spec
        self.dev = device
        dt = torch.float16 if spec["dtype"] == "fp16" else torch.bfloat16
        self.dt = dt
        g = torch.Generator(device=device).manual_seed(spec["seed"])
        self.T = sum(spec["lens"])
        self.tl = sum(l for l, f in zip(spec["lens"], spec["ft"]) if f)
        self.npart = sum(spec["ft"])
        seg = np.concatenate([[0], np.cumsum(spec["lens"])]).astype(np.int32)
        self.seg_h = seg
        self.seg = torch.tensor(seg, dtype=torch.int32, device=device)
        self.ids = torch.tensor(spec["ids"], dtype=torch.int32, device=device)
        self.part = torch.tensor(seg[:self.npart + 1], dtype=torch.int32, device=device)
        self.part_ids = self.ids[:self.npart].contiguous()
        r, n_ad = spec["rank"], spec["n_adapters"]
        self.scale = torch.full((n_ad,), SCALE, dtype=torch.float32, device=device)
        self.proj = []
        tab = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=device)
        for name, hi, ho in spec["projections"]:
            p = dict(name=name, h_in=hi, h_out=ho)
            p["x"] = torch.randn((self.T, hi), generator=g, device=device, dtype=torch.float32).to(dt)
            p["A"] = (torch.randn((n_ad, r, hi), generator=g, device=device) / np.sqrt(hi)).to(dt)
            p["B"] = (torch.randn((n_ad, ho, r), generator=g, device=device) * 0.02).to(dt)
            p["wa"], p["wb"] = tab(list(p["A"])), tab(list(p["B"]))
            p["y"] = torch.empty((self.T, ho), device=device, dtype=dt)
            p["v"] = torch.empty((self.T, r), device=device, dtype=dt)
            if self.tl:
                p["go"] = torch.randn((self.tl, ho), generator=g, device=device, dtype=torch.float32).to(dt)
                p["dx"] = torch.empty((self.tl, hi), device=device, dtype=dt)
                p["dv"] = torch.empty((self.tl, r), device=device, dtype=dt)
                p["dA"] = torch.empty((self.npart, r, hi), device=device, dtype=dt)
                p["dB"] = torch.empty((self.npart, ho, r), device=device, dtype=dt)
                p["dA_t"], p["dB_t"] = tab(list(p["dA"])), tab(list(p["dB"]))
            self.proj.append(p)
        self.plan = None
        self.pplan = None
        self.iplan = None
        self.ops = ops
        self.accumulate_grads = False
        self.grouped = True
        self.after_wgrad = None  # callable(projection index), called on the stream of its weight gradients
        self.overlap = True
        self.n_streams = 3
        self.side = []
        self.torch = torch
        # "multi": one launch per kernel class over all projections; "split": the same with the forward of
        # the inference rows on a second stream; "single": one launch per projection and class
        self.sched = "multi"
        self.pset = ops.ProjSet([dict(x=p["x"], y=p["y"], v=p["v"], go=p.get("go"), dx=p.get("dx"), dv=p.get("dv"),
                                      wa=p["wa"], wb=p["wb"], dA_t=p.get("dA_t"), dB_t=p.get("dB_t"),
                                      h_in=p["h_in"], h_out=p["h_out"]) for p in self.proj]) \
            if len(self.proj) <= 8 else None
        if self.npart and self.npart < len(spec["lens"]):
            self.iseg = self.seg[self.npart:].contiguous()
            self.iids = self.ids[self.npart:].contiguous()
        else:
            self.iseg = self.iids = None

    def rebuild_projset(self):
        """After the gradient tables were re-pointed (the data-parallel bucket)."""
        self.pset = self.ops.ProjSet([dict(x=p["x"], y=p["y"], v=p["v"], go=p.get("go"), dx=p.get("dx"),
                                           dv=p.get("dv"), wa=p["wa"], wb=p["wb"], dA_t=p.get("dA_t"),
                                           dB_t=p.get("dB_t"), h_in=p["h_in"], h_out=p["h_out"])
                                      for p in self.proj])

    def build_plans(self):
        # grouped where it changes anything: decode tokens are gathered by adapter for the forward launches
        from loquetier_b200.segments import wants_grouped_plan
        lens, ids = self.spec["lens"], self.spec["ids"]
        if self.sched in ("split", "split2", "split3") and self.iseg is not None:
            # the train rows go through the partition plan, the other rows get a plan of their own
            g = self.grouped and wants_grouped_plan(lens[self.npart:], ids[self.npart:])
            self.plan = None
            if self.sched == "split3" and self.tl:
                self.iplan, self.pplan = self.ops.plan_pair(self.iseg, self.T, self.part, self.tl,
                                                            seg_ids_a=self.iids if g else None,
                                                            n_table_a=self.spec["n_adapters"])
                return
            self.iplan = self.ops.Plan(self.iseg, self.T, seg_ids=self.iids if g else None,
                                       n_table=self.spec["n_adapters"])
        else:
            g = self.grouped and wants_grouped_plan(lens, ids)
            self.iplan = None
            if self.tl and self.sched != "single":
                # both plans of the step from one launch
                self.plan, self.pplan = self.ops.plan_pair(self.seg, self.T, self.part, self.tl,
                                                           seg_ids_a=self.ids if g else None,
                                                           n_table_a=self.spec["n_adapters"])
                return
            self.plan = self.ops.Plan(self.seg, self.T, seg_ids=self.ids if g else None,
                                      n_table=self.spec["n_adapters"])
        if self.tl:
            self.pplan = self.ops.Plan(self.part, self.tl)

    def plans(self):
        return [p for p in (self.plan, self.pplan, self.iplan) if p is not None]

    @property
    def launches_per_step(self):
        """Kernels of this library launched per step: the plans, then per class one launch (multi / split)
        or one per projection (single)."""
        nplan = 1 + (1 if self.tl and (self.sched in ("single", "split", "split2", "split3") or self.pset is None) else 0)
        if self.sched == "single" or self.pset is None:
            return nplan + len(self.proj) * (1 + (2 if self.tl else 0))
        if self.sched == "split3" and self.iseg is not None and self.tl:
            return 1 + 4
        if self.sched in ("split", "split2") and self.iseg is not None and self.tl:
            return nplan + 4
        return nplan + 1 + ((3 if self.sched == "multi_s" else 2) if self.tl else 0)

    def step(self):
        if self.sched == "single" or self.pset is None:
            return self.step_single()
        ops, r, torch = self.ops, self.spec["rank"], self.torch
        self.build_plans()
        n_ad = self.spec["n_adapters"]
        if self.sched == "split3" and self.iseg is not None and self.tl:
            # One stream.  The weight gradients need v and dV of the train rows only, so the forward is cut in
            # two: the train rows' forward runs next to dV/dX, the weight gradients follow, and the forward of
            # the other rows - most of the step - is launched last as an independent launch: it touches nothing
            # the weight gradients touch, so its CTAs run next to theirs (pure reads next to reads and writes).
            ops.bwd_dx_multi(self.pset, self.pplan, r, part_ids=self.part_ids, part_scale=self.scale)
            ops.fwd_multi(self.pset, self.pplan, r, seg_ids=self.part_ids, seg_scale=self.scale,
                          independent=self.overlap)
            ops.wgrad_pair_multi(self.pset, self.part, self.pplan, r, part_ids=self.part_ids,
                                 part_scale=self.scale, n_table=n_ad, accumulate=self.accumulate_grads)
            ops.fwd_multi(self.pset, self.iplan, r, seg_ids=self.iids, seg_scale=self.scale,
                          independent=self.overlap)
            return
        if self.sched in ("split", "split2") and self.iseg is not None and self.tl:
            # The weight gradients need v and dV of the train rows only, so the forward is cut in two: the
            # train rows (through the partition plan) and the other rows (a plan of their own).
            main = torch.cuda.current_stream()
            if self.sched == "split":
                # the forward of the inference rows - most of the step - on a second stream, next to
                # dV/dX, the train rows' forward and the weight gradients
                if not self.side:
                    self.side = [torch.cuda.Stream()]
                fork = torch.cuda.Event()
                fork.record(main)
                self.side[0].wait_event(fork)
                with torch.cuda.stream(self.side[0]):
                    ops.fwd_multi(self.pset, self.iplan, r, seg_ids=self.iids, seg_scale=self.scale)
                ops.bwd_dx_multi(self.pset, self.pplan, r, part_ids=self.part_ids, part_scale=self.scale)
                ops.fwd_multi(self.pset, self.pplan, r, seg_ids=self.part_ids, seg_scale=self.scale,
                              independent=self.overlap)
                ops.wgrad_pair_multi(self.pset, self.part, self.pplan, r, part_ids=self.part_ids,
                                     part_scale=self.scale, n_table=n_ad, accumulate=self.accumulate_grads)
                main.wait_stream(self.side[0])
                return
            # split2: everything on the calling stream except the weight gradients, which run on a
            # high-priority stream as soon as dV/dX and the train rows' forward are done: their CTAs -
            # pure reads - are placed ahead of the inference rows' forward and run next to its writes
            if not self.side:
                self.side = [torch.cuda.Stream(priority=-1)]
            ops.bwd_dx_multi(self.pset, self.pplan, r, part_ids=self.part_ids, part_scale=self.scale)
            ops.fwd_multi(self.pset, self.pplan, r, seg_ids=self.part_ids, seg_scale=self.scale,
                          independent=self.overlap)
            ready = torch.cuda.Event()
            ready.record(main)
            ops.fwd_multi(self.pset, self.iplan, r, seg_ids=self.iids, seg_scale=self.scale, independent=self.overlap)
            with torch.cuda.stream(self.side[0]):
                self.side[0].wait_event(ready)
                ops.wgrad_pair_multi(self.pset, self.part, self.pplan, r, part_ids=self.part_ids,
                                     part_scale=self.scale, n_table=n_ad, accumulate=self.accumulate_grads)
            main.wait_stream(self.side[0])
            return
        # One launch per kernel class.  dV/dX and the forward do not depend on each other: the second of the
        # two is marked independent and starts while the first drains; the weight gradients consume v
        # and dV and come last.  "multi": dV/dX first; "multi_f": the forward first, so that the weight
        # gradients follow dV/dX directly (the gO rows it read last are still in L2).
        if self.sched == "multi_s" and self.tl:
            # dA = dV^T . X needs nothing of the forward: it follows dV/dX directly, the forward runs next to it
            # as an independent launch (reads next to reads and writes), and only dB = gO^T . V is left for the end
            ops.bwd_dx_multi(self.pset, self.pplan, r, part_ids=self.part_ids, part_scale=self.scale)
            ops.wgrad_pair_multi(self.pset, self.part, self.pplan, r, part_ids=self.part_ids, part_scale=self.scale,
                                 n_table=n_ad, accumulate=self.accumulate_grads, which=ops.WGRAD_DA)
            ops.fwd_multi(self.pset, self.plan, r, seg_ids=self.ids, seg_scale=self.scale, independent=self.overlap)
            ops.wgrad_pair_multi(self.pset, self.part, self.pplan, r, part_ids=self.part_ids, part_scale=self.scale,
                                 n_table=n_ad, accumulate=self.accumulate_grads, which=ops.WGRAD_DB)
            return
        if self.sched == "multi_f":
            ops.fwd_multi(self.pset, self.plan, r, seg_ids=self.ids, seg_scale=self.scale)
            if self.tl:
                ops.bwd_dx_multi(self.pset, self.pplan, r, part_ids=self.part_ids, part_scale=self.scale,
                                 independent=self.overlap)
        else:
            if self.tl:
                ops.bwd_dx_multi(self.pset, self.pplan, r, part_ids=self.part_ids, part_scale=self.scale)
            ops.fwd_multi(self.pset, self.plan, r, seg_ids=self.ids, seg_scale=self.scale,
                          independent=self.overlap and self.tl > 0)
        if self.tl:
            ops.wgrad_pair_multi(self.pset, self.part, self.pplan, r, part_ids=self.part_ids, part_scale=self.scale,
                                 n_table=n_ad, accumulate=self.accumulate_grads)

    def step_single(self):
        """One launch per projection and kernel class: plans once, then for every projection the fused
        forward, the fused dV/dX backward and the weight gradients.  The projections are independent of
        each other, so the launches of one kind are issued back to back and marked independent: the read
        phase of one overlaps the write phase of the one before.  The weight gradients come last
        because they consume v and dV."""
        ops = self.ops
        self.build_plans()
        r = self.spec["rank"]
        torch = self.torch
        main = torch.cuda.current_stream()
        ns = max(0, min(self.n_streams, len(self.proj))) if self.tl else 0
        if len(self.side) < ns:
            self.side = [torch.cuda.Stream() for _ in range(ns)]
        if ns:
            fork = torch.cuda.Event()
            fork.record(main)
            for s in self.side[:ns]:
                s.wait_event(fork)
        # forward chain on the calling stream
        done = []
        for i, p in enumerate(self.proj):
            ops.fwd(p["y"], p["x"], p["v"], p["wa"], p["wb"], self.plan, r, seg_ids=self.ids,
                    seg_scale=self.scale, independent=self.overlap and i > 0)
            if ns:
                ev = torch.cuda.Event()
                ev.record(main)
                done.append(ev)
        if self.tl:
            # The backward launches are small (2048 rows) and a stream keeps at most two kernels in
            # flight, so the projections are dealt over a few side streams that run next to the
            # forward chain.  dV/dX of a projection needs nothing from its forward; the weight
            # gradients need v (forward) and dV, so they wait for that projection's forward.
            for i, p in enumerate(self.proj):
                s = self.side[i % ns] if ns else main
                with torch.cuda.stream(s):
                    ops.bwd_dx(p["dx"], p["dv"], p["go"], p["wa"], p["wb"], self.pplan, r, part_ids=self.part_ids,
                               part_scale=self.scale, independent=self.overlap and ns > 0 and i >= ns)
                    if ns:
                        s.wait_event(done[i])
                    # one workspace per projection: launches of different streams run side by side
                    ws = ops.wgrad_workspace(self.dev, self.tl, self.npart, r, p["h_out"], p["h_in"], slot=i)
                    ops.wgrad_pair(p["dA_t"], p["dB_t"], p["dv"], p["x"], p["v"], p["go"], self.part, self.pplan, r,
                                   part_ids=self.part_ids, part_scale=self.scale,
                                   n_table=self.spec["n_adapters"], accumulate=self.accumulate_grads,
                                   workspace=ws)
                    if self.after_wgrad is not None:
                        self.after_wgrad(i)
            for s in self.side[:ns]:
                main.wait_stream(s)

# ---------------------------------------------------------------------------
# timing helpers
# ---------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs; only samples
    whose timestamp falls between mark_start() and mark_end() are used."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.t0 = self.t1 = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
        return self

    def mark_start(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def __exit__(self, *a):
        import datetime
        self.result = dict(sm_mhz=None, sm_max_mhz=None, reasons=[])
        if self.proc is None:
            return
        time.sleep(0.1)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            return
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [v.strip() for v in line.split(",")]
            if len(f) < 8:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                if self.t0 is not None and self.t1 is not None and not (self.t0 - 0.02 <= ts <= self.t1 + 0.02):
                    continue
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        if sm:
            self.result = dict(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons),
                               samples=len(sm))


def timed(fn, steps, warmup, torch, dist=None, clk=None, blocks=1):
    """W untimed iterations, then `blocks` timed blocks of EXACTLY `steps` iterations, each bracketed
    by barrier + synchronize on both sides; device time from CUDA events on the current stream; max
    over ranks per block.  Returns (median ms per step over the blocks, [ms per step of every block])."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    per_block = []
    if clk is not None:
        clk.mark_start()
    for _ in range(max(1, blocks)):
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        per_block.append(ms / steps)
    if clk is not None:
        clk.mark_end()
    return float(np.median(per_block)), per_block


def class_bytes(wl):
    """Algorithmic bytes of one step per kernel class (2-byte elements; every distinct adapter panel
    once per class; the rank-r intermediate a class writes or reads is counted with it)."""
    r, e = wl.spec["rank"], 2
    used = len(set(wl.spec["ids"]))
    used_ft = len(set(wl.spec["ids"][:wl.npart]))
    T, n = wl.T, wl.tl
    fwd = sum(e * (T * p["h_in"] + T * p["h_out"] + T * r + used * r * (p["h_in"] + p["h_out"])) for p in wl.proj)
    bdx = sum(e * (n * p["h_out"] + n * p["h_in"] + n * r + used_ft * r * (p["h_in"] + p["h_out"])) for p in wl.proj)
    wg = sum(e * (n * (p["h_in"] + p["h_out"]) + 2 * n * r + used_ft * r * (p["h_in"] + p["h_out"])) for p in wl.proj)
    return fwd, bdx, wg


def kernel_breakdown(wl, torch, reps=5):
    """Device time of every kernel class over one step, each class timed alone between two CUDA
    events on the launching stream with L2 flushed before: with the multi schedules a class is ONE
    launch over all projections, with the single schedule it is the class launched back to back for
    every projection (so that launch gaps do not count).  Same C-ABI entry points as the step.
    Returns {class: (ms per step, algorithmic bytes per step, launches per step)}."""
    ops, r = wl.ops, wl.spec["rank"]
    n, n_ad = wl.tl, wl.spec["n_adapters"]
    sched = wl.sched
    multi = sched != "single" and wl.pset is not None
    wl.sched = "multi" if multi else "single"   # the classes run over the whole batch with the full plan
    wl.build_plans()
    for p in wl.proj:  # make v / dv valid for the classes that read them
        ops.fwd(p["y"], p["x"], p["v"], p["wa"], p["wb"], wl.plan, r, seg_ids=wl.ids, seg_scale=wl.scale)
        if n:
            ops.bwd(p["dx"], p["dA_t"], p["dB_t"], p["dv"], p["go"], p["x"], p["v"], p["wa"], p["wb"], wl.pplan,
                    r, part_ids=wl.part_ids, part_scale=wl.scale, accumulate_grads=wl.accumulate_grads)
    fwd_b, bdx_b, wg_b = class_bytes(wl)
    nproj = len(wl.proj)
    tc = r > 32
    names = (("fused_tc_kernel" if tc else "fused_kernel"), ("wgrad_tc_kernel" if tc else "wgrad_kernel"))

    def fwd_all():
        if multi:
            ops.fwd_multi(wl.pset, wl.plan, r, seg_ids=wl.ids, seg_scale=wl.scale)
        else:
            for i, p in enumerate(wl.proj):
                ops.fwd(p["y"], p["x"], p["v"], p["wa"], p["wb"], wl.plan, r, seg_ids=wl.ids, seg_scale=wl.scale,
                        independent=wl.overlap and i > 0)

    def bdx_all():
        if multi:
            ops.bwd_dx_multi(wl.pset, wl.pplan, r, part_ids=wl.part_ids, part_scale=wl.scale)
        else:
            for i, p in enumerate(wl.proj):
                ops.bwd_dx(p["dx"], p["dv"], p["go"], p["wa"], p["wb"], wl.pplan, r, part_ids=wl.part_ids,
                           part_scale=wl.scale, independent=wl.overlap and i > 0)

    def wg_all():
        if multi:
            ops.wgrad_pair_multi(wl.pset, wl.part, wl.pplan, r, part_ids=wl.part_ids, part_scale=wl.scale,
                                 n_table=n_ad, accumulate=wl.accumulate_grads)
        else:
            for i, p in enumerate(wl.proj):
                ops.wgrad_pair(p["dA_t"], p["dB_t"], p["dv"], p["x"], p["v"], p["go"], wl.part, wl.pplan, r,
                               part_ids=wl.part_ids, part_scale=wl.scale, n_table=n_ad,
                               accumulate=wl.accumulate_grads,
                               workspace=ops.wgrad_workspace(wl.dev, n, wl.npart, r, p["h_out"], p["h_in"], slot=i),
                               independent=wl.overlap and i > 0)

    nl = 1 if multi and not tc else nproj
    classes = {f"{names[0]}(fwd x->v->y)": (fwd_all, fwd_b)}
    if n:
        classes[f"{names[0]}(bwd gO->dV->dX)"] = (bdx_all, bdx_b)
        classes[f"{names[1]}(dB=gO^T.V, dA=dV^T.X)"] = (wg_all, wg_b)
    out = {}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=wl.dev)
    for name, (fn, nbytes) in classes.items():
        ts = []
        for it in range(reps + 1):
            flush.zero_()  # evict L2 between repetitions of the same class
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if it > 0:
                ts.append(e0.elapsed_time(e1))
        out[name] = (float(np.median(ts)), float(nbytes), nl if not name.startswith("wgrad") else (1 if multi else nproj))
    wl.sched = sched
    return out


# ---------------------------------------------------------------------------
# parity of the timed step
# ---------------------------------------------------------------------------

def check_step(wl, torch, rtol=1e-2, atol=1e-2):
    """Compares what the step left in device memory - y and v of every projection over all rows, dX, dA
    and dB of every projection and train partition - with the CPU oracle evaluated on the same 16-bit
    inputs, at the rounding points of the reference (v and dV rounded to the storage type).

    y, v and dX: every element within |got - want| <= atol + rtol * |want| (the literal tolerance).
    dA and dB are sums over a partition's tokens (up to 1900 here) of products with a rank-r intermediate
    that both sides round to 16 bits on their own.  Two fp32 sums of 4096+ terms in different order land
    on different sides of a rounding boundary for about one intermediate element in a thousand, and each
    such flip moves a gradient element by ulp(intermediate) * |other operand| - here up to
    2^-6 * 4 = 0.06 - whatever the size of that gradient element.  So small elements of a long
    partition's gradient cannot meet an absolute bound of 0.01; they are held to
    |got - want| <= rtol * |want| + atol * max(1, max|want|), and the share of elements outside the
    literal tolerance is reported (observed: under 0.2 % at rank 16, under 2 % at rank 64, where an element
    sums 64 such products) and must stay below 5 %.
    Returns ({tensor class: max|err| / max|want|}, {gradient class: largest share outside the literal
    tolerance}); raises AssertionError naming the first tensor outside its bound."""
    from oracle import smlm_oracle as O
    spec = wl.spec
    T, npart, tl, r = wl.T, wl.npart, wl.tl, spec["rank"]
    seg = [int(v) for v in wl.seg_h]
    ids = spec["ids"]
    worst, outside = {}, {}

    def cmp(name, got, want, grad=False):
        g, w = got.detach().to("cpu", torch.float32), want.detach().to("cpu", torch.float32)
        assert g.shape == w.shape, f"{name}: shape {tuple(g.shape)} vs {tuple(w.shape)}"
        assert bool(torch.isfinite(g).all()), f"{name}: non-finite values"
        err = (g - w).abs()
        wmax = float(w.abs().max()) if w.numel() else 0.0
        literal = err > atol + rtol * w.abs()
        bad = err > atol * max(1.0, wmax) + rtol * w.abs() if grad else literal
        key = name.split("[")[0].split(".")[-1]
        if g.numel():
            worst[key] = max(worst.get(key, 0.0), float(err.max()) / max(wmax, 1e-30))
        if grad and g.numel():
            share = float(literal.float().mean())
            outside[key] = max(outside.get(key, 0.0), share)
            assert share < 5e-2, f"{name}: {share:.2%} of the elements outside the literal rtol={rtol} atol={atol}"
        if bool(bad.any()):
            i = torch.nonzero(bad)[0].tolist()
            raise AssertionError(f"{name}: {int(bad.sum())}/{g.numel()} elements outside rtol={rtol} atol={atol}; "
                                 f"max abs err {float(err.max()):.4g}; first at {i}: got {float(g[tuple(i)])} "
                                 f"want {float(w[tuple(i)])}")

    for p in wl.proj:
        x, A, B = p["x"].cpu(), p["A"].cpu(), p["B"].cpu()
        y_ref, v_ref = O.add_lora_forward((T, p["h_out"]), x, [A[i] for i in ids], [B[i] for i in ids], seg, r,
                                          round_v=True)
        cmp(f"{p['name']}.y", p["y"], y_ref.to(torch.float32) * SCALE)
        cmp(f"{p['name']}.v", p["v"], v_ref)
        if tl:
            # the scale is a power of two here, so scaling gO in the storage type is exact and the oracle's
            # rounding points (dV = round(scale * gO . B)) are the kernels'
            go = (p["go"].cpu().to(torch.float32) * SCALE).to(wl.dt)
            gx, grads = O.add_lora_backward(go, x[:tl], [A[i] for i in ids[:npart]], [B[i] for i in ids[:npart]],
                                            seg[:npart + 1], round_mid=True)
            cmp(f"{p['name']}.dX", p["dx"], gx)
            for k in range(npart):
                cmp(f"{p['name']}.dA[{k}]", p["dA"][k], grads[2 * k], grad=True)
                cmp(f"{p['name']}.dB[{k}]", p["dB"][k], grads[2 * k + 1], grad=True)
    return worst, outside


# ---------------------------------------------------------------------------
# end to end through host buffers
# ---------------------------------------------------------------------------

def bind_to_gpu_numa_node(local):
    """Runs this process on the CPUs of the NUMA node its GPU hangs off, so that the pinned buffers
    allocated afterwards are local to the PCIe root of the GPU.  Reads sysfs and nvidia-smi only;
    changes nothing but this process's own affinity.  Returns the node or None."""
    try:
        bdf = subprocess.run(["nvidia-smi", f"--id={local}", "--query-gpu=pci.bus_id", "--format=csv,noheader"],
                             capture_output=True, text=True, timeout=20).stdout.strip().lower()
        if bdf.count(":") == 2 and len(bdf.split(":")[0]) == 8:
            bdf = bdf[4:]  # sysfs uses a 4-digit PCI domain
        node = int(open(f"/sys/bus/pci/devices/{bdf}/numa_node").read().strip())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            a, _, b = part.partition("-")
            cpus.update(range(int(a), int(b or a) + 1))
        allowed = os.sched_getaffinity(0)
        if cpus & allowed:
            os.sched_setaffinity(0, cpus & allowed)
            return node
    except Exception:
        pass
    return None


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the default workload's three kernels, from one ncu
# capture of `python bench.py --steps 1 --warmup 3 --blocks 1 --no-graph ...` (the capture is summarised with the other profiles)
C3_TRAFFIC = {"fused_kernel(fwd x->v->y)": 693309696 + 675111424,
              "fused_kernel(bwd gO->dV->dX)": 198073856 + 106014720,
              "wgrad_kernel(dB=gO^T.V, dA=dV^T.X)": 336965888 + 29999616}


class HostPipeline:
    """The step with HOST inputs and outputs: x and gO of every projection start in pinned host memory;
    y, dX, dA and dB end in pinned host memory.  The batch is cut into row blocks - the train rows, then
    the other rows in equal parts - and every (projection, row block) is one unit: its rows are uploaded
    on one stream, run through the single-projection entry points (fused forward; for the train rows also
    the backward) on the compute stream, and downloaded on a third stream, so that only the first unit's
    upload and the last unit's download are not overlapped.  Segments are independent, so a row block is
    served by a plan on the segment index pointer clipped to its rows."""

    def __init__(self, wl, torch, nblocks=4):
        self.wl, self.torch = wl, torch
        pin = lambda t: torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t)
        pin_out = lambda t: torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        self.h = []
        self.h2d_bytes = self.d2h_bytes = 0
        for p in wl.proj:
            h = dict(x=pin(p["x"]), y=pin_out(p["y"]))
            self.h2d_bytes += p["x"].numel() * 2
            self.d2h_bytes += p["y"].numel() * 2
            if wl.tl:
                h.update(go=pin(p["go"]), dx=pin_out(p["dx"]), dA=pin_out(p["dA"]), dB=pin_out(p["dB"]))
                self.h2d_bytes += p["go"].numel() * 2
                self.d2h_bytes += (p["dx"].numel() + p["dA"].numel() + p["dB"].numel()) * 2
            self.h.append(h)
        self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
        # row blocks: [0, tl) holds the train rows; the rest in (nblocks - 1) parts cut at multiples of 64 rows
        T, tl = wl.T, wl.tl
        cuts = [0]
        if tl:
            cuts.append(tl)
        rest = max(1, nblocks - (1 if tl else 0))
        for k in range(1, rest + 1):
            c = tl + ((T - tl) * k // rest) // 64 * 64 if k < rest else T
            if c > cuts[-1]:
                cuts.append(c)
        self.blocks = []
        seg = torch.tensor(wl.seg_h, dtype=torch.int64)
        for lo, hi in zip(cuts[:-1], cuts[1:]):
            clipped = seg.clamp(lo, hi).to(torch.int32).to(wl.dev)
            self.blocks.append((lo, hi, clipped))
        # units in upload order: an inference block first (the smallest first upload), the train rows second,
        # the small-output projections last (the smallest last download)
        order_p = sorted(range(len(wl.proj)), key=lambda i: -wl.proj[i]["h_out"])
        order_b = list(range(len(self.blocks)))
        if tl and len(order_b) > 1:
            order_b = [1, 0] + order_b[2:]
        self.units = [(i, b) for b in order_b for i in order_p]

    def step(self):
        torch, wl, ops = self.torch, self.wl, self.wl.ops
        cur = torch.cuda.current_stream()
        r = wl.spec["rank"]
        self.s_in.wait_stream(cur)
        self.s_out.wait_stream(cur)
        plans = [ops.Plan(ind, wl.T) for (_, _, ind) in self.blocks]
        pplan = ops.Plan(wl.part, wl.tl) if wl.tl else None
        wl.plan, wl.pplan, wl.iplan = plans[-1], pplan, None   # what the caller checks for recorded faults
        self.plans = plans + ([pplan] if pplan is not None else [])
        ready = []
        with torch.cuda.stream(self.s_in):
            for i, b in self.units:
                p, h = wl.proj[i], self.h[i]
                lo, hi, _ = self.blocks[b]
                p["x"][lo:hi].copy_(h["x"][lo:hi], non_blocking=True)
                if wl.tl and lo == 0:
                    p["go"].copy_(h["go"], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.s_in)
                ready.append(ev)
        for (i, b), ev in zip(self.units, ready):
            p, h = wl.proj[i], self.h[i]
            lo, hi, _ = self.blocks[b]
            cur.wait_event(ev)
            ops.fwd(p["y"], p["x"], p["v"], p["wa"], p["wb"], plans[b], r, seg_ids=wl.ids, seg_scale=wl.scale)
            train = wl.tl and lo == 0
            if train:
                ops.bwd(p["dx"], p["dA_t"], p["dB_t"], p["dv"], p["go"], p["x"], p["v"], p["wa"], p["wb"],
                        pplan, r, part_ids=wl.part_ids, part_scale=wl.scale, accumulate_grads=wl.accumulate_grads)
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                h["y"][lo:hi].copy_(p["y"][lo:hi], non_blocking=True)
                if train:
                    h["dx"].copy_(p["dx"], non_blocking=True)
                    h["dA"].copy_(p["dA"], non_blocking=True)
                    h["dB"].copy_(p["dB"], non_blocking=True)
        cur.wait_stream(self.s_out)

    def copies_only(self):
        """The host-link bound of a step, measured: the same uploads and downloads on the same two streams
        with no kernel and no dependency between them, both directions busy from start to end."""
        torch, wl = self.torch, self.wl
        cur = torch.cuda.current_stream()
        self.s_in.wait_stream(cur)
        self.s_out.wait_stream(cur)
        with torch.cuda.stream(self.s_in):
            for i, b in self.units:
                p, h = wl.proj[i], self.h[i]
                lo, hi, _ = self.blocks[b]
                p["x"][lo:hi].copy_(h["x"][lo:hi], non_blocking=True)
                if wl.tl and lo == 0:
                    p["go"].copy_(h["go"], non_blocking=True)
        with torch.cuda.stream(self.s_out):
            for i, b in self.units:
                p, h = wl.proj[i], self.h[i]
                lo, hi, _ = self.blocks[b]
                h["y"][lo:hi].copy_(p["y"][lo:hi], non_blocking=True)
                if wl.tl and lo == 0:
                    h["dx"].copy_(p["dx"], non_blocking=True)
                    h["dA"].copy_(p["dA"], non_blocking=True)
                    h["dB"].copy_(p["dB"], non_blocking=True)
        cur.wait_stream(self.s_in)
        cur.wait_stream(self.s_out)


# ---------------------------------------------------------------------------
# CPU path (the oracle port of the reference's per-segment torch path)
# ---------------------------------------------------------------------------

def cpu_step_fn(spec, torch, max_proj=None):
    """Builds the batch on the host (same seeded distributions) and returns
    (fn running one step on the CPU, tokens per step).  16-bit inputs are upcast to
    fp32 once, outside the timed function, as CPU 16-bit GEMM is not representative."""
    from oracle import smlm_oracle as O
    g = torch.Generator().manual_seed(spec["seed"])
    T = sum(spec["lens"])
    npart = sum(spec["ft"])
    seg = [0]
    for n in spec["lens"]:
        seg.append(seg[-1] + n)
    tl = seg[npart]
    r, n_ad, ids = spec["rank"], spec["n_adapters"], spec["ids"]
    projs = spec["projections"][:max_proj] if max_proj else spec["projections"]
    data = []
    for name, hi, ho in projs:
        x = torch.randn((T, hi), generator=g)
        used = sorted(set(ids))
        A = {a: torch.randn((r, hi), generator=g) / np.sqrt(hi) for a in used}
        B = {a: torch.randn((ho, r), generator=g) * 0.02 for a in used}
        go = torch.randn((tl, ho), generator=g) if tl else None
        data.append((x, A, B, go, hi, ho))

    def fn():
        for x, A, B, go, hi, ho in data:
            y, v = O.add_lora_forward((T, ho), x, [A[i] for i in ids], [B[i] for i in ids], seg, r,
                                      round_v=False)
            y *= SCALE
            if tl:
                O.add_lora_backward(go * SCALE, x, [A[i] for i in ids[:npart]], [B[i] for i in ids[:npart]],
                                    seg[:npart + 1], round_mid=False)
    return fn, T, len(projs)


def run_cpu(spec, torch, budget_s=12.0, max_reps=5):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    fn, T, nproj = cpu_step_fn(spec, torch)
    fn()  # warm-up
    times = []
    t_all = time.perf_counter()
    while len(times) < max_reps and (time.perf_counter() - t_all) < budget_s:
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    sec = float(np.median(times))
    return dict(value=T / sec, unit="tokens/s", cores=cores, kind="port",
                sample=f"{len(times)} full steps of workload {spec['name']} ({nproj} projections, {T} tokens, "
                       f"fwd+bwd) in fp32 with torch.set_num_threads({cores}); median {sec * 1e3:.1f} ms/step"), sec


# ---------------------------------------------------------------------------
# main
# ---------------------------------------------------------------------------

WORKLOAD_TEXT = {
    "c2": "Llama-2-7B q_proj mixed batch, fp16, rank 16, 32 adapters, 2x1024 FT + 4x512 prefill + 64 decode",
    "c3": "Llama-3-8B 7 LoRA projections of one layer, bf16, rank 16, 128 adapters, 8192 tokens, "
          "Zipf(1.2) segment lengths in [1,2048], 25% fine-tune tokens (fwd+bwd), rest forward only",
    "c4": "decode sweep, bf16, 1024 one-token segments, 256 adapters, rank 32, 4096->11008 and 11008->4096",
    "c4s": "decode sweep as c4 with the tokens sorted by adapter and merged into segments, as the "
           "reference's batch assembler orders decode requests",
    "c5": "fine-tune heavy, bf16, rank 64, 64 adapters, 16x2048 FT tokens per GPU, 4096<->14336, "
          "dA/dB all-reduced over NCCL"}


def hbm_peak():
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class DataParallelStep:
    """Workload c5 on one rank of a data-parallel group: forward + backward of both projections with the
    sum of dA/dB over the ranks as the one exchange step.

    Gradients go straight into the slots of a flat bucket (loquetier_b200.dp.GradBucket); only adapters
    that some rank trains in this batch have a slot.  Order of a step: the up projection first, whole
    (forward, dV/dX, weight gradients), then its slots are handed to NCCL and travel under everything
    the down projection still has to do; the down projection's weight gradients are cut into `chunks`
    slot ranges (the train partitions are ordered by adapter, so a slot range is a row range), and
    every range is handed to NCCL as soon as its kernel has been issued, so that only the last range's
    exchange has nothing to hide under."""

    def __init__(self, wl, torch, dist, chunks=4):
        from loquetier_b200.dp import GradBucket, touched_union
        self.wl, self.torch, self.dist = wl, torch, dist
        spec = wl.spec
        self.bucket = GradBucket([(p["h_in"], p["h_out"]) for p in wl.proj], spec["n_adapters"], spec["rank"],
                                 wl.dt, wl.dev)
        self.local_ids = list(spec["ids"][:wl.npart])
        assert self.local_ids == sorted(self.local_ids), "train partitions must be ordered by adapter"
        self.union = touched_union(self.local_ids, spec["n_adapters"])
        self.bucket.set_touched(self.union)
        for i, p in enumerate(wl.proj):
            p["dA_t"], p["dB_t"] = self.bucket.tables(i, self.local_ids)
            p["dA"], p["dB"] = self.bucket.dA[i], self.bucket.dB[i]
        wl.rebuild_projset()
        # slot ranges of the last projection and the partitions (= row ranges) that fall into each
        ns = self.bucket.n_slots
        chunks = max(1, min(chunks, ns))
        self.ranges = []
        my_slots = self.bucket.slots(self.local_ids)
        for c in range(chunks):
            s0, s1 = ns * c // chunks, ns * (c + 1) // chunks
            parts = [k for k, sl in enumerate(my_slots) if s0 <= sl < s1]
            self.ranges.append((s0, s1, (parts[0], parts[-1] + 1) if parts else None))
        self.exchange = True
        self.sub = {}
        # "fused": per projection forward, dV/dX (one fused launch), weight gradients.  "grads_first": the
        # input gradients are cut in two - dV = scale gO . B right away, dX = dV . A at the very end - so that
        # the weight gradients of BOTH projections are out early and their exchange runs under the dX launches
        self.order = "fused"

    def _sub(self, p0, p1):
        """Index pointer, ids, tables and plan of partitions [p0, p1) for a partial weight-gradient launch."""
        wl, ops = self.wl, self.wl.ops
        key = (p0, p1)
        if key not in self.sub:
            self.sub[key] = dict(part=wl.part[p0:p1 + 1].contiguous(), ids=wl.part_ids[p0:p1].contiguous())
        d = dict(self.sub[key])
        d["plan"] = ops.Plan(d["part"], wl.tl)
        return d

    def step_grads_first(self):
        wl, ops, b = self.wl, self.wl.ops, self.bucket
        r, n_ad = wl.spec["rank"], wl.spec["n_adapters"]
        b.zero_except(self.local_ids)
        wl.sched = "single"
        wl.build_plans()
        for i, p in enumerate(wl.proj):
            ops.fwd(p["y"], p["x"], p["v"], p["wa"], p["wb"], wl.plan, r, seg_ids=wl.ids, seg_scale=wl.scale,
                    independent=i > 0)
            # dV = scale * gO . B alone (B is [h_out, r]: the row-major operand of this product)
            ops.gemm(p["dv"], p["go"], p["wb"], wl.pplan, is_row_major=True, seg_ids=wl.part_ids, seg_scale=wl.scale)
        for i, p in enumerate(wl.proj):
            ops.wgrad_pair(p["dA_t"], p["dB_t"], p["dv"], p["x"], p["v"], p["go"], wl.part, wl.pplan, r,
                           part_ids=wl.part_ids, part_scale=wl.scale, n_table=n_ad,
                           workspace=ops.wgrad_workspace(wl.dev, wl.tl, wl.npart, r, p["h_out"], p["h_in"], slot=i))
            if self.exchange:
                b.reduce_slots(i, 0, b.n_slots)
        for p in wl.proj:
            # dX = dV . A last: the largest writes of the backward run while the gradients travel
            ops.gemm(p["dx"], p["dv"], p["wa"], wl.pplan, is_row_major=True, seg_ids=wl.part_ids)
        b.finish()

    def step(self):
        if self.order == "grads_first":
            return self.step_grads_first()
        wl, ops, b = self.wl, self.wl.ops, self.bucket
        r, n_ad = wl.spec["rank"], wl.spec["n_adapters"]
        b.zero_except(self.local_ids)
        wl.sched = "single"
        wl.build_plans()
        last = len(wl.proj) - 1
        for i, p in enumerate(wl.proj):
            ops.fwd(p["y"], p["x"], p["v"], p["wa"], p["wb"], wl.plan, r, seg_ids=wl.ids, seg_scale=wl.scale,
                    independent=i > 0)
            ops.bwd_dx(p["dx"], p["dv"], p["go"], p["wa"], p["wb"], wl.pplan, r, part_ids=wl.part_ids,
                       part_scale=wl.scale, independent=True)
            if i < last or len(self.ranges) == 1:
                ops.wgrad_pair(p["dA_t"], p["dB_t"], p["dv"], p["x"], p["v"], p["go"], wl.part, wl.pplan, r,
                               part_ids=wl.part_ids, part_scale=wl.scale, n_table=n_ad,
                               workspace=ops.wgrad_workspace(wl.dev, wl.tl, wl.npart, r, p["h_out"], p["h_in"], slot=i))
                if self.exchange:
                    b.reduce_slots(i, 0, b.n_slots)
            else:
                # the plans of all ranges first: the launches after the first one do not wait for their
                # predecessors, so nothing they read may be written in between
                subs = [self._sub(*parts) if parts is not None else None for (_, _, parts) in self.ranges]
                launched = 0
                for c, (s0, s1, parts) in enumerate(self.ranges):
                    if parts is not None:
                        p0, p1 = parts
                        d = subs[c]
                        # the ranges touch different partitions, outputs and workspaces: each launch after
                        # the first may start while its predecessor drains
                        ops.wgrad_pair(p["dA_t"][p0:p1], p["dB_t"][p0:p1], p["dv"], p["x"], p["v"], p["go"], d["part"],
                                       d["plan"], r, part_ids=d["ids"], part_scale=wl.scale, n_table=n_ad,
                                       workspace=ops.wgrad_workspace(wl.dev, wl.tl, wl.npart, r, p["h_out"], p["h_in"],
                                                                     slot=100 + c), independent=launched > 0)
                        launched += 1
                    if self.exchange:
                        b.reduce_slots(i, s0, s1)
        b.finish()


def capture(step, torch):
    """Warm the step up on a side stream, then capture it into a CUDA graph.  Returns graph.replay."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    return graph.replay


def run_c5(a, rank, world, local, torch, dist, blocks, steps):
    """Workload c5 as a record of its own: device time per step with the exchange, without it (what one
    GPU alone needs for the same work) and the difference, which is the exposed part of the exchange."""
    spec = workload_spec("c5", rank, world)
    if a.seg_len > 0:
        spec["lens"] = [a.seg_len] * len(spec["lens"])
    wl = Workload(spec, torch.device("cuda", local))
    # one rank alone exchanges nothing: its weight gradients stay one launch per projection
    dp = DataParallelStep(wl, torch, dist if world > 1 else None, chunks=a.chunks if world > 1 else 1)
    dp.order = a.c5_order
    T = wl.T
    dp.step()
    torch.cuda.synchronize()
    for pl in wl.plans():
        pl.raise_if_failed()
    rec = dict(workload="c5: " + WORKLOAD_TEXT["c5"], tokens_per_gpu=T, n_gpus=world,
               allreduce_bytes_per_step=dp.bucket.nbytes if world > 1 else 0, slots=dp.bucket.n_slots,
               chunks_of_last_projection=len(dp.ranges), order=dp.order)
    mode = "eager"
    fn = dp.step
    if not a.no_graph:
        try:
            fn = capture(dp.step, torch)
            mode = "cuda graph replay"
        except Exception as e:  # a collective that cannot be captured on this stack: time the eager step
            torch.cuda.synchronize()
            rec["graph_capture_failed"] = str(e).splitlines()[0][:200]
            fn = dp.step
    ms, per = timed(fn, steps, max(3, a.warmup), torch, dist, None, blocks)
    rec.update(ms_per_step=ms, ms_per_step_min=min(per), ms_per_step_max=max(per), blocks=len(per),
               value=T * world / (ms * 1e-3), unit="tokens/s", launch_mode=mode)
    fwd_b, bwd_b = algorithmic_bytes(spec)
    peak, which = hbm_peak()
    rec["step_hbm"] = dict(algorithmic_bytes=fwd_b + bwd_b, achieved_gbs=(fwd_b + bwd_b) / (ms * 1e-3) / 1e9,
                           frac=(fwd_b + bwd_b) / (ms * 1e-3) / 1e9 / peak, peak_gbs=peak, peak_source=which)
    if a.check and world == 1:
        # (with several ranks the slots hold sums over ranks; the 2-GPU test compares those)
        rec["parity_max_rel_err"], rec["parity_share_outside_literal_tolerance"] = check_step(wl, torch)
        rec["parity_checked"] = True
    if world > 1:
        # the step one GPU needs alone for the same work: no exchange, the fused order (per-GPU work is fixed)
        order = dp.order
        dp.exchange, dp.order = False, "fused"
        fn0 = dp.step
        if mode != "eager":
            fn0 = capture(dp.step, torch)
        ms0, _ = timed(fn0, steps, 3, torch, dist, None, max(1, blocks // 2))
        dp.exchange, dp.order = True, order
        rec.update(ms_per_step_without_exchange=ms0, exposed_comm_ms=ms - ms0, efficiency_vs_n1=ms0 / ms)
    return rec


def run_decode(a, rank, world, local, torch, dist, blocks, steps):
    """Decode attention over the paged key-value cache (the step between the q/k/v and o projections of a
    decode batch) with the key/value append in front of it: Llama-3-8B heads (32 query, 8 kv, dim 128),
    page size 16, one layer's pages, 128 one-token requests with context lengths uniform in [512, 4096].
    Requests shard over ranks with no collective.  Algorithmic bytes: every K and V entry of every context
    once, q and o once."""
    from loquetier_b200 import kvcache
    dev = torch.device("cuda", local)
    B, N, G, P, D = 128, 8, 4, 16, 128
    rng = np.random.default_rng(9000 + rank)
    seqlens = [int(v) for v in rng.integers(512, 4097, size=B)]
    pool = kvcache.KvPool(1, N, D, P, torch.bfloat16, dev, pages_per_slab=4096)
    caches = [kvcache.KvCache(pool, L) for L in seqlens]
    for slab in pool._slabs:
        slab.normal_()
    bkv = kvcache.BatchedKvCache(caches)
    g = torch.Generator(device=dev).manual_seed(9000 + rank)
    q = torch.randn((B, N * G, D), generator=g, device=dev).to(torch.bfloat16)
    k = torch.randn((B, N, D), generator=g, device=dev).to(torch.bfloat16)
    v = torch.randn((B, N, D), generator=g, device=dev).to(torch.bfloat16)
    o = torch.empty_like(q)
    ws = kvcache.decode_workspace(dev, B, N * G, N)
    word = torch.zeros(1, dtype=torch.int32, device=dev)

    def step():
        kvcache.append_kv_raw(bkv.ptrs, bkv.indptr, bkv.last_page_offset, k, v, 1, 0, N, P, status_word=word)
        kvcache.batch_decode_into(o, q, bkv.ptrs, bkv.indptr, bkv.last_page_offset, 1, 0, N, 500000.0, P, workspace=ws,
                                  status_word=word)

    step()
    torch.cuda.synchronize()
    assert int(word.item()) == 0, "the kernels recorded a fault"
    fn = capture(step, torch) if not a.no_graph else step
    ms, per = timed(fn, steps, max(3, a.warmup), torch, dist, None, blocks)
    nbytes = 2 * (2 * sum(seqlens) * N * D + 2 * B * N * G * D + 2 * B * N * D)
    peak, which = hbm_peak()
    rec = dict(workload="decode: paged-KV batch decode attention + append, bf16, 128 requests, contexts 512..4096, "
                        "32 query / 8 kv heads of dim 128, page size 16",
               metric="decode attention tokens/s", value=B * world / (ms * 1e-3), unit="tokens/s", n_gpus=world,
               ms_per_step=ms, ms_per_step_min=min(per), ms_per_step_max=max(per), blocks=len(per),
               context_tokens=sum(seqlens), pages=int(bkv.ptrs.numel()),
               l2="%.0f MB of keys and values per step (> 126 MB L2)" % (nbytes / 1e6),
               step_hbm=dict(algorithmic_bytes=nbytes, achieved_gbs=nbytes / (ms * 1e-3) / 1e9,
                             frac=nbytes / (ms * 1e-3) / 1e9 / peak, peak_gbs=peak, peak_source=which),
               launch_mode="eager" if a.no_graph else "cuda graph replay", gpu_launches_per_step=2)
    if a.check and rank == 0:
        from oracle import attention_oracle as AO
        sel = [int(i) for i in np.argsort(seqlens)[[0, B // 2, B - 1]]]   # shortest, median, longest context
        pages = []
        ind, last = [0], []
        for i in sel:
            c = caches[i]
            pages += [pg.cpu() for pg in c.pages]
            ind.append(ind[-1] + c.num_pages)
            last.append(AO.last_page_offset_of(c.seqlen, P))
        want = AO.batch_decode(q[sel].cpu(), pages, ind, last, 0, 500000.0)
        err = (o[sel].cpu().float() - want.float()).abs()
        assert bool((err <= 1e-2 + 1e-2 * want.float().abs()).all()), "decode differs from the oracle"
        for j, i in enumerate(sel):   # the appended key/value sits in the last valid entry
            got = caches[i].pages[-1][0, 0, :, last[j] - 1, :]
            assert torch.equal(got, k[i]), "append differs from the oracle"
        rec["parity_checked"] = True
        rec["parity_max_abs_err"] = float(err.max())
    return rec


def tensor_peak():
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]), "measured (burst)"
    except Exception:
        return 1590.0, "fallback"


def run_prefill(a, rank, world, local, torch, dist, blocks, steps):
    """Causal prefill attention over the paged key-value cache with the copy of the prompts' keys/values
    into the pages in front of it (init_kv): Llama-3-8B heads (32 query, 8 kv, dim 128), page size 16, one
    layer's pages, 32 prompts with lengths uniform in [256, 2048].  Prompts shard over ranks with no
    collective.  The bound is the tensor cores: 4 * head_dim flops per (query, visible key, query head),
    visible keys = positions up to the query's own."""
    from loquetier_b200 import kvcache
    dev = torch.device("cuda", local)
    B, N, G, P, D = 32, 8, 4, 16, 128
    rng = np.random.default_rng(9100 + rank)
    seqlens = [int(v) for v in rng.integers(256, 2049, size=B)]
    T = sum(seqlens)
    pool = kvcache.KvPool(1, N, D, P, torch.bfloat16, dev, pages_per_slab=4096)
    caches = [kvcache.KvCache(pool, L) for L in seqlens]
    bkv = kvcache.BatchedKvCache(caches)
    g = torch.Generator(device=dev).manual_seed(9100 + rank)
    q = torch.randn((T, N * G, D), generator=g, device=dev).to(torch.bfloat16)
    k = torch.randn((T, N, D), generator=g, device=dev).to(torch.bfloat16)
    v = torch.randn((T, N, D), generator=g, device=dev).to(torch.bfloat16)
    o = torch.empty_like(q)
    qind_h = np.concatenate([[0], np.cumsum(seqlens)]).astype(np.int32)
    qind = torch.tensor(qind_h, device=dev)
    word = torch.zeros(1, dtype=torch.int32, device=dev)

    def step():
        kvcache.init_kv_raw(bkv.ptrs, bkv.indptr, bkv.last_page_offset, k, v, qind, 1, 0, N, P, status_word=word)
        kvcache.batch_prefill_into(o, q, qind, bkv.ptrs, bkv.indptr, bkv.last_page_offset, 1, 0, N, 500000.0, P,
                                   status_word=word)

    step()
    torch.cuda.synchronize()
    assert int(word.item()) == 0, "the kernels recorded a fault"
    fn = capture(step, torch) if not a.no_graph else step
    ms, per = timed(fn, steps, max(3, a.warmup), torch, dist, None, blocks)
    flops = float(sum(4 * D * N * G * (L * (L + 1) // 2) for L in seqlens))
    nbytes = 2 * (2 * T * N * G * D + 4 * T * N * D)    # q, o; k, v read and written into the pages
    peak, which = tensor_peak()
    name = ("prefill: paged-KV causal prefill attention + init_kv, bf16, 32 prompts of 256..2048 tokens, "
            "32 query / 8 kv heads of dim 128, page size 16")
    rec = dict(workload=name, metric="prefill attention tokens/s", value=T * world / (ms * 1e-3), unit="tokens/s",
               n_gpus=world, ms_per_step=ms, ms_per_step_min=min(per), ms_per_step_max=max(per), blocks=len(per),
               prompt_tokens=T, pages=int(bkv.ptrs.numel()),
               l2="%.0f MB of q, o, k, v per step (> 126 MB L2)" % (nbytes / 1e6),
               roofline=dict(bound="tensor", achieved=flops / (ms * 1e-3) / 1e12, peak=peak, unit="TFLOP/s",
                             frac=flops / (ms * 1e-3) / 1e12 / peak, peak_source=which, traffic=None,
                             algorithmic_flops=flops,
                             note="causal flops only (visible keys); the step also holds the init_kv copy"),
               launch_mode="eager" if a.no_graph else "cuda graph replay", gpu_launches_per_step=3)
    if a.check and rank == 0:
        from oracle import attention_oracle as AO
        sel = [int(i) for i in np.argsort(seqlens)[[0, B // 2]]]   # the shortest and the median prompt
        pages, ind, last, qi, rows = [], [0], [], [0], []
        for i in sel:
            c = caches[i]
            pages += [pg.cpu() for pg in c.pages]
            ind.append(ind[-1] + c.num_pages)
            last.append(AO.last_page_offset_of(c.seqlen, P))
            qi.append(qi[-1] + seqlens[i])
            rows += list(range(int(qind_h[i]), int(qind_h[i + 1])))
        want = AO.batch_prefill(q[rows].cpu(), qi, pages, ind, last, 0, 500000.0)
        err = (o[rows].cpu().float() - want.float()).abs()
        assert bool((err <= 1e-2 + 1e-2 * want.float().abs()).all()), "prefill differs from the oracle"
        rec["parity_checked"] = True
        rec["parity_max_abs_err"] = float(err.max())
    return rec


def run_linear_host(a, local, torch):
    """Host time of one eager MixedLoraLinear.forward - what a model pays per LoRA linear and step on top
    of the kernels: wall clock around many forwards without a synchronisation in between, for the segment
    counts of c2 (70) and c4 (1024).  The context (plan, adapter index) is built once per step, as in a
    model where all LoRA linears share it."""
    from loquetier_b200.kernel_utils import BatchLenInfo
    from loquetier_b200.mixed_lora import MixedLoraContext, MixedLoraLinear, NamedLoraLayer
    dev = torch.device("cuda", local)
    out = {}
    for name in ("c2", "c4"):
        spec = workload_spec(name)
        dt = torch.float16 if spec["dtype"] == "fp16" else torch.bfloat16
        _, hi, ho = spec["projections"][0]
        r, n_ad = spec["rank"], spec["n_adapters"]
        g = torch.Generator(device=dev).manual_seed(1)
        base = torch.nn.Linear(hi, ho, bias=False, dtype=dt, device=dev)
        ads = [NamedLoraLayer(f"a{i}", (torch.randn((r, hi), generator=g, device=dev) / np.sqrt(hi)).to(dt),
                              (torch.randn((ho, r), generator=g, device=dev) * 0.02).to(dt), torch.nn.Identity(), 2.0)
               for i in range(n_ad)]
        ctx = MixedLoraContext()
        lin = MixedLoraLinear(ctx, base, ads, r, dt)
        lens, ids = spec["lens"], spec["ids"]
        seg = torch.tensor(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32), device=dev)
        blen = BatchLenInfo([], [], 0, [], dev)
        ctx.update(blen, ids, torch.tensor(lens, dtype=torch.int32, device=dev), seg, [])
        x = torch.randn((sum(lens), hi), generator=g, device=dev).to(dt)
        with torch.no_grad():
            for _ in range(5):
                lin(x)
            torch.cuda.synchronize()
            n = 200
            t0 = time.perf_counter()
            for _ in range(n):
                lin(x)
            t1 = time.perf_counter()
            torch.cuda.synchronize()
            t2 = time.perf_counter()
        out[name] = dict(segments=len(lens), host_us_per_forward=(t1 - t0) / n * 1e6,
                         device_bound_us_per_forward=(t2 - t0) / n * 1e6)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="c3", choices=["c2", "c3", "c4", "c4s", "c5", "rmsnorm", "linear", "decode", "prefill"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--blocks", type=int, default=25, help="timed blocks of --steps steps; the median is reported")
    ap.add_argument("--sched", default="multi", choices=["multi", "multi_s", "multi_f", "split", "split2", "split3", "single"],
                    help="multi: one launch per kernel class over all projections (dV/dX, forward, weight "
                         "gradients); multi_f: the same with the forward first; split: the forward of the inference "
                         "rows on a second stream; single: one launch per projection")
    ap.add_argument("--no-check", dest="check", action="store_false",
                    help="skip the comparison of every output of the timed step with the CPU oracle (rank 0)")
    ap.add_argument("--no-extras", action="store_true", help="c3 only: skip the c5 and rmsnorm records")
    ap.add_argument("--c5-order", default="fused", choices=["fused", "grads_first"],
                    help="c5: fused = dV/dX in one launch per projection; grads_first = dV early, dX last, so that the "
                         "exchange of all weight gradients runs under the dX launches (measured: no faster at two GPUs)")
    ap.add_argument("--chunks", type=int, default=1, help="c5: slot ranges of the last projection's exchange")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--e2e-blocks", type=int, default=4, help="row blocks the end-to-end step cuts the batch into")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-overlap", action="store_true", help="do not mark launches independent of each other")
    ap.add_argument("--streams", type=int, default=3, help="single: streams the backward launches are dealt over")
    ap.add_argument("--no-breakdown", action="store_true", help="skip the per-kernel-class timing pass")
    ap.add_argument("--only", default="", help="comma-separated projection names: restrict the workload "
                                               "(for profiler captures of one shape)")
    ap.add_argument("--no-group", action="store_true", help="plan without grouping short segments by adapter")
    ap.add_argument("--ks", type=int, default=0, help="force the cluster split of the fused kernel (measurements)")
    ap.add_argument("--seg-len", type=int, default=0, help="c5 only: tokens per segment instead of 2048 "
                                                          "(a smaller footprint for profiler captures)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    a.blocks = max(1, a.blocks)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    import torch

    if a.workload == "rmsnorm":
        line = run_rmsnorm(a, rank, world, local, torch)
        if line is not None and rank == 0:
            print(json.dumps(line))
        return
    if a.workload in ("decode", "prefill"):
        assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
        torch.cuda.set_device(local)
        dist = None
        if world > 1:
            import torch.distributed as dist_mod
            dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist = dist_mod
        rec = (run_decode if a.workload == "decode" else run_prefill)(a, rank, world, local, torch, dist, a.blocks,
                                                                     a.steps)
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        if rank == 0:
            rec.update(steps=a.steps, warmup=a.warmup, higher_is_better=True, scaling="weak", vs_baseline=None,
                       dtype="bf16", data="synthetic", config=dict(workload=rec["workload"]))
            print(json.dumps(rec))
        return
    if a.workload == "linear":
        assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
        print(json.dumps(dict(metric="host microseconds per eager MixedLoraLinear.forward", unit="us",
                              higher_is_better=False, data="synthetic", result=run_linear_host(a, local, torch))))
        return
    spec = workload_spec(a.workload, rank, world)
    if a.seg_len > 0:
        assert a.workload == "c5", "--seg-len applies to c5"
        spec["lens"] = [a.seg_len] * len(spec["lens"])
    if a.only:
        keep = set(a.only.split(","))
        spec["projections"] = [p for p in spec["projections"] if p[0] in keep]
        assert spec["projections"], "--only matched no projection of the workload"
    T = sum(spec["lens"])
    fwd_b, bwd_b = algorithmic_bytes(spec)
    cfg = dict(workload=f"{a.workload}: " + WORKLOAD_TEXT[a.workload],
        tokens_per_gpu=T, segments=len(spec["lens"]), finetune_tokens=sum(l for l, f in zip(spec["lens"], spec["ft"]) if f),
        l2="one step touches %.0f MB of distinct operands (> 126 MB L2); nothing is reused between steps"
           % ((fwd_b + bwd_b) / 1e6),
        sharding="segments partitioned by adapter owner (adapter mod N), no collective" if a.workload != "c5"
                 else "data parallel; dA/dB of the adapters some rank trains are summed over the ranks, slot range "
                      "by slot range, each range started behind the kernel that produces it")

    if a.impl == "reference":
        if rank != 0:
            return
        base, sec = run_cpu(spec, torch, budget_s=min(90.0, max(10.0, 0.5 * a.steps)), max_reps=max(1, a.steps))
        line = dict(metric="SMLM fwd+bwd tokens/s", value=base["value"], unit="tokens/s", n_gpus=a.gpus,
                    steps=a.steps, warmup=a.warmup, ms_per_step=sec * 1e3, higher_is_better=True, scaling="weak",
                    vs_baseline=None, dtype="fp32 on CPU (16-bit inputs upcast)", data="synthetic", config=cfg,
                    impl="reference", cpu_baseline=base,
                    e2e=dict(value=base["value"], unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                    gpu_launches=0)
        print(json.dumps(line))
        return

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    numa = bind_to_gpu_numa_node(local) if world > 1 else None
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        try:
            # the exchange of c5 runs next to kernels that fill every SM: give NCCL's stream priority
            opts = dist_mod.ProcessGroupNCCL.Options(is_high_priority_stream=True)
            dist_mod.init_process_group("nccl", device_id=dev, pg_options=opts)
        except Exception:
            dist_mod.init_process_group("nccl", device_id=dev)
        dist = dist_mod
    peak, which = hbm_peak()

    if a.workload == "c5":
        rec = run_c5(a, rank, world, local, torch, dist, a.blocks, a.steps)
        line = dict(metric="SMLM fwd+bwd tokens/s", value=rec["value"], unit="tokens/s", n_gpus=world, steps=a.steps,
                    warmup=a.warmup, ms_per_step=rec["ms_per_step"], higher_is_better=True, scaling="weak",
                    vs_baseline=None, dtype=spec["dtype"], data="synthetic", config=cfg, c5=rec,
                    gpu_launches=(2 + 2 * 2 + 1 + rec["chunks_of_last_projection"]) * a.steps,
                    launch_mode=rec["launch_mode"], step_hbm=rec["step_hbm"])
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        if rank == 0:
            print(json.dumps(line))
        return

    if a.ks:
        from loquetier_b200 import ops as _ops
        _ops.set_cluster_split(a.ks)
    wl = Workload(spec, dev)
    wl.overlap = not a.no_overlap
    wl.grouped = not a.no_group
    wl.n_streams = a.streams
    wl.sched = a.sched

    wl.step()
    torch.cuda.synchronize()
    for pl in wl.plans():
        pl.raise_if_failed()

    use_graph = not a.no_graph
    step_fn = capture(wl.step, torch) if use_graph else wl.step

    with ClockSampler(local) as clk:
        time.sleep(0.3)  # let the sampler come up so that its samples fall inside the timed region
        ms, per = timed(step_fn, a.steps, a.warmup, torch, dist, clk, a.blocks)
    tokens_all = T * world
    value = tokens_all / (ms * 1e-3)

    line = dict(metric="SMLM fwd+bwd tokens/s", value=value, unit="tokens/s", n_gpus=world, steps=a.steps,
                warmup=a.warmup, ms_per_step=ms, ms_per_step_min=min(per), ms_per_step_max=max(per),
                blocks=len(per), higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype=spec["dtype"], data="synthetic", config=cfg, clocks=clk.result,
                gpu_launches=wl.launches_per_step * a.steps * len(per), gpu_launches_per_step=wl.launches_per_step,
                launch_mode="cuda graph replay" if use_graph else "eager", sched=wl.sched)
    if numa is not None:
        line["numa_node"] = numa

    if a.check and rank == 0:
        # the outputs in device memory are those of the last replay of the very step that was timed
        torch.cuda.synchronize()
        for pl in wl.plans():
            pl.raise_if_failed()
        worst, outside = check_step(wl, torch)
        line["parity_checked"] = True
        line["parity_max_rel_err"] = worst
        line["parity_share_outside_literal_tolerance"] = outside

    if rank == 0:
        line["step_hbm"] = dict(algorithmic_bytes=fwd_b + bwd_b, achieved_gbs=(fwd_b + bwd_b) / (ms * 1e-3) / 1e9,
                                frac=(fwd_b + bwd_b) / (ms * 1e-3) / 1e9 / peak, peak_gbs=peak, peak_source=which)
    if rank == 0 and not a.no_breakdown:
        kb = kernel_breakdown(wl, torch)
        top = max(kb, key=lambda k: kb[k][0])
        t_ms, nbytes, nl = kb[top]
        ach = nbytes / (t_ms * 1e-3) / 1e9
        # DRAM bytes of one launch from the ncu capture of this very workload (seeded, so every run moves the
        # same bytes); null for any other workload or restriction of it
        traffic = C3_TRAFFIC.get(top) if (a.workload == "c3" and not a.only and world == 1) else None
        line["roofline"] = dict(bound="hbm", kernel=top, achieved=ach, peak=peak, unit="GB/s", frac=ach / peak,
                                peak_source=which, traffic=traffic, launches_per_step=nl,
                                avg_launch_us=t_ms * 1e3 / nl, algorithmic_bytes_per_launch=nbytes / nl)
        line["kernels"] = {k: dict(ms_per_step=v[0], gbs=v[1] / (v[0] * 1e-3) / 1e9, frac=v[1] / (v[0] * 1e-3) / 1e9 / peak,
                                   launches=v[2], share=v[0] / sum(x[0] for x in kb.values())) for k, v in kb.items()}

    if not a.no_e2e:
        hp = HostPipeline(wl, torch, nblocks=a.e2e_blocks)
        e_ms, e_per = timed(hp.step, max(3, min(a.steps, 10)), 3, torch, dist, None, 3)
        for pl in hp.plans:
            pl.raise_if_failed()
        line["e2e"] = dict(value=tokens_all / (e_ms * 1e-3), unit="tokens/s", h2d_bytes_per_step=hp.h2d_bytes,
                           d2h_bytes_per_step=hp.d2h_bytes, ms_per_step=e_ms,
                           host_gbs_all_ranks=(hp.h2d_bytes + hp.d2h_bytes) * world / (e_ms * 1e-3) / 1e9,
                           units=len(hp.units),
                           note="inputs from pinned host memory, results to pinned host memory; every (projection, "
                                "row block) is uploaded, computed and downloaded on its own streams, so the copies of "
                                "one unit overlap the kernels and copies of the others; bound by the host link")
        if a.check and rank == 0:
            line["e2e"]["parity_max_rel_err"] = check_step(wl, torch)[0]
        # what the host link alone takes for a step's bytes (after the check: it overwrites the host results
        # with the same device results, nothing else)
        l_ms, _ = timed(hp.copies_only, max(3, min(a.steps, 10)), 3, torch, dist, None, 3)
        line["e2e"]["host_link"] = dict(copies_only_ms=l_ms, frac=l_ms / e_ms,
                                        note="the step's uploads and downloads alone, both directions at once, "
                                             "measured in this run; frac = that time / the end-to-end step")
    if a.workload == "c3" and not a.no_extras and not a.only:
        del wl, step_fn
        if not a.no_e2e:
            del hp
        torch.cuda.empty_cache()
        line["c5"] = run_c5(a, rank, world, local, torch, dist, max(3, a.blocks // 5), max(5, min(a.steps, 20)))
        torch.cuda.empty_cache()
        sub = argparse.Namespace(**vars(a))
        sub.no_e2e, sub.no_cpu, sub.blocks = True, True, max(3, a.blocks // 5)
        rms = run_rmsnorm(sub, rank, world, local, torch, dist=dist, own_group=False)
        if rms is not None:
            line["rmsnorm"] = {k: rms[k] for k in ("metric", "value", "unit", "ms_per_step", "step_hbm", "kernels",
                                                   "config") if k in rms}
        torch.cuda.empty_cache()
        dec = run_decode(sub, rank, world, local, torch, dist, max(3, a.blocks // 5), max(5, min(a.steps, 20)))
        if rank == 0:
            line["attention_decode"] = dec
        torch.cuda.empty_cache()
        pre = run_prefill(sub, rank, world, local, torch, dist, max(3, a.blocks // 5), max(5, min(a.steps, 20)))
        if rank == 0:
            line["attention_prefill"] = pre
    if rank == 0 and world == 1 and not a.no_cpu:
        base, _ = run_cpu(spec, torch)
        line["cpu_baseline"] = base
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


# ---------------------------------------------------------------------------
# RMSNorm, the caller on either side of the projections (--workload rmsnorm)
# ---------------------------------------------------------------------------

def run_rmsnorm(a, rank, world, local, torch, dist=None, own_group=True):
    """Forward + backward of the Llama-3-8B RMSNorm over 32768 token rows of 4096 columns, bf16.
    Rows shard over ranks with no collective (every rank holds the same weight; its dW would join the
    gradient all-reduce of the model, which is not part of this operator).  Returns the JSON line as a
    dict on rank 0 (None elsewhere); with ``own_group`` false it runs inside the caller's process group."""
    from oracle import smlm_oracle as O
    rows, cols, eps = 32768, 4096, 1e-5
    e = 2
    fwd_b = e * (2 * rows * cols + cols) + 4 * rows
    bwd_b = e * (3 * rows * cols + 2 * cols) + 4 * rows
    cfg = dict(workload="rmsnorm: Llama-3-8B RMSNorm forward + backward, bf16, 32768 token rows x 4096 columns",
               tokens_per_gpu=rows, l2="one step touches %.0f MB of distinct operands (> 126 MB L2)" % ((fwd_b + bwd_b) / 1e6),
               sharding="rows partitioned over ranks, no collective")
    g = torch.Generator().manual_seed(7000 + rank)

    def cpu_data(n):
        x = (torch.randn((n, cols), generator=g) * 1.5).to(torch.bfloat16)
        w = (1.0 + 0.1 * torch.randn((cols,), generator=g)).to(torch.bfloat16)
        go = torch.randn((n, cols), generator=g).to(torch.bfloat16)
        return x, w, go

    def cpu_leg(budget_s, max_reps):
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        x, w, go = cpu_data(rows)

        def fn():
            o, m = O.rms_norm_forward(x, w, eps)
            O.rms_norm_backward(go, x, w, m)
        fn()
        times, t_all = [], time.perf_counter()
        while len(times) < max_reps and (time.perf_counter() - t_all) < budget_s:
            t0 = time.perf_counter()
            fn()
            times.append(time.perf_counter() - t0)
        sec = float(np.median(times))
        return dict(value=rows / sec, unit="tokens/s", cores=cores, kind="port",
                    sample=f"{len(times)} full steps ({rows} rows x {cols}, fwd+bwd) of the fp32 restatement with "
                           f"torch.set_num_threads({cores}); median {sec * 1e3:.1f} ms/step"), sec

    if a.impl == "reference":
        if rank != 0:
            return
        base, sec = cpu_leg(min(90.0, max(10.0, 0.5 * a.steps)), max(1, a.steps))
        return dict(metric="RMSNorm fwd+bwd tokens/s", value=base["value"], unit="tokens/s", n_gpus=a.gpus,
                    steps=a.steps, warmup=a.warmup, ms_per_step=sec * 1e3, higher_is_better=True,
                    scaling="weak", vs_baseline=None, dtype="fp32 on CPU (16-bit inputs upcast)",
                    data="synthetic", config=cfg, impl="reference", cpu_baseline=base, gpu_launches=0,
                    e2e=dict(value=base["value"], unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    from loquetier_b200 import ops
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and own_group:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=dev)
        dist = dist_mod
    gd = torch.Generator(device=dev).manual_seed(7000 + rank)
    x = (torch.randn((rows, cols), generator=gd, device=dev) * 1.5).to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn((cols,), generator=gd, device=dev)).to(torch.bfloat16)
    go = torch.randn((rows, cols), generator=gd, device=dev).to(torch.bfloat16)
    o, dx = torch.empty_like(x), torch.empty_like(x)
    m = torch.empty((rows, 1), dtype=torch.float32, device=dev)
    dw = torch.empty((cols,), dtype=torch.bfloat16, device=dev)
    ws = torch.empty(max(16, int(ops.lib.smlm_b200_rms_norm_bwd_workspace_bytes(rows, cols))), dtype=torch.uint8,
                     device=dev)

    def step():
        ops.rms_norm(o, m, x, w, eps)
        ops.rms_norm_bwd(dx, dw, go, x, w, m, workspace=ws)

    step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph):
        step()
    with ClockSampler(local) as clk:
        time.sleep(0.3)
        ms, per = timed(graph.replay, a.steps, a.warmup, torch, dist, clk, a.blocks)
    line = dict(metric="RMSNorm fwd+bwd tokens/s", value=rows * world / (ms * 1e-3), unit="tokens/s", n_gpus=world,
                steps=a.steps, warmup=a.warmup, ms_per_step=ms, ms_per_step_min=min(per), ms_per_step_max=max(per),
                blocks=len(per), higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="bf16", data="synthetic", config=cfg, clocks=clk.result,
                gpu_launches=3 * a.steps * len(per), launch_mode="cuda graph replay")
    if rank == 0:
        peak, which = hbm_peak()
        line["step_hbm"] = dict(algorithmic_bytes=fwd_b + bwd_b, achieved_gbs=(fwd_b + bwd_b) / (ms * 1e-3) / 1e9,
                                frac=(fwd_b + bwd_b) / (ms * 1e-3) / 1e9 / peak, peak_gbs=peak, peak_source=which)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        kern = {}
        for name, fn, nb in (("rms_norm_fwd_kernel", lambda: ops.rms_norm(o, m, x, w, eps), fwd_b),
                             ("rms_norm_bwd_kernel + rms_norm_dw_kernel",
                              lambda: ops.rms_norm_bwd(dx, dw, go, x, w, m, workspace=ws), bwd_b)):
            tot = 0.0
            for it in range(6):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); fn(); e1.record()
                torch.cuda.synchronize()
                if it:
                    tot += e0.elapsed_time(e1)
            t = tot / 5
            kern[name] = dict(ms_per_step=t, gbs=nb / (t * 1e-3) / 1e9, frac=nb / (t * 1e-3) / 1e9 / peak)
        top = max(kern, key=lambda k: kern[k]["ms_per_step"])
        line["kernels"] = kern
        line["roofline"] = dict(bound="hbm", kernel=top, achieved=kern[top]["gbs"], peak=peak, unit="GB/s",
                                frac=kern[top]["frac"], peak_source=which, traffic=None)
    if not a.no_e2e:
        hx, hg = x.cpu().pin_memory(), go.cpu().pin_memory()
        ho, hdx = torch.empty_like(hx).pin_memory(), torch.empty_like(hx).pin_memory()
        hdw = torch.empty((cols,), dtype=torch.bfloat16).pin_memory()

        def e2e_step():
            x.copy_(hx, non_blocking=True)
            go.copy_(hg, non_blocking=True)
            step()
            ho.copy_(o, non_blocking=True)
            hdx.copy_(dx, non_blocking=True)
            hdw.copy_(dw, non_blocking=True)
        e_ms, _ = timed(e2e_step, max(3, min(a.steps, 10)), 3, torch, dist)
        line["e2e"] = dict(value=rows * world / (e_ms * 1e-3), unit="tokens/s", h2d_bytes_per_step=2 * rows * cols * e,
                           d2h_bytes_per_step=2 * rows * cols * e + cols * e, ms_per_step=e_ms)
    if rank == 0 and world == 1 and not a.no_cpu:
        line["cpu_baseline"], _ = cpu_leg(12.0, 5)
    if dist is not None and own_group:
        dist.barrier()
        dist.destroy_process_group()
    return line if rank == 0 else None


if __name__ == "__main__":
    main()
