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

# DRAM bytes (read + written during the launch) per algorithmic byte of the forward fused launch, from
# the ncu capture summarised in profiles/fused_kernel_c3_q_proj.md: (70.82 + 9.56) MB / 138.7 MB.  Part of
# the freshly written output is still dirty in L2 when the launch ends, hence a ratio below one.
TRAFFIC_PER_ALGORITHMIC_BYTE = 0.58


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
        ids = [int(v) for v in rng.choice(n_ad, size=16, replace=False)]
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
        self.ops = ops
        self.accumulate_grads = False
        self.grouped = True
        self.after_wgrad = None  # callable(projection index), called on the stream of its weight gradients
        self.overlap = True
        self.n_streams = 3
        self.side = []
        self.torch = torch

    def build_plans(self):
        # grouped where it changes anything: decode tokens are gathered by adapter for the forward launches
        from loquetier_b200.segments import wants_grouped_plan
        g = self.grouped and wants_grouped_plan(self.spec["lens"], self.spec["ids"])
        self.plan = self.ops.Plan(self.seg, self.T, seg_ids=self.ids if g else None, n_table=self.spec["n_adapters"])
        if self.tl:
            self.pplan = self.ops.Plan(self.part, self.tl)

    # one plan per index pointer, then 1 forward and 2 backward kernels per projection
    launches_per_step = property(lambda self: 1 + (1 if self.tl else 0)
                                 + len(self.proj) * (1 + (2 if self.tl else 0)))

    def step(self):
        """The hot path: plans once, then for every projection the fused forward, the fused
        dV/dX backward and the weight gradients.  The projections are independent of each other,
        so the launches of one kind are issued back to back and marked independent: the read
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


def timed(fn, steps, warmup, torch, dist=None, clk=None):
    """W untimed + K timed iterations bracketed by barrier + synchronize; device
    time from CUDA events on the current stream; max over ranks."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if clk is not None:
        clk.mark_start()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if clk is not None:
        clk.mark_end()
    if dist is not None:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps


def kernel_breakdown(wl, torch, reps=5):
    """Device time of every kernel class over one step, measured by launching the
    class back to back for all projections between two events (so that launch gaps
    do not count), through the same C-ABI entry points the fused calls use.
    Returns {class: (ms per step, algorithmic bytes per step, launches per step)}."""
    ops, r, e = wl.ops, wl.spec["rank"], 2
    used = len(set(wl.spec["ids"]))
    used_ft = len(set(wl.spec["ids"][:wl.npart]))
    T, n = wl.T, wl.tl
    wl.build_plans()
    for p in wl.proj:  # make v / dv valid for the classes that read them
        ops.fwd(p["y"], p["x"], p["v"], p["wa"], p["wb"], wl.plan, r, seg_ids=wl.ids, seg_scale=wl.scale)
        if n:
            ops.bwd(p["dx"], p["dA_t"], p["dB_t"], p["dv"], p["go"], p["x"], p["v"], p["wa"], p["wb"], wl.pplan,
                    r, part_ids=wl.part_ids, part_scale=wl.scale)
    classes = {
        "fused_kernel(fwd x->v->y)": (
            lambda p, i: ops.fwd(p["y"], p["x"], p["v"], p["wa"], p["wb"], wl.plan, r, seg_ids=wl.ids,
                                 seg_scale=wl.scale, independent=wl.overlap and i > 0),
            lambda p: e * (T * p["h_in"] + T * p["h_out"] + T * r + used * r * (p["h_in"] + p["h_out"]))),
    }
    if n:
        classes.update({
            "fused_kernel(bwd gO->dV->dX)": (
                lambda p, i: ops.bwd_dx(p["dx"], p["dv"], p["go"], p["wa"], p["wb"], wl.pplan, r,
                                        part_ids=wl.part_ids, part_scale=wl.scale,
                                        independent=wl.overlap and i > 0),
                lambda p: e * (n * p["h_out"] + n * p["h_in"] + n * r + used_ft * r * (p["h_in"] + p["h_out"]))),
            "wgrad_kernel(dB=gO^T.V, dA=dV^T.X)": (
                lambda p, i: ops.wgrad_pair(p["dA_t"], p["dB_t"], p["dv"], p["x"], p["v"], p["go"], wl.part, wl.pplan,
                                            r, part_ids=wl.part_ids, part_scale=wl.scale,
                                            n_table=wl.spec["n_adapters"],
                                            workspace=ops.wgrad_workspace(wl.dev, n, wl.npart, r, p["h_out"],
                                                                          p["h_in"], slot=i),
                                            independent=wl.overlap and i > 0),
                lambda p: e * (n * (p["h_in"] + p["h_out"]) + 2 * n * r + used_ft * r * (p["h_in"] + p["h_out"]))),
        })
    out = {}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=wl.dev)
    for name, (fn, nbytes) in classes.items():
        tot = 0.0
        for it in range(reps + 1):
            flush.zero_()  # evict L2 between repetitions of the same class
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i, p in enumerate(wl.proj):
                fn(p, i)
            e1.record()
            torch.cuda.synchronize()
            if it > 0:
                tot += e0.elapsed_time(e1)
        out[name] = (tot / reps, float(sum(nbytes(p) for p in wl.proj)), len(wl.proj))
    return out


# ---------------------------------------------------------------------------
# end to end through host buffers
# ---------------------------------------------------------------------------

class HostPipeline:
    """The step with HOST inputs and outputs: x and gO of every projection start in
    pinned host memory, y, dX, dA and dB end in pinned host memory.  Copies run on
    their own streams so that the upload of projection p+1 and the download of
    projection p-1 overlap the kernels of projection p."""

    def __init__(self, wl, torch):
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

    def step(self):
        torch, wl, ops = self.torch, self.wl, self.wl.ops
        cur = torch.cuda.current_stream()
        r = wl.spec["rank"]
        self.s_in.wait_stream(cur)
        self.s_out.wait_stream(cur)
        wl.build_plans()
        ready = []
        with torch.cuda.stream(self.s_in):
            for p, h in zip(wl.proj, self.h):
                p["x"].copy_(h["x"], non_blocking=True)
                if wl.tl:
                    p["go"].copy_(h["go"], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.s_in)
                ready.append(ev)
        for p, h, ev in zip(wl.proj, self.h, ready):
            cur.wait_event(ev)
            ops.fwd(p["y"], p["x"], p["v"], p["wa"], p["wb"], wl.plan, r, seg_ids=wl.ids, seg_scale=wl.scale)
            if wl.tl:
                ops.bwd(p["dx"], p["dA_t"], p["dB_t"], p["dv"], p["go"], p["x"], p["v"], p["wa"], p["wb"],
                        wl.pplan, r, part_ids=wl.part_ids, part_scale=wl.scale)
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                h["y"].copy_(p["y"], non_blocking=True)
                if wl.tl:
                    h["dx"].copy_(p["dx"], non_blocking=True)
                    h["dA"].copy_(p["dA"], non_blocking=True)
                    h["dB"].copy_(p["dB"], non_blocking=True)
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

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="c3", choices=["c2", "c3", "c4", "c4s", "c5", "rmsnorm"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-overlap", action="store_true", help="do not mark launches independent of each other")
    ap.add_argument("--streams", type=int, default=3, help="streams the backward launches are dealt over")
    ap.add_argument("--no-breakdown", action="store_true", help="skip the per-kernel-class timing pass")
    ap.add_argument("--only", default="", help="comma-separated projection names: restrict the workload "
                                               "(for profiler captures of one shape)")
    ap.add_argument("--no-group", action="store_true", help="plan without grouping short segments by adapter")
    ap.add_argument("--seg-len", type=int, default=0, help="c5 only: tokens per segment instead of 2048 "
                                                          "(a smaller footprint for profiler captures)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    import torch

    if a.workload == "rmsnorm":
        return run_rmsnorm(a, rank, world, local, torch)
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
    cfg = dict(workload=f"{a.workload}: " + {
        "c2": "Llama-2-7B q_proj mixed batch, fp16, rank 16, 32 adapters, 2x1024 FT + 4x512 prefill + 64 decode",
        "c3": "Llama-3-8B 7 LoRA projections of one layer, bf16, rank 16, 128 adapters, 8192 tokens, "
              "Zipf(1.2) segment lengths in [1,2048], 25% fine-tune tokens (fwd+bwd), rest forward only",
        "c4": "decode sweep, bf16, 1024 one-token segments, 256 adapters, rank 32, 4096->11008 and 11008->4096",
        "c4s": "decode sweep as c4 with the tokens sorted by adapter and merged into segments, as the "
               "reference's batch assembler orders decode requests",
        "c5": "fine-tune heavy, bf16, rank 64, 64 adapters, 16x2048 FT tokens per GPU, 4096<->14336, "
              "dA/dB all-reduced over NCCL"}[a.workload],
        tokens_per_gpu=T, segments=len(spec["lens"]), finetune_tokens=sum(l for l, f in zip(spec["lens"], spec["ft"]) if f),
        l2="one step touches %.0f MB of distinct operands (> 126 MB L2); nothing is reused between steps"
           % ((fwd_b + bwd_b) / 1e6),
        sharding="segments partitioned by adapter owner (adapter mod N), no collective" if a.workload != "c5"
                 else "data parallel, one all-reduce per projection of its dA/dB slice, started behind its weight-gradient kernel")

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
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=dev)
        dist = dist_mod

    wl = Workload(spec, dev)
    wl.overlap = not a.no_overlap
    wl.grouped = not a.no_group
    wl.n_streams = a.streams
    bucket = None
    if a.workload == "c5":
        # data-parallel fine-tuning: dA/dB of all adapters live in one flat bucket that the backward
        # kernels accumulate into and that is all-reduced once per step
        from loquetier_b200.dp import GradBucket
        bucket = GradBucket([(p["h_in"], p["h_out"]) for p in wl.proj], spec["n_adapters"], spec["rank"], wl.dt, dev)
        for i, p in enumerate(wl.proj):
            p["dA_t"], p["dB_t"] = bucket.tables(i, wl.part_ids)
            p["dA"], p["dB"] = bucket.dA[i], bucket.dB[i]
        wl.accumulate_grads = True
        cfg["allreduce_bytes_per_step"] = bucket.nbytes
        # the exchange of a projection starts right behind its weight-gradient kernel and runs under
        # the backward of the next projection
        wl.after_wgrad = bucket.reduce_projection

    def eager_step():
        if bucket is not None:
            bucket.zero()
        wl.step()
        if bucket is not None:
            bucket.finish()

    eager_step()
    torch.cuda.synchronize()
    wl.plan.raise_if_failed()
    if wl.pplan is not None:
        wl.pplan.raise_if_failed()

    use_graph = not a.no_graph and not (bucket is not None and world > 1)
    if use_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                eager_step()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            eager_step()
        step_fn = graph.replay
    else:
        step_fn = eager_step

    with ClockSampler(local) as clk:
        time.sleep(0.3)  # let the sampler come up so that its samples fall inside the timed region
        ms = timed(step_fn, a.steps, a.warmup, torch, dist, clk)
    tokens_all = T * world
    value = tokens_all / (ms * 1e-3)

    line = dict(metric="SMLM fwd+bwd tokens/s", value=value, unit="tokens/s", n_gpus=world, steps=a.steps,
                warmup=a.warmup, ms_per_step=ms, higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype=spec["dtype"], data="synthetic", config=cfg, clocks=clk.result,
                gpu_launches=wl.launches_per_step * a.steps,
                launch_mode="cuda graph replay" if use_graph else "eager")

    if rank == 0:
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
            peak, which = float(peaks["hbm_gbs"]), "measured"
        except Exception:
            peak, which = 6650.0, "fallback"
        line["step_hbm"] = dict(algorithmic_bytes=fwd_b + bwd_b, achieved_gbs=(fwd_b + bwd_b) / (ms * 1e-3) / 1e9,
                                frac=(fwd_b + bwd_b) / (ms * 1e-3) / 1e9 / peak, peak_gbs=peak, peak_source=which)
    if rank == 0 and not a.no_breakdown:
        kb = kernel_breakdown(wl, torch)
        top = max(kb, key=lambda k: kb[k][0])
        t_ms, nbytes, nl = kb[top]
        ach = nbytes / (t_ms * 1e-3) / 1e9
        line["roofline"] = dict(bound="hbm", kernel=top, achieved=ach, peak=peak, unit="GB/s", frac=ach / peak,
                                peak_source=which, traffic=(ach and nbytes / nl * TRAFFIC_PER_ALGORITHMIC_BYTE) if top.startswith('fused_kernel(fwd') else None,
                                launches_per_step=nl,
                                avg_launch_us=t_ms * 1e3 / nl, algorithmic_bytes_per_launch=nbytes / nl)
        line["kernels"] = {k: dict(ms_per_step=v[0], gbs=v[1] / (v[0] * 1e-3) / 1e9, frac=v[1] / (v[0] * 1e-3) / 1e9 / peak,
                                   share=v[0] / sum(x[0] for x in kb.values())) for k, v in kb.items()}

    if not a.no_e2e:
        hp = HostPipeline(wl, torch)
        e_ms = timed(hp.step, max(3, min(a.steps, 10)), 3, torch, dist)
        line["e2e"] = dict(value=tokens_all / (e_ms * 1e-3), unit="tokens/s", h2d_bytes_per_step=hp.h2d_bytes,
                           d2h_bytes_per_step=hp.d2h_bytes, ms_per_step=e_ms,
                           note="inputs from pinned host memory, results to pinned host memory, copies "
                                "overlapped with kernels on separate streams")
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

def run_rmsnorm(a, rank, world, local, torch):
    """Forward + backward of the Llama-3-8B RMSNorm over 32768 token rows of 4096 columns, bf16.
    Rows shard over ranks with no collective (every rank holds the same weight; its dW would join the
    gradient all-reduce of the model, which is not part of this operator)."""
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
        print(json.dumps(dict(metric="RMSNorm fwd+bwd tokens/s", value=base["value"], unit="tokens/s", n_gpus=a.gpus,
                              steps=a.steps, warmup=a.warmup, ms_per_step=sec * 1e3, higher_is_better=True,
                              scaling="weak", vs_baseline=None, dtype="fp32 on CPU (16-bit inputs upcast)",
                              data="synthetic", config=cfg, impl="reference", cpu_baseline=base, gpu_launches=0,
                              e2e=dict(value=base["value"], unit="tokens/s", h2d_bytes_per_step=0,
                                       d2h_bytes_per_step=0))))
        return

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    from loquetier_b200 import ops
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
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
        ms = timed(graph.replay, a.steps, a.warmup, torch, dist, clk)
    line = dict(metric="RMSNorm fwd+bwd tokens/s", value=rows * world / (ms * 1e-3), unit="tokens/s", n_gpus=world,
                steps=a.steps, warmup=a.warmup, ms_per_step=ms, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="bf16", data="synthetic", config=cfg, clocks=clk.result,
                gpu_launches=3 * a.steps, launch_mode="cuda graph replay")
    if rank == 0:
        try:
            peak, which = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured"
        except Exception:
            peak, which = 6650.0, "fallback"
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
        e_ms = timed(e2e_step, max(3, min(a.steps, 10)), 3, torch, dist)
        line["e2e"] = dict(value=rows * world / (e_ms * 1e-3), unit="tokens/s", h2d_bytes_per_step=2 * rows * cols * e,
                           d2h_bytes_per_step=2 * rows * cols * e + cols * e, ms_per_step=e_ms)
    if rank == 0 and world == 1 and not a.no_cpu:
        line["cpu_baseline"], _ = cpu_leg(12.0, 5)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


if __name__ == "__main__":
    main()
