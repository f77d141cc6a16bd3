"""Times the reference's own CUDA kernels (``oracle/_ref/libref.so``, built by ``oracle/build_ref.py``)
next to this library's on the same seeded inputs, on one GPU.  TEST INFRASTRUCTURE: a measurement aid
for the baseline tables, not part of the product and not used by ``bench.py``.

    python oracle/time_ref.py > time_ref.json

Cases: the SMLM forward (shrink then expand, the two operator calls of add_lora.forward) on the
q_proj-shaped mixed batch (C2), on the q_proj and gate_proj shapes of the Llama-3-8B batch (C3) and on
the decode sweep (C4, both shapes); the RMSNorm forward on 32768 x 4096; decode attention with the
key/value append on 128 requests.  The reference synchronises the stream inside every call, so its
figure is wall clock around the calls (what its caller waits for); the library's figure is CUDA events
around the stream-ordered calls.  L2 is flushed between repetitions."""
from __future__ import annotations

import json
import os
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import bench  # noqa: E402
import ref_cuda  # noqa: E402
from loquetier_b200 import kernels, kvcache, ops  # noqa: E402

DEV = torch.device("cuda:0")


def _flush():
    if not hasattr(_flush, "buf"):
        _flush.buf = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    _flush.buf.zero_()


def _wall(fn, reps=7):
    ts = []
    for _ in range(reps + 1):
        _flush()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        fn()
        torch.cuda.synchronize()
        ts.append((time.perf_counter() - t0) * 1e3)
    return float(np.median(ts[1:]))


def _events(fn, reps=7):
    ts = []
    for _ in range(reps + 1):
        _flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return float(np.median(ts[1:]))


def smlm_case(name, only=None):
    spec = bench.workload_spec(name)
    if only:
        spec["projections"] = [p for p in spec["projections"] if p[0] in only]
    wl = bench.Workload(spec, DEV)
    out = {}
    r = spec["rank"]
    ids = spec["ids"]
    for p in wl.proj:
        wa = p["wa"][torch.tensor(ids, device=DEV)].contiguous()      # one pointer per segment, as the reference wants
        wb = p["wb"][torch.tensor(ids, device=DEV)].contiguous()
        v = torch.empty_like(p["v"])
        y = torch.empty_like(p["y"])
        nbytes = 2 * (wl.T * (p["h_in"] + p["h_out"]) + len(set(ids)) * r * (p["h_in"] + p["h_out"]))

        def ref():
            ref_cuda.smlm_forward_cutlass(v, p["x"], wa, wl.seg, False)
            ref_cuda.smlm_forward_cutlass(y, v, wb, wl.seg, False)

        tmp = torch.empty(kernels.smlm_forward_cutlass_tmp_size(len(ids)), dtype=torch.uint8, device=DEV)

        def lib_ops():
            kernels.smlm_forward_cutlass(v, p["x"], wa, wl.seg, tmp, False)
            kernels.smlm_forward_cutlass(y, v, wb, wl.seg, tmp, False)

        def lib_fused():
            plan = ops.Plan(wl.seg, wl.T, seg_ids=wl.ids, n_table=spec["n_adapters"])
            ops.fwd(y, p["x"], v, p["wa"], p["wb"], plan, r, seg_ids=wl.ids)

        t_ref, t_ops, t_fused = _wall(ref), _events(lib_ops), _events(lib_fused)
        out[p["name"]] = dict(tokens=wl.T, segments=len(ids), algorithmic_mb=nbytes / 1e6,
                              reference_ms=t_ref, library_two_operator_calls_ms=t_ops, library_fused_ms=t_fused,
                              reference_gbs=nbytes / t_ref / 1e6, library_fused_gbs=nbytes / t_fused / 1e6)
    return out


def rms_case():
    rows, cols = 32768, 4096
    g = torch.Generator(device=DEV).manual_seed(1)
    x = (torch.randn((rows, cols), generator=g, device=DEV) * 1.5).to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn((cols,), generator=g, device=DEV)).to(torch.bfloat16)
    o = torch.empty_like(x)
    m = torch.empty((rows, 1), dtype=torch.float32, device=DEV)
    nbytes = 2 * (2 * rows * cols + cols) + 4 * rows
    t_ref = _wall(lambda: ref_cuda.rms_norm(o, m, x, w, 1e-5))
    t_lib = _events(lambda: kernels.rms_norm(o, m, x, w, 1e-5))
    return dict(rows=rows, cols=cols, algorithmic_mb=nbytes / 1e6, reference_ms=t_ref, library_ms=t_lib,
                reference_gbs=nbytes / t_ref / 1e6, library_gbs=nbytes / t_lib / 1e6)


def decode_case():
    B, N, G, P, D = 128, 8, 4, 16, 128
    rng = np.random.default_rng(9000)
    seqlens = [int(v) for v in rng.integers(512, 4097, size=B)]
    pool = kvcache.KvPool(1, N, D, P, torch.bfloat16, DEV, pages_per_slab=4096)
    caches = [kvcache.KvCache(pool, L) for L in seqlens]
    for slab in pool._slabs:
        slab.normal_()
    bkv = kvcache.BatchedKvCache(caches)
    g = torch.Generator(device=DEV).manual_seed(2)
    q = torch.randn((B, N * G, D), generator=g, device=DEV).to(torch.bfloat16)
    k = torch.randn((B, N, D), generator=g, device=DEV).to(torch.bfloat16)
    v = torch.randn((B, N, D), generator=g, device=DEV).to(torch.bfloat16)
    o = torch.empty_like(q)
    nbytes = 2 * (2 * sum(seqlens) * N * D + 2 * B * N * G * D + 2 * B * N * D)

    def ref():
        ref_cuda.append_kv(bkv.ptrs, bkv.indptr, bkv.last_page_offset, k, v, 1, 0, N, P)
        ref_cuda.batch_decode(o, q, bkv.ptrs, bkv.indptr, bkv.last_page_offset, 1, 0, N, 500000.0)

    def lib():
        kvcache.append_kv(bkv, k, v, 0)
        kvcache.batch_decode_into(o, q, bkv.ptrs, bkv.indptr, bkv.last_page_offset, 1, 0, N, 500000.0, P)

    t_ref, t_lib = _wall(ref), _events(lib)
    return dict(requests=B, context_tokens=sum(seqlens), algorithmic_mb=nbytes / 1e6, reference_ms=t_ref,
                library_ms=t_lib, reference_gbs=nbytes / t_ref / 1e6, library_gbs=nbytes / t_lib / 1e6)


def prefill_case():
    B, N, G, P, D = 32, 8, 4, 16, 128
    rng = np.random.default_rng(9100)
    seqlens = [int(v) for v in rng.integers(256, 2049, size=B)]
    T = sum(seqlens)
    pool = kvcache.KvPool(1, N, D, P, torch.bfloat16, DEV, pages_per_slab=4096)
    caches = [kvcache.KvCache(pool, L) for L in seqlens]
    bkv = kvcache.BatchedKvCache(caches)
    g = torch.Generator(device=DEV).manual_seed(3)
    q = torch.randn((T, N * G, D), generator=g, device=DEV).to(torch.bfloat16)
    k = torch.randn((T, N, D), generator=g, device=DEV).to(torch.bfloat16)
    v = torch.randn((T, N, D), generator=g, device=DEV).to(torch.bfloat16)
    o_ref, o_lib = torch.empty_like(q), torch.empty_like(q)
    qind = torch.tensor(np.concatenate([[0], np.cumsum(seqlens)]).astype(np.int32), device=DEV)
    flops = float(sum(4 * D * N * G * (L * (L + 1) // 2) for L in seqlens))

    def ref():
        ref_cuda.append_kv(bkv.ptrs, bkv.indptr, bkv.last_page_offset, k, v, 1, 0, N, P, seqlen_indptr=qind)
        ref_cuda.batch_prefill(o_ref, q, qind, bkv.ptrs, bkv.indptr, bkv.last_page_offset, 1, 0, N, 500000.0)

    def lib():
        kvcache.init_kv(bkv, k, v, qind, 0)
        kvcache.batch_prefill_into(o_lib, q, qind, bkv.ptrs, bkv.indptr, bkv.last_page_offset, 1, 0, N, 500000.0, P)

    t_ref, t_lib = _wall(ref), _events(lib)
    err = float((o_ref.float() - o_lib.float()).abs().max())
    return dict(prompts=B, prompt_tokens=T, causal_tflop=flops / 1e12, reference_ms=t_ref, library_ms=t_lib,
                reference_tflops=flops / t_ref / 1e9, library_tflops=flops / t_lib / 1e9, max_abs_difference=err)


def main():
    assert ref_cuda.available(), "build oracle/_ref/libref.so first (python oracle/build_ref.py --reference ...)"
    res = dict(gpu=torch.cuda.get_device_name(0),
               smlm_forward=dict(c2=smlm_case("c2"), c3=smlm_case("c3", only=("q_proj", "gate_proj")),
                                 c4=smlm_case("c4"), c5=smlm_case("c5")),
               rms_norm_forward=rms_case(), decode_attention=decode_case(), prefill_attention=prefill_case())
    print(json.dumps(res, indent=1))


if __name__ == "__main__":
    main()
