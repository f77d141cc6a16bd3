"""Generate golden vectors by running the reference's own Python code on the CPU.

TEST INFRASTRUCTURE ONLY.  Run where the reference checkout is available:

    python oracle/make_golden.py --reference /path/to/Loquetier --out tests/golden

It imports, unmodified, from the reference checkout
    src/loquetier_src/kernel_utils.py       (add_lora, BatchLenInfo)
    src/loquetier_src/models/mixed_lora.py  (MixedLoraLinear, NamedLoraLayer, MixedLoraContext)
    src/loquetier_src/model_generation.py   (ModelGeneration, InputRequest)
with three stand-in modules for what is not installable on a CPU box:
    loquetier.ops._kernels   - smlm_forward_cutlass emulated as one fp32 matmul per
                               segment (pointer -> tensor through a registry), same
                               checks as kernel_src/csrc/loquetier_ops.cc:277-319
    loquetier.utils(.kvcache)- empty KvPool / KvCache / BatchedKvCache
    peft                     - the three names mixed_lora.py imports
The vectors are stored as .npz (16-bit tensors as raw uint16 bit patterns) next to
this script's output directory and are what tests/test_oracle_golden.py pins the
oracle against.
"""
from __future__ import annotations

import argparse
import importlib
import importlib.util
import os
import sys
import types

import numpy as np
import torch

_REG = {}


def _reg(t: torch.Tensor) -> torch.Tensor:
    _REG[t.data_ptr()] = t
    return t


def _install_stubs(ref_root: str):
    # --- loquetier native package -------------------------------------------------
    kern = types.ModuleType("loquetier.ops._kernels")

    def smlm_forward_cutlass_tmp_size(n):
        return (3 * 8 + 3 * 8 + 12) * int(n)

    def smlm_forward_cutlass(y, x, w_ptr, s, tmp, is_row_major):
        assert y.dim() == 2 and x.dim() == 2 and w_ptr.dim() == 1 and s.dim() == 1 and tmp.dim() == 1
        n = s.size(0) - 1
        assert tmp.size(0) == smlm_forward_cutlass_tmp_size(n)
        d_in, d_out = x.size(1), y.size(1)
        sl = s.tolist()
        for i in range(n):
            a, b = sl[i], sl[i + 1]
            if b <= a:
                continue
            w = _REG[int(w_ptr[i])]
            w32 = w.to(torch.float32)
            wm = w32.reshape(d_in, d_out) if is_row_major else w32.reshape(d_out, d_in).t()
            y[a:b] = (x[a:b].to(torch.float32) @ wm).to(y.dtype)

    def rms_norm(o, m, x, w, eps):
        # the CUDA kernel cannot run here: its arithmetic restated from rms_norm_cutlass.cu:100-155
        x32 = x.to(torch.float32)
        s = torch.rsqrt((x32 * x32).sum(dim=1, keepdim=True) / x.size(1) + eps)
        m.copy_(s)
        o.copy_((x32 * s * w.to(torch.float32)).to(o.dtype))

    kern.rms_norm = rms_norm
    kern.smlm_forward_cutlass = smlm_forward_cutlass
    kern.smlm_forward_cutlass_tmp_size = smlm_forward_cutlass_tmp_size
    loq = types.ModuleType("loquetier"); loq.__path__ = []
    ops = types.ModuleType("loquetier.ops"); ops.__path__ = []
    ops._kernels = kern
    utils = types.ModuleType("loquetier.utils"); utils.__path__ = []
    kvc = types.ModuleType("loquetier.utils.kvcache")

    class KvPool:  # noqa: D401 - placeholders, never exercised by the SMLM path
        def __init__(self, *a, **k): pass

    class KvCache:
        def __init__(self, *a, **k): pass
        def acquire_one(self): pass
        def release(self): pass

    class BatchedKvCache:
        def __init__(self, *a, **k): pass

    for m in (utils, kvc):
        m.KvPool, m.KvCache, m.BatchedKvCache = KvPool, KvCache, BatchedKvCache
    loq.ops, loq.utils = ops, utils
    sys.modules.update({
        "loquetier": loq, "loquetier.ops": ops, "loquetier.ops._kernels": kern,
        "loquetier.utils": utils, "loquetier.utils.kvcache": kvc,
    })
    # --- peft (names only) --------------------------------------------------------
    peft = types.ModuleType("peft"); peft.__path__ = []
    tuners = types.ModuleType("peft.tuners"); tuners.__path__ = []
    lora = types.ModuleType("peft.tuners.lora")
    lora.LoraLayer = type("LoraLayer", (), {})
    lora.LoraModel = type("LoraModel", (), {})
    putils = types.ModuleType("peft.utils")
    putils._get_submodules = lambda *a, **k: None
    sys.modules.update({"peft": peft, "peft.tuners": tuners, "peft.tuners.lora": lora,
                        "peft.utils": putils})
    # --- the reference package, without its star-importing __init__ ---------------
    src = os.path.join(ref_root, "src", "loquetier_src")
    pkg = types.ModuleType("loquetier_src"); pkg.__path__ = [src]
    mpkg = types.ModuleType("loquetier_src.models"); mpkg.__path__ = [os.path.join(src, "models")]
    sys.modules["loquetier_src"] = pkg
    sys.modules["loquetier_src.models"] = mpkg
    ku = importlib.import_module("loquetier_src.kernel_utils")
    ml = importlib.import_module("loquetier_src.models.mixed_lora")
    mg = importlib.import_module("loquetier_src.model_generation")
    en = importlib.import_module("loquetier_src.enums")
    return ku, ml, mg, en


def _bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().numpy()


def _weights(g, n, h_in, h_out, r, dtype, math_layout=False):
    a_std = 1.0 / np.sqrt(h_in)
    if math_layout:
        wa = [_reg((torch.randn((h_in, r), generator=g) * a_std).to(dtype).contiguous()) for _ in range(n)]
        wb = [_reg((torch.randn((r, h_out), generator=g) * 0.02).to(dtype).contiguous()) for _ in range(n)]
    else:
        wa = [_reg((torch.randn((r, h_in), generator=g) * a_std).to(dtype).contiguous()) for _ in range(n)]
        wb = [_reg((torch.randn((h_out, r), generator=g) * 0.02).to(dtype).contiguous()) for _ in range(n)]
    return wa, wb


def golden_lora_linear(ku, ml, name, seed, dtype, lens, ids, n_ad, h_in, h_out, r, scale, trains=()):
    """Drive MixedLoraLinear.forward (mixed_lora.py:173-218); ``scale=None`` means the
    adapters were pre-scaled (is_scaled=True)."""
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    x = torch.randn((T, h_in), generator=g).to(dtype)
    base = torch.nn.Linear(h_in, h_out, bias=False, dtype=dtype)
    with torch.no_grad():
        base.weight.copy_((torch.randn((h_out, h_in), generator=g) * 0.02).to(dtype))
    wa, wb = _weights(g, n_ad, h_in, h_out, r, dtype)
    adapters = [ml.NamedLoraLayer(f"a{i}", wa[i], wb[i], torch.nn.Identity(), scale) for i in range(n_ad)]
    ctx = ml.MixedLoraContext()
    lin = ml.MixedLoraLinear(ctx, base, adapters, r, dtype, is_scaled=scale is None)
    blen = ku.BatchLenInfo(list(trains), [], 0, [], torch.device("cpu"))
    seg = torch.cumsum(torch.tensor([0] + list(lens), dtype=torch.int32), 0, dtype=torch.int32)
    ctx.update(blen, list(ids), torch.tensor(lens, dtype=torch.int32), seg, [])
    with torch.no_grad():
        y = lin(x)
    out = dict(x=_bits(x), w_base=_bits(base.weight.detach()), y=_bits(y),
               lens=np.asarray(lens), ids=np.asarray(ids),
               meta=np.asarray([h_in, h_out, r, n_ad, -1 if scale is None else scale], dtype=np.float64),
               dtype=str(dtype))
    for i in range(n_ad):
        out[f"wa{i}"] = _bits(wa[i]); out[f"wb{i}"] = _bits(wb[i])
    return name, out


def golden_add_lora_fwd(ku, name, seed, dtype, seg, ids, n_ad, h_in, h_out, r, T):
    """add_lora.forward called directly (kernel_utils.py:102-120), including empty
    segments and rows no segment covers."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((T, h_in), generator=g).to(dtype)
    wa, wb = _weights(g, n_ad, h_in, h_out, r, dtype)
    wa_ptr = torch.tensor([wa[i].data_ptr() for i in ids], dtype=torch.int64)
    wb_ptr = torch.tensor([wb[i].data_ptr() for i in ids], dtype=torch.int64)
    s = torch.tensor(seg, dtype=torch.int32)
    y = ku.add_lora.forward((T, h_out), x, wa_ptr, wb_ptr, s, r, 0, [])
    a, b = seg[0], seg[-1]
    out = dict(x=_bits(x), y=_bits(y[a:b]), seg=np.asarray(seg), ids=np.asarray(ids),
               meta=np.asarray([h_in, h_out, r, n_ad, T], dtype=np.float64), dtype=str(dtype))
    for i in range(n_ad):
        out[f"wa{i}"] = _bits(wa[i]); out[f"wb{i}"] = _bits(wb[i])
    return name, out


def golden_add_lora_bwd(ku, name, seed, dtype, part, h_in, h_out, r, T):
    """add_lora.backward as released (kernel_utils.py:129-147).  Its formulas only
    type-check for the math layout A[h_in,r], B[r,h_out], so that is what is fed."""
    g = torch.Generator().manual_seed(seed)
    npart = len(part) - 1
    x = torch.randn((T, h_in), generator=g).to(dtype)
    go = torch.randn((T, h_out), generator=g).to(dtype)
    wa, wb = _weights(g, npart, h_in, h_out, r, dtype, math_layout=True)
    ctx = types.SimpleNamespace()
    ctx.tp = list(part)
    ctx.saved_tensors = (x[:part[-1]],) + tuple(w for p in range(npart) for w in (wa[p], wb[p]))
    res = ku.add_lora.backward(ctx, go)
    assert all(r_ is None for r_ in res[:1] + res[2:8])
    out = dict(x=_bits(x), go=_bits(go), gx=_bits(res[1]), part=np.asarray(part),
               meta=np.asarray([h_in, h_out, r, npart, T], dtype=np.float64), dtype=str(dtype))
    for p in range(npart):
        out[f"wa{p}"] = _bits(wa[p]); out[f"wb{p}"] = _bits(wb[p])
        out[f"dA{p}"] = _bits(res[8 + 2 * p]); out[f"dB{p}"] = _bits(res[9 + 2 * p])
    return name, out


def golden_rms_norm(ku, name, seed, dtype, rows, cols, eps):
    """rms_norm.forward / backward of the reference (kernel_utils.py:149-176) run on the CPU: the forward
    through the stubbed native op, the backward is the reference's own torch code."""
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn((rows, cols), generator=g) * 1.5).to(dtype)
    w = (1.0 + 0.1 * torch.randn((cols,), generator=g)).to(dtype)
    go = torch.randn((rows, cols), generator=g).to(dtype)
    ctx = types.SimpleNamespace()
    ctx.save_for_backward = lambda *t: setattr(ctx, "saved_tensors", t)
    o = ku.rms_norm.forward(ctx, x, w, eps)
    dx, dw, none = ku.rms_norm.backward(ctx, go)
    assert none is None
    return name, dict(x=_bits(x), w=_bits(w), go=_bits(go), o=_bits(o), rms=ctx.saved_tensors[2].numpy(),
                      dx=dx.to(torch.float32).numpy(), dw=dw.to(torch.float32).numpy(),
                      meta=np.asarray([rows, cols, eps], dtype=np.float64), dtype=str(dtype))


def golden_prepare_weight(ml, name, seed, dtype):
    """MixedLoraModel._prepare_weight (mixed_lora.py:501-521) called unbound on the three kinds of input
    it sees at load time: an A panel whose rank is below the model-wide rank (zero-padded along dim 0)
    with the scale baked in, a B panel padded along dim 1 without a scale, and a panel of full rank
    with a scale.  Inputs are fp32 as PEFT holds them; outputs are in the module dtype."""
    g = torch.Generator().manual_seed(seed)
    me = types.SimpleNamespace(rank=16, dtype=dtype)
    a_small = torch.randn((8, 64), generator=g) / 8
    b_small = torch.randn((48, 8), generator=g) * 0.02
    a_full = torch.randn((16, 64), generator=g) / 8
    cpu = torch.device("cpu")
    f = ml.MixedLoraModel._prepare_weight
    out = dict(a_small=a_small.numpy(), b_small=b_small.numpy(), a_full=a_full.numpy(),
               a_small_out=_bits(f(me, a_small, cpu, 0, 2.0)),
               b_small_out=_bits(f(me, b_small, cpu, 1, None)),
               a_full_out=_bits(f(me, a_full, cpu, 0, 0.3)),
               dtype=str(dtype))
    return name, out


def golden_batch_len_info(ku):
    cases = [
        dict(trains=[], prefills=[], decode=0, evals=[]),
        dict(trains=[(1, 7)], prefills=[], decode=3, evals=[]),
        dict(trains=[(2, 5), (1, 9)], prefills=[4, 1, 12], decode=5, evals=[]),
        dict(trains=[], prefills=[3], decode=0, evals=[(1, 3)]),
        dict(trains=[(4, 128), (2, 64), (1, 1)], prefills=[7, 9], decode=64, evals=[(2, 7), (1, 9)]),
        dict(trains=[(1, 1024), (1, 1024)], prefills=[512] * 4, decode=64, evals=[]),
    ]
    rows = []
    for c in cases:
        b = ku.BatchLenInfo(c["trains"], c["prefills"], c["decode"], c["evals"], torch.device("cpu"))
        rows.append(dict(
            case=c,
            train_partition=[int(v) for v in b.train_partition],
            tlen=int(b.tlen),
            eval_partition=[int(v) for v in b.eval_partition],
            prefills=[int(v) for v in b.prefills],
            decode=int(b.decode),
            doff=int(b.doff),
            indptr=None if b.indptr is None else [int(v) for v in b.indptr.tolist()],
            indptr_dtype=None if b.indptr is None else str(b.indptr.dtype),
        ))
    return rows


class _Captured(Exception):
    def __init__(self, kw):
        self.kw = kw


def golden_segments(mg, en):
    """Drive ModelGeneration.generate (model_generation.py:176-226, 251-283) up to the
    point where it hands lora_ids / lora_len / segment to the model."""
    S = en.InferStatus

    class FakeModel:
        def prepare_inputs_for_generation(self, input_ids, attention_mask, **kw):
            raise _Captured(dict(kw, n_tokens=int(input_ids.numel())))

    def run(reqs_spec, resident=()):
        gen = object.__new__(mg.ModelGeneration)
        gen.model = FakeModel()
        gen.device = torch.device("cpu")
        gen.requests, gen.train_requests, gen.eval_requests, gen.prefill_requests = [], [], [], []
        gen.output_with_mark_ids, gen.finished_mark_ids = {}, set()
        gen.new_decode_request = False
        gen.decode_request_changed = False
        gen.cached_decode_kv = []

        def mk(kind, lid, n, mark):
            st = {"train": S.Train, "eval": S.Prefill, "prefill": S.Prefill, "decode": S.Decode}[kind]
            r = mg.InputRequest(status=st, input_ids=torch.zeros(n, dtype=torch.long),
                                next_input_ids=[0] * n, mark_id=mark, lora_name=f"l{lid}", lora_id=lid)
            r.kvcache = sys.modules["loquetier.utils"].KvCache()
            if kind == "train":
                r.batch_info = (1, n)
                gen.train_requests.append(r)
            elif kind == "eval":
                r.batch_info = (1, n); r.labels = torch.zeros(n, dtype=torch.long)
                gen.eval_requests.append(r)
            elif kind == "prefill":
                gen.prefill_requests.append(r)
            else:
                gen.requests.append(r); gen.new_decode_request = True

        for i, (kind, lid, n) in enumerate(reqs_spec):
            mk(kind, lid, n, i)
        try:
            gen.generate()
        except _Captured as c:
            kw = c.kw
            return dict(
                spec=[list(r) for r in reqs_spec],
                lora_ids=[int(v) for v in kw["lora_ids"]],
                lora_len=[int(v) for v in kw["lora_len"].tolist()],
                lora_len_dtype=str(kw["lora_len"].dtype),
                segment=[int(v) for v in kw["segment"].tolist()],
                segment_dtype=str(kw["segment"].dtype),
                train_idx=[int(v) for v in kw["train_idx"]],
                tlen=int(kw["blen"].tlen), doff=int(kw["blen"].doff),
                train_partition=[int(v) for v in kw["blen"].train_partition],
                n_tokens=kw["n_tokens"],
            )
        raise RuntimeError("generate() did not reach the model")

    rng = np.random.default_rng(7)
    specs = [
        [("decode", 1, 1), ("decode", 0, 1), ("decode", 1, 1), ("decode", 2, 1)],
        [("prefill", 3, 5), ("prefill", 1, 9), ("decode", 1, 1), ("decode", 3, 1)],
        [("train", 2, 16), ("train", 0, 8), ("prefill", 0, 4), ("decode", 0, 1), ("decode", 2, 1)],
        [("train", 1, 6), ("eval", 1, 3), ("prefill", 1, 2), ("decode", 1, 1)],
        [("train", 0, 1024), ("train", 5, 1024)] + [("prefill", int(rng.integers(0, 32)), 512) for _ in range(4)]
        + [("decode", int(rng.integers(0, 32)), 1) for _ in range(64)],
    ]
    for _ in range(6):
        n = int(rng.integers(1, 40))
        kinds = rng.choice(["train", "eval", "prefill", "decode"], size=n, p=[0.15, 0.1, 0.25, 0.5])
        specs.append([(str(k), int(rng.integers(0, 6)), 1 if k == "decode" else int(rng.integers(1, 50)))
                      for k in kinds])
    return [run(s) for s in specs]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("LOQUETIER_REFERENCE"), required="LOQUETIER_REFERENCE" not in os.environ,
                    help="path of a checkout of the reference (or set LOQUETIER_REFERENCE)")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(__file__), "..", "tests", "golden"))
    a = ap.parse_args()
    ku, ml, mg, en = _install_stubs(a.reference)
    os.makedirs(a.out, exist_ok=True)
    torch.set_num_threads(1)
    cases = [
        # the CPU plumbing configuration: h 256->256, rank 8, 3 adapters, lengths [7,33,1,64]
        golden_lora_linear(ku, ml, "linear_c1_fp32", 1000, torch.float32, [7, 33, 1, 64], [0, 2, 1, 0],
                           3, 256, 256, 8, 2.0),
        golden_lora_linear(ku, ml, "linear_c1_bf16", 1000, torch.bfloat16, [7, 33, 1, 64], [0, 2, 1, 0],
                           3, 256, 256, 8, 2.0),
        golden_lora_linear(ku, ml, "linear_c1_fp16_prescaled", 1001, torch.float16, [7, 33, 1, 64], [0, 2, 1, 0],
                           3, 256, 256, 8, None),
        golden_lora_linear(ku, ml, "linear_ragged_bf16", 1002, torch.bfloat16,
                           [1, 15, 16, 17, 31, 33, 1, 1, 64, 65], [3, 0, 1, 3, 2, 0, 1, 2, 3, 0],
                           4, 192, 320, 16, 0.5),
        golden_add_lora_fwd(ku, "addlora_edges_bf16", 1003, torch.bfloat16,
                            [3, 3, 10, 10, 11, 40, 40], [0, 1, 2, 0, 1, 2], 3, 128, 64, 8, 48),
        golden_add_lora_fwd(ku, "addlora_edges_fp16", 1004, torch.float16,
                            [0, 1, 2, 18, 18, 50], [1, 0, 1, 0, 1], 2, 64, 136, 32, 50),
        golden_add_lora_fwd(ku, "addlora_fp32", 1005, torch.float32,
                            [0, 5, 70, 71], [2, 1, 0], 3, 96, 48, 8, 71),
        golden_add_lora_bwd(ku, "bwd_math_fp32", 1006, torch.float32, [0, 24, 24, 61], 96, 80, 8, 70),
        golden_add_lora_bwd(ku, "bwd_math_bf16", 1007, torch.bfloat16, [0, 33, 97], 128, 192, 16, 100),
        golden_add_lora_bwd(ku, "bwd_math_fp16", 1008, torch.float16, [0, 70], 64, 64, 8, 70),
        golden_rms_norm(ku, "rmsnorm_bf16", 1009, torch.bfloat16, 37, 256, 1e-6),
        golden_rms_norm(ku, "rmsnorm_fp16", 1010, torch.float16, 5, 520, 1e-5),
        golden_prepare_weight(ml, "prepare_weight_bf16", 1011, torch.bfloat16),
        golden_prepare_weight(ml, "prepare_weight_fp16", 1012, torch.float16),
    ]
    for name, arrs in cases:
        np.savez_compressed(os.path.join(a.out, name + ".npz"), **arrs)
    import json
    with open(os.path.join(a.out, "bookkeeping.json"), "w") as f:
        json.dump(dict(batch_len_info=golden_batch_len_info(ku), segments=golden_segments(mg, en)), f, indent=1)
    print("wrote", len(cases), "tensor cases + bookkeeping.json to", os.path.abspath(a.out))


if __name__ == "__main__":
    main()
