"""Shared helpers for the test-suite: golden-vector loading and comparisons."""
import json
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
_DT = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16}

# tolerance of the path for 16-bit storage with fp32 accumulation
RTOL = 1e-2
ATOL = 1e-2


def load_npz(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"), allow_pickle=False)
    dt = _DT[str(z["dtype"])]
    out = {"dtype": dt}
    for k in z.files:
        if k == "dtype":
            continue
        a = z[k]
        if a.dtype == np.uint16:
            out[k] = torch.from_numpy(a.view(np.int16).copy()).view(dt)
        elif a.dtype == np.float32 and k not in ("meta",):
            out[k] = torch.from_numpy(a.copy())
        else:
            out[k] = a
    return out


def load_bookkeeping():
    with open(os.path.join(GOLDEN, "bookkeeping.json")) as f:
        return json.load(f)


def assert_close(got, want, rtol=RTOL, atol=ATOL, what=""):
    g = got.detach().to("cpu", torch.float32)
    w = want.detach().to("cpu", torch.float32)
    assert g.shape == w.shape, f"{what}: shape {tuple(g.shape)} vs {tuple(w.shape)}"
    if g.numel() == 0:
        return
    assert torch.isfinite(g).all(), f"{what}: non-finite values"
    err = (g - w).abs()
    bound = atol + rtol * w.abs()
    bad = err > bound
    if bad.any():
        i = torch.nonzero(bad)[0].tolist()
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{g.numel()} outside rtol={rtol} atol={atol}; "
            f"max abs err {float(err.max()):.4g}; first at {i}: got {float(g[tuple(i)])} want {float(w[tuple(i)])}")
