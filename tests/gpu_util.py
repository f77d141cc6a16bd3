"""Helpers of the GPU parity tests: move an oracle case to the device, run it
through the C ABI (via loquetier_b200.ops) and compare with the oracle."""
import torch

from helpers import assert_close
from oracle import smlm_oracle as O


def dev():
    return torch.device("cuda:0")


def ptr_table(tensors):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=dev())


def to_dev(case):
    d = dict(case)
    d["x"] = case["x"].to(dev())
    d["go"] = case["go"].to(dev())
    d["wa_d"] = [w.to(dev()).contiguous() for w in case["wa"]]
    d["wb_d"] = [w.to(dev()).contiguous() for w in case["wb"]]
    d["seg_d"] = torch.tensor(case["seg"], dtype=torch.int32, device=dev())
    d["ids_d"] = torch.tensor(case["ids"], dtype=torch.int32, device=dev())
    return d


def run_forward(case, indexed=False, scale=None, accumulate=False, y_init=None, grouped=None):
    """Returns (y, v) computed on the GPU by the fused forward.  ``indexed`` passes an adapter table plus
    per-segment indices (and then, unless ``grouped`` is False, a plan that groups short segments by
    adapter); otherwise one pointer per segment."""
    from loquetier_b200 import ops
    c = to_dev(case)
    T = c["x"].shape[0]
    if grouped is None:
        grouped = indexed
    assert indexed or not grouped
    plan = (ops.Plan(c["seg_d"], T, seg_ids=c["ids_d"], n_table=len(c["wa_d"])) if grouped
            else ops.Plan(c["seg_d"], T))
    y = (torch.zeros((T, c["h_out"]), dtype=c["dtype"], device=dev()) if y_init is None
         else y_init.to(dev()).clone())
    v = torch.zeros((T, c["rank"]), dtype=c["dtype"], device=dev())
    if indexed:
        wa_t, wb_t, ids = ptr_table(c["wa_d"]), ptr_table(c["wb_d"]), c["ids_d"]
        sc = None if scale is None else torch.tensor(scale, dtype=torch.float32, device=dev())
    else:
        wa_t = ptr_table([c["wa_d"][i] for i in c["ids"]])
        wb_t = ptr_table([c["wb_d"][i] for i in c["ids"]])
        ids = None
        sc = None if scale is None else torch.tensor([scale[i] for i in c["ids"]], dtype=torch.float32,
                                                     device=dev())
    ops.fwd(y, c["x"], v, wa_t, wb_t, plan, c["rank"], is_row_major=c["is_row_major"], seg_ids=ids,
            seg_scale=sc, accumulate=accumulate)
    torch.cuda.synchronize()
    plan.raise_if_failed()
    return y.cpu(), v.cpu()


def oracle_forward(case, scale=None, y_init=None):
    ids = case["ids"]
    T = case["x"].shape[0]
    y, v = O.add_lora_forward((T, case["h_out"]), case["x"], [case["wa"][i] for i in ids],
                              [case["wb"][i] for i in ids], case["seg"], case["rank"],
                              is_row_major=case["is_row_major"], round_v=True)
    y32 = y.to(torch.float32)
    if scale is not None:
        per = torch.repeat_interleave(torch.tensor([scale[i] for i in ids], dtype=torch.float32),
                                      torch.tensor(case["lens"], dtype=torch.long))
        full = torch.zeros(T)
        full[case["seg"][0]:case["seg"][-1]] = per
        y32 = y32 * full.unsqueeze(-1)
    if y_init is not None:
        y32 = y32 + y_init.to(torch.float32)
    return y32, v


def check_forward(case, **kw):
    scale = kw.get("scale")
    y_init = kw.get("y_init")
    y, v = run_forward(case, **kw)
    y_ref, v_ref = oracle_forward(case, scale=scale, y_init=y_init)
    a, b = case["seg"][0], case["seg"][-1]
    assert_close(v[a:b], v_ref[a:b], what="v")
    assert_close(y[a:b], y_ref[a:b], what="y")
    return y, v
