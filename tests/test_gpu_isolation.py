"""Isolation between neighbours in the batch: what sits in the rows next to a train partition - another
partition's rows, or rows that are not fine-tuned at all - must not leak into that partition's weight
gradients, whatever it holds.  The kernels fetch 16-token boxes, so the last box of a ragged partition
carries the first rows of its neighbour; those rows are neutralised in BOTH operands (0 x Inf would be
NaN).  All inputs of the partitions under test are finite; nothing here faults."""
import pytest
import torch

from gpu_util import dev, ptr_table
from helpers import assert_close
from oracle import smlm_oracle as O

pytestmark = pytest.mark.gpu


def _run(rank, lens, poison_rows, tc_mode, h_in=256, h_out=384):
    from loquetier_b200 import ops
    dt = torch.bfloat16
    npart = len(lens)
    c = O.make_case(900 + rank, lens + [40], list(range(npart)) + [0], npart, h_in, h_out, rank, dt)
    T = sum(lens) + 40
    tl = sum(lens)
    x, go = c["x"].clone(), c["go"].clone()
    # the forward's v and the backward's dV as the kernels would leave them (16-bit)
    v = torch.zeros((T, rank), dtype=dt)
    O.smlm_gemm(v, x, [c["wa"][i] for i in c["ids"]], c["seg"])
    dv = torch.zeros((T, rank), dtype=dt)
    for k in range(npart):
        a, b = c["seg"][k], c["seg"][k + 1]
        dv[a:b] = (go[a:b].float() @ c["wb"][k].float()).to(dt)
    want = []
    for k in range(npart):
        a, b = c["seg"][k], c["seg"][k + 1]
        want.append(((dv[a:b].float().t() @ x[a:b].float()), (go[a:b].float().t() @ v[a:b].float())))
    # poison: whole rows of every operand the weight-gradient kernel reads
    for r in poison_rows:
        for t in (x, go, v, dv):
            t[r] = float("inf")
            t[r, ::2] = float("nan")
    d = dev()
    xd, god, vd, dvd = x.to(d), go.to(d), v.to(d), dv.to(d)
    part = torch.tensor(c["seg"][:npart + 1], dtype=torch.int32, device=d)
    plan = ops.Plan(part, T)   # the tensors have T rows: the rows past the partitions are really fetched
    dA = [torch.empty((rank, h_in), dtype=dt, device=d) for _ in range(npart)]
    dB = [torch.empty((h_out, rank), dtype=dt, device=d) for _ in range(npart)]
    prev = ops.set_tensor_core_mode(tc_mode)
    try:
        ops.wgrad_pair(ptr_table(dA), ptr_table(dB), dvd, xd, vd, god, part, plan, rank)
        torch.cuda.synchronize()
    finally:
        ops.set_tensor_core_mode(prev)
    plan.raise_if_failed()
    return dA, dB, want


@pytest.mark.parametrize("rank,tc_mode", [(16, -1), (32, -1), (16, 1), (64, 1), (64, -1)])
def test_rows_after_the_last_partition_do_not_reach_its_gradients(rank, tc_mode):
    lens = [70, 9, 37]                    # every partition ends inside a 16-token box
    tl = sum(lens)
    dA, dB, want = _run(rank, lens, poison_rows=range(tl, tl + 40), tc_mode=tc_mode)
    for k in range(len(lens)):
        assert torch.isfinite(dA[k]).all() and torch.isfinite(dB[k]).all(), f"partition {k} poisoned"
        assert_close(dA[k], want[k][0], atol=1e-2 * float(want[k][0].abs().max()), what=f"dA{k}")
        assert_close(dB[k], want[k][1], atol=1e-2 * float(want[k][1].abs().max()), what=f"dB{k}")


@pytest.mark.parametrize("rank,tc_mode", [(16, -1), (64, 1)])
def test_a_diverged_partition_does_not_poison_its_neighbours(rank, tc_mode):
    lens = [70, 9, 37]
    # partition 1 (rows 70..78) holds Inf / NaN everywhere: its own gradients are lost, the others' are not
    dA, dB, want = _run(rank, lens, poison_rows=range(70, 79), tc_mode=tc_mode)
    for k in (0, 2):
        assert torch.isfinite(dA[k]).all() and torch.isfinite(dB[k]).all(), f"partition {k} poisoned by partition 1"
        assert_close(dA[k], want[k][0], atol=1e-2 * float(want[k][0].abs().max()), what=f"dA{k}")
        assert_close(dB[k], want[k][1], atol=1e-2 * float(want[k][1].abs().max()), what=f"dB{k}")
    assert not torch.isfinite(dA[1]).all()
