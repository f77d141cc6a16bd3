"""Data-parallel fine-tuning on two GPUs over NCCL: every rank runs the backward of its own train
partitions into the slots of a GradBucket, the slots are summed over the ranks slot range by slot range,
and the result must equal what ONE rank computes for all partitions of both ranks (same kernels, gradients
of partitions that share an adapter accumulated into its slot).  Skipped with fewer than two GPUs."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

RANK_R, H_IN, H_OUT, N_AD = 64, 512, 768, 6
PARTS = {0: ([0, 300, 428], [1, 4]), 1: ([0, 64, 500], [2, 4])}     # per rank: partition index pointer, adapter ids


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _data(rank):
    g = torch.Generator().manual_seed(500 + rank)
    part, ids = PARTS[rank]
    T = part[-1]
    x = torch.randn((T, H_IN), generator=g).to(torch.bfloat16)
    go = torch.randn((T, H_OUT), generator=g).to(torch.bfloat16)
    return x, go, part, ids


def _weights():
    g = torch.Generator().manual_seed(77)
    A = (torch.randn((N_AD, RANK_R, H_IN), generator=g) / 22).to(torch.bfloat16)
    B = (torch.randn((N_AD, H_OUT, RANK_R), generator=g) * 0.02).to(torch.bfloat16)
    return A, B


def _backward_into(bucket, dev, x, go, part, ids, A, B, accumulate):
    from loquetier_b200 import ops
    tab = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
    T = part[-1]
    xd, god = x.to(dev), go.to(dev)
    pd = torch.tensor(part, dtype=torch.int32, device=dev)
    idd = torch.tensor(ids, dtype=torch.int32, device=dev)
    wa, wb = tab(list(A)), tab(list(B))
    plan = ops.Plan(pd, T)
    y = torch.empty((T, H_OUT), dtype=torch.bfloat16, device=dev)
    v = torch.empty((T, RANK_R), dtype=torch.bfloat16, device=dev)
    dx = torch.empty((T, H_IN), dtype=torch.bfloat16, device=dev)
    dv = torch.empty((T, RANK_R), dtype=torch.bfloat16, device=dev)
    ops.fwd(y, xd, v, wa, wb, plan, RANK_R, seg_ids=idd)
    dA_t, dB_t = bucket.tables(0, ids)
    ops.bwd(dx, dA_t, dB_t, dv, god, xd, v, wa, wb, plan, RANK_R, part_ids=idd, accumulate_grads=accumulate)
    torch.cuda.synchronize()
    plan.raise_if_failed()


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from loquetier_b200.dp import GradBucket, touched_union
        A, B = _weights()
        Ad, Bd = A.to(dev), B.to(dev)
        x, go, part, ids = _data(rank)
        bucket = GradBucket([(H_IN, H_OUT)], N_AD, RANK_R, torch.bfloat16, dev)
        union = touched_union(ids, N_AD)
        ok = union == [1, 2, 4]
        bucket.set_touched(union)
        bucket.flat.fill_(float("nan"))          # stale contents: every slot is either cleared or overwritten
        bucket.zero_except(ids)
        _backward_into(bucket, dev, x, go, part, ids, Ad, Bd, accumulate=False)
        bucket.reduce_slots(0, 0, 2)             # two slot ranges, as the benchmark step issues them
        bucket.reduce_slots(0, 2, 3)
        bucket.finish()
        torch.cuda.synchronize()
        if rank == 0:
            # one rank alone over the partitions of both ranks: shared adapters accumulate into their slot
            single = GradBucket([(H_IN, H_OUT)], N_AD, RANK_R, torch.bfloat16, dev)
            single.set_touched(union)
            for r in range(world):
                xr, gor, pr, ir = _data(r)
                _backward_into(single, dev, xr, gor, pr, ir, Ad, Bd, accumulate=True)
            for t_got, t_want in ((bucket.dA[0], single.dA[0]), (bucket.dB[0], single.dB[0])):
                g, w = t_got.float(), t_want.float()
                ok = ok and bool(torch.isfinite(g).all())
                ok = ok and bool(((g - w).abs() <= 1e-2 * max(1.0, float(w.abs().max())) + 1e-2 * w.abs()).all())
            # adapters 1 and 2 were trained on one rank only: their slots are that rank's result, bit for bit
            ok = ok and torch.equal(bucket.dA[0][0], single.dA[0][0]) and torch.equal(bucket.dB[0][0], single.dB[0][0])
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_gradients_equal_single_rank_on_concatenated_tokens():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert dict(out) == {0: True, 1: True}
