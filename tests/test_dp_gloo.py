"""World-size-2 checks of the multi-GPU host logic on CPU ranks (gloo): request
sharding by adapter owner, and the flat gradient bucket's all-reduce."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from loquetier_b200.dp import GradBucket, owner_of, shard_requests, tokens_per_rank, touched_union


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_shard_requests_sends_every_request_to_its_owner():
    reqs = [(5, 10), (0, 3), (2, 1), (5, 7), (1, 1), (4, 200), (3, 9)]
    for world in (1, 2, 4, 8):
        shards = shard_requests(reqs, world)
        seen = sorted(i for s in shards for i in s)
        assert seen == list(range(len(reqs)))
        for r, s in enumerate(shards):
            assert s == sorted(s)                      # arrival order kept
            assert all(owner_of(reqs[i][0], world) == r for i in s)
        assert sum(tokens_per_rank(reqs, world)) == sum(n for _, n in reqs)


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(100 + rank)
        shapes = [(32, 48), (48, 32)]
        b = GradBucket(shapes, n_adapters=4, rank=8, dtype=torch.float32, device="cpu")
        # each rank "trains" two adapters; adapter 1 is trained on both ranks
        mine = [0, 1] if rank == 0 else [1, 3]
        ids = torch.tensor(mine)
        for p in range(len(shapes)):
            ta, tb = b.tables(p, ids)
            assert ta.tolist() == [b.dA[p][i].data_ptr() for i in mine]
            assert tb.tolist() == [b.dB[p][i].data_ptr() for i in mine]
            for i in mine:
                b.dA[p][i].copy_(torch.randn_like(b.dA[p][i]))
                b.dB[p][i].copy_(torch.randn_like(b.dB[p][i]))
        local = b.flat.clone()
        b.reduce()
        gathered = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(gathered, local)
        want = sum(gathered)
        ok = torch.allclose(b.flat, want)
        # the per-projection reductions together give the same sums as the single one
        b.flat.copy_(local)
        for p in range(len(shapes)):
            b.reduce_projection(p)
        b.finish()
        ok = ok and torch.allclose(b.flat, want)
        # ... and so do reductions slot range by slot range
        b.flat.copy_(local)
        for p in range(len(shapes)):
            b.reduce_slots(p, 0, 1)
            b.reduce_slots(p, 1, 4)
        b.finish()
        ok = ok and torch.allclose(b.flat, want)
        # untouched adapter 2 stays zero everywhere
        ok = ok and all(float(b.dA[p][2].abs().max()) == 0.0 for p in range(len(shapes)))

        # only adapters some rank trains get a slot: the union is {0, 1, 3} on both ranks
        union = touched_union(mine, 4)
        ok = ok and union == [0, 1, 3]
        full = {(p, a): (b.dA[p][a].clone(), b.dB[p][a].clone()) for p in range(len(shapes)) for a in union}
        b.set_touched(union)
        ok = ok and b.n_slots == 3 and b.nbytes == 3 * sum(8 * (hi + ho) for hi, ho in shapes) * 4
        for step in range(2):   # the second step starts from the first one's sums
            b.zero_except(mine)
            for p in range(len(shapes)):
                ta, tb = b.tables(p, ids)
                assert ta.tolist() == [b.dA[p][b.slot_of[i]].data_ptr() for i in mine]
                for i in mine:
                    g = torch.Generator().manual_seed(1000 * p + 10 * i + rank)
                    b.dA[p][b.slot_of[i]].copy_(torch.randn(b.dA[p][0].shape, generator=g))
                    b.dB[p][b.slot_of[i]].copy_(torch.randn(b.dB[p][0].shape, generator=g))
                b.reduce_slots(p, 0, 2)
                b.reduce_slots(p, 2, 3)
            b.finish()
            for p in range(len(shapes)):
                for a in union:
                    wa = torch.zeros_like(b.dA[p][0])
                    wb = torch.zeros_like(b.dB[p][0])
                    for r, theirs in enumerate(([0, 1], [1, 3])):
                        if a in theirs:
                            g = torch.Generator().manual_seed(1000 * p + 10 * a + r)
                            wa += torch.randn(wa.shape, generator=g)
                            wb += torch.randn(wb.shape, generator=g)
                    ok = ok and torch.allclose(b.dA[p][b.slot_of[a]], wa) and torch.allclose(b.dB[p][b.slot_of[a]], wb)
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_grad_bucket_allreduce_world_size_2():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    assert dict(out) == {0: True, 1: True}


def test_grad_bucket_slots_are_contiguous_slices_of_one_buffer():
    b = GradBucket([(16, 24)], n_adapters=3, rank=8, dtype=torch.bfloat16, device="cpu")
    per = 8 * 16 + 24 * 8
    assert b.flat.numel() == 3 * per
    for i in range(3):   # slot i: dA then dB of adapter i
        assert b.dA[0][i].data_ptr() == b.flat.data_ptr() + i * per * 2
        assert b.dB[0][i].data_ptr() == b.flat.data_ptr() + (i * per + 8 * 16) * 2
        assert b.dA[0][i].is_contiguous() and b.dB[0][i].is_contiguous()
        assert b.dA[0][i].data_ptr() % 16 == 0 and b.dB[0][i].data_ptr() % 16 == 0
    assert b.slot_slice(0, 1, 3).data_ptr() == b.dA[0][1].data_ptr() and b.slot_slice(0, 1, 3).numel() == 2 * per
    assert b.reduce() is None      # no process group: nothing to do
    # a batch that touches adapters 0 and 2 only: two slots, the exchange shrinks with them
    b.set_touched([0, 2])
    assert b.n_slots == 2 and b.nbytes == 2 * per * 2 and b.slots([2, 0]) == [1, 0]
    b.flat.fill_(1.0)
    b.zero_except([2])
    assert float(b.dA[0][0].abs().max()) == 0.0 and float(b.dB[0][1].min()) == 1.0
