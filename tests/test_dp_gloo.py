"""World-size-2 checks of the multi-GPU host logic on CPU ranks (gloo): request
sharding by adapter owner, and the flat gradient bucket's all-reduce."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from loquetier_b200.dp import GradBucket, owner_of, shard_requests, tokens_per_rank


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
        # untouched adapter 2 stays zero everywhere
        ok = ok and all(float(b.dA[p][2].abs().max()) == 0.0 for p in range(len(shapes)))
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


def test_grad_bucket_views_are_contiguous_slices_of_one_buffer():
    b = GradBucket([(16, 24)], n_adapters=3, rank=8, dtype=torch.bfloat16, device="cpu")
    assert b.flat.numel() == 3 * 8 * 16 + 3 * 24 * 8
    assert b.dA[0].data_ptr() == b.flat.data_ptr()
    assert b.dB[0].data_ptr() == b.flat.data_ptr() + 3 * 8 * 16 * 2
    assert all(b.dA[0][i].data_ptr() % 16 == 0 and b.dB[0][i].data_ptr() % 16 == 0 for i in range(3))
    assert b.reduce() is None      # no process group: nothing to do
