"""Multi-GPU side of the SMLM path: one process per GPU, plumbing over
``torch.distributed``.

The reference is single-GPU (its trainer refuses more,
src/loquetier_src/trainer_utils.py:28-29), so there is no behaviour to match beyond
"the N-rank result equals the single-rank result on the concatenated work".

* Inference and fine-tuning of rank-owned adapters shard by segment with no
  collective: ``owner_of`` / ``shard_requests`` send every request to the rank that
  owns its adapter, and each rank then builds its own batch with the ordinary
  segment bookkeeping.
* Data-parallel fine-tuning of adapters shared by several ranks has one exchange
  step: the sum of dA/dB.  ``GradBucket`` is one flat, contiguous buffer that holds
  the gradients of every (projection, adapter); the backward kernels write into
  it directly through per-partition pointer tables (no repack pass).

  The buffer is laid out projection by projection and, inside a projection, slot by
  slot: slot s holds dA then dB of one adapter, so any range of slots is one
  contiguous slice that can be summed over the ranks on its own.  Which adapter sits
  in which slot is decided per batch by ``set_touched``: only adapters that some rank
  trains in this batch get a slot (in ascending adapter order, the same on every
  rank), so adapters nobody touched are never sent.  ``reduce_slots(p, s0, s1)`` starts
  the all-reduce of a slot range of one projection as soon as the kernels that produce
  it have been issued, so that the exchange runs under the kernels issued afterwards;
  ``finish()`` joins every started reduction (NCCL over NVLink on GPUs, gloo in the CPU
  tests)."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch


def owner_of(lora_id: int, world_size: int) -> int:
    """Rank that owns an adapter: adapters are dealt round-robin."""
    return int(lora_id) % int(world_size)


def shard_requests(requests: Sequence[Tuple[int, int]], world_size: int) -> List[List[int]]:
    """Indices of the requests each rank serves.  ``requests`` holds (lora_id,
    n_tokens); a request goes to the owner of its adapter and keeps its relative
    order, so that the per-rank batch assembler sees arrival order."""
    out: List[List[int]] = [[] for _ in range(world_size)]
    for i, (lid, _n) in enumerate(requests):
        out[owner_of(lid, world_size)].append(i)
    return out


def tokens_per_rank(requests: Sequence[Tuple[int, int]], world_size: int) -> List[int]:
    tot = [0] * world_size
    for lid, n in requests:
        tot[owner_of(lid, world_size)] += int(n)
    return tot


def touched_union(local_ids: Sequence[int], n_adapters: int, group=None) -> List[int]:
    """Adapters trained by at least one rank of the group in this batch, ascending.  One small
    all-reduce (max) of a 0/1 vector; it belongs to batch assembly, not to the step: the result is
    known on the host before any kernel of the step is launched."""
    import torch.distributed as dist
    mask = torch.zeros(n_adapters, dtype=torch.int32)
    for a in local_ids:
        mask[int(a)] = 1
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        backend = dist.get_backend(group)
        m = mask.cuda() if backend == "nccl" else mask
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        mask = m.cpu()
    return [i for i in range(n_adapters) if int(mask[i])]


class GradBucket:
    """Flat gradient buffer for ``n_adapters`` adapters of several projections.

    ``shapes``: per projection (h_in, h_out); layout of one adapter's gradients
    follows the weights (PEFT layout: dA [rank, h_in], dB [h_out, rank]).  Until
    ``set_touched`` is called every adapter has the slot of its own index."""

    def __init__(self, shapes: Sequence[Tuple[int, int]], n_adapters: int, rank: int, dtype: torch.dtype, device,
                 group=None):
        self.group = group
        self.n_adapters = int(n_adapters)
        self.rank = int(rank)
        self.shapes = [(int(a), int(b)) for a, b in shapes]
        # elements per slot; every part is a multiple of 8 elements, so all views stay 16-byte aligned
        self.slot_elems = [rank * (h_in + h_out) for h_in, h_out in self.shapes]
        self.flat = torch.zeros(n_adapters * sum(self.slot_elems), dtype=dtype, device=device)
        self._pending: list = []
        self.set_touched(list(range(self.n_adapters)))

    # -- slots ----------------------------------------------------------------------------------
    def set_touched(self, adapters: Sequence[int]):
        """Gives every adapter of ``adapters`` (ascending, the same list on every rank) a slot, in
        that order; the other adapters have none in this batch.  Rebuilds the views and tables."""
        ad = [int(a) for a in adapters]
        assert ad == sorted(set(ad)) and all(0 <= a < self.n_adapters for a in ad)
        self.adapters = ad
        self.slot_of = {a: s for s, a in enumerate(ad)}
        self.n_slots = len(ad)
        dev = self.flat.device
        self.dA: List[torch.Tensor] = []
        self.dB: List[torch.Tensor] = []
        self._base: List[int] = []
        self._ptrs: List[Tuple[torch.Tensor, torch.Tensor]] = []
        off = 0
        es = self.flat.element_size()
        for (h_in, h_out), se in zip(self.shapes, self.slot_elems):
            self._base.append(off)
            region = self.flat[off:off + self.n_slots * se]
            a = region.as_strided((self.n_slots, self.rank, h_in), (se, h_in, 1), region.storage_offset())
            b = region.as_strided((self.n_slots, h_out, self.rank), (se, self.rank, 1),
                                  region.storage_offset() + self.rank * h_in)
            self.dA.append(a)
            self.dB.append(b)
            p0 = self.flat.data_ptr() + off * es
            pa = torch.tensor([p0 + s * se * es for s in range(self.n_slots)], dtype=torch.int64, device=dev)
            pb = torch.tensor([p0 + (s * se + self.rank * h_in) * es for s in range(self.n_slots)],
                              dtype=torch.int64, device=dev)
            self._ptrs.append((pa, pb))
            off += self.n_adapters * se   # a projection's region keeps its full size whatever the slot count

    def slots(self, adapter_ids) -> List[int]:
        ids = adapter_ids.tolist() if hasattr(adapter_ids, "tolist") else list(adapter_ids)
        return [self.slot_of[int(a)] for a in ids]

    def tables(self, proj: int, part_adapter_ids) -> Tuple[torch.Tensor, torch.Tensor]:
        """Per-partition output pointer tables (int64 on the device) for the backward:
        partition p writes into the slot of adapter ``part_adapter_ids[p]``."""
        pa, pb = self._ptrs[proj]
        idx = torch.tensor(self.slots(part_adapter_ids), dtype=torch.long, device=pa.device)
        return pa[idx].contiguous(), pb[idx].contiguous()

    def slot_slice(self, proj: int, s0: int, s1: int) -> torch.Tensor:
        """The contiguous part of the flat buffer that holds slots [s0, s1) of one projection."""
        se = self.slot_elems[proj]
        return self.flat[self._base[proj] + s0 * se:self._base[proj] + s1 * se]

    def used(self) -> List[torch.Tensor]:
        """The slices that hold slots, one per projection."""
        return [self.slot_slice(p, 0, self.n_slots) for p in range(len(self.shapes))]

    # -- clearing -------------------------------------------------------------------------------
    def zero(self):
        for t in self.used():
            t.zero_()

    def zero_except(self, local_adapter_ids):
        """Clears the slots this rank does not write in this batch (they still hold the previous
        step's sums); the slots it does write are overwritten by the backward kernels, so they need
        no clearing when the kernels run with accumulate off.  Contiguous runs of slots are cleared
        with one fill each."""
        mine = set(self.slots(local_adapter_ids))
        for p in range(len(self.shapes)):
            s = 0
            while s < self.n_slots:
                if s in mine:
                    s += 1
                    continue
                e = s
                while e < self.n_slots and e not in mine:
                    e += 1
                self.slot_slice(p, s, e).zero_()
                s = e

    # -- the exchange ---------------------------------------------------------------------------
    def _active(self) -> bool:
        import torch.distributed as dist
        return dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1

    def reduce(self, async_op: bool = False):
        """Sum over the ranks of the group, in place, of every slot of every projection."""
        if not self._active():
            return None
        import torch.distributed as dist
        if self.n_slots == self.n_adapters:
            return dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=self.group, async_op=async_op)
        works = [dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group, async_op=async_op) for t in self.used()]
        return works[-1] if works else None

    def reduce_slots(self, proj: int, s0: int, s1: int):
        """Starts the sum over ranks of slots [s0, s1) of one projection.  The collective is ordered
        after the work already issued on the current stream and runs next to whatever is issued
        afterwards; ``finish()`` joins it."""
        if not self._active() or s1 <= s0:
            return None
        import torch.distributed as dist
        w = dist.all_reduce(self.slot_slice(proj, s0, s1), op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        self._pending.append(w)
        return w

    def reduce_projection(self, proj: int):
        """``reduce_slots`` over all slots of one projection."""
        return self.reduce_slots(proj, 0, self.n_slots)

    def finish(self):
        """Makes the current stream (or the host, on CPU) wait for every started reduction."""
        for w in self._pending:
            w.wait()
        self._pending = []

    @property
    def nbytes(self) -> int:
        """Bytes one step exchanges: the slots in use."""
        return self.n_slots * sum(self.slot_elems) * self.flat.element_size()
