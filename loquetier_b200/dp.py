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
  it directly through per-partition pointer tables (no repack pass).  ``reduce()`` is
  a single all-reduce of the flat buffer; ``reduce_projection(p)`` starts the
  all-reduce of one projection's slice as soon as its weight-gradient kernel has been
  issued, so that the exchange of projection p runs under the backward of projection
  p+1, and ``finish()`` joins them (NCCL over NVLink on GPUs, gloo in the CPU tests)."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

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


class GradBucket:
    """Flat gradient buffer for ``n_adapters`` adapters of several projections.

    ``shapes``: per projection (h_in, h_out); layout of one adapter's gradients
    follows the weights (PEFT layout: dA [rank, h_in], dB [h_out, rank])."""

    def __init__(self, shapes: Sequence[Tuple[int, int]], n_adapters: int, rank: int, dtype: torch.dtype, device,
                 group=None):
        self.group = group
        self.n_adapters = int(n_adapters)
        sizes = []
        for h_in, h_out in shapes:
            sizes += [n_adapters * rank * h_in, n_adapters * h_out * rank]
        # keep every view 16-byte aligned: all sizes are multiples of 8 elements already
        self.flat = torch.zeros(sum(sizes), dtype=dtype, device=device)
        self.dA: List[torch.Tensor] = []
        self.dB: List[torch.Tensor] = []
        self._ptrs: List[Tuple[torch.Tensor, torch.Tensor]] = []
        self._slices: List[torch.Tensor] = []
        self._pending: list = []
        off = 0
        for (h_in, h_out) in shapes:
            self._slices.append(self.flat[off:off + n_adapters * rank * (h_in + h_out)])
            a = self.flat[off:off + n_adapters * rank * h_in].view(n_adapters, rank, h_in)
            off += a.numel()
            b = self.flat[off:off + n_adapters * h_out * rank].view(n_adapters, h_out, rank)
            off += b.numel()
            self.dA.append(a)
            self.dB.append(b)
            pa = torch.tensor([a[i].data_ptr() for i in range(n_adapters)], dtype=torch.int64, device=device)
            pb = torch.tensor([b[i].data_ptr() for i in range(n_adapters)], dtype=torch.int64, device=device)
            self._ptrs.append((pa, pb))

    def tables(self, proj: int, part_adapter_ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Per-partition output pointer tables (int64 on the device) for the backward:
        partition p accumulates into the slot of adapter ``part_adapter_ids[p]``."""
        pa, pb = self._ptrs[proj]
        idx = part_adapter_ids.to(device=pa.device, dtype=torch.long)
        return pa[idx].contiguous(), pb[idx].contiguous()

    def zero(self):
        self.flat.zero_()

    def reduce(self, async_op: bool = False):
        """Sum over the ranks of the group, in place."""
        import torch.distributed as dist
        if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(self.group) == 1:
            return None
        return dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=self.group, async_op=async_op)

    def reduce_projection(self, proj: int):
        """Starts the sum over ranks of one projection's dA/dB (a contiguous slice of the flat
        buffer).  The collective is ordered after the work already issued on the current stream
        and runs next to whatever is issued afterwards; ``finish()`` joins it."""
        import torch.distributed as dist
        if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(self.group) == 1:
            return None
        w = dist.all_reduce(self._slices[proj], op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        self._pending.append(w)
        return w

    def finish(self):
        """Makes the current stream (or the host, on CPU) wait for every started reduction."""
        for w in self._pending:
            w.wait()
        self._pending = []

    @property
    def nbytes(self) -> int:
        return self.flat.numel() * self.flat.element_size()
