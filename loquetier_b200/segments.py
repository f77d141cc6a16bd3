"""Segment bookkeeping of one batch step: row order of the requests, run-length
merge of equal adjacent adapters into segments, and the device-side index arrays
the kernels consume.  Integer work; must match the reference bit for bit
(src/loquetier_src/model_generation.py:176-226 for the order, :267-283 for the
merge and the int32 ``lora_len`` / ``segment`` tensors)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .enums import InferStatus


@dataclass
class SegmentRequest:
    """What the bookkeeping needs to know about a request."""
    status: InferStatus
    lora_id: int
    n_tokens: int
    is_eval: bool = False          # a prefill request that carries labels
    batch_info: Optional[Tuple[int, int]] = None   # (batch, seq_len) of a train/eval request


def order_requests(train: Sequence[SegmentRequest], evals: Sequence[SegmentRequest],
                   prefill: Sequence[SegmentRequest], decode: Sequence[SegmentRequest]) -> List[SegmentRequest]:
    """Row order of a step: train requests in arrival order, then eval requests, then
    prefill requests sorted by adapter, then the resident decode requests sorted by
    (status, adapter).  Sorting is stable like Python's ``sorted``."""
    dec = sorted(decode, key=lambda r: (int(r.status), r.lora_id))
    pre = list(evals) + sorted(prefill, key=lambda r: r.lora_id)
    return list(train) + pre + dec


def merge_segments(ordered: Sequence[SegmentRequest]):
    """Adjacent requests with the same adapter become one segment, also across the
    train / prefill / decode boundaries.  Returns (lora_ids, lora_lens)."""
    if not ordered:
        return [], []
    ids, lens = [ordered[0].lora_id], [0]
    for r in ordered:
        if ids[-1] == r.lora_id:
            lens[-1] += int(r.n_tokens)
        else:
            ids.append(r.lora_id)
            lens.append(int(r.n_tokens))
    return ids, lens


@dataclass
class SegmentBatch:
    """Per-step segment description in the reference's own terms."""
    lora_ids: List[int]
    lora_len: torch.Tensor      # int32 [nseg] on the device
    segment: torch.Tensor       # int32 [nseg + 1] on the device, cumsum with leading 0
    train_idx: List[int]
    n_tokens: int


def build_segment_batch(ordered: Sequence[SegmentRequest], device) -> SegmentBatch:
    ids, lens = merge_segments(ordered)
    lora_len = torch.tensor(lens, dtype=torch.int32, device=device)
    seg_host = np.concatenate([[0], np.cumsum(np.asarray(lens, dtype=np.int64))]).astype(np.int32)
    segment = torch.tensor(seg_host, dtype=torch.int32, device=device)
    train_idx = [r.lora_id for r in ordered if r.status == InferStatus.Train]
    return SegmentBatch(ids, lora_len, segment, train_idx, int(seg_host[-1]))


def merge_segments_device(req_ids: torch.Tensor, req_len: torch.Tensor):
    """The run-length merge on the GPU: ``req_ids`` / ``req_len`` are int32 device tensors with one
    entry per request in batch row order.  Returns (seg_ids, seg_len, segment, nseg) as device
    tensors of n, n, n + 1 and 1 entries; entries past ``nseg`` describe empty segments, so the
    padded arrays can be used as they are (no read-back, graph-capturable)."""
    from .cabi import check, lib
    assert req_ids.is_cuda and req_ids.dtype == torch.int32 and req_len.dtype == torch.int32
    n = int(req_ids.numel())
    dev = req_ids.device
    seg_ids = torch.empty(n, dtype=torch.int32, device=dev)
    seg_len = torch.empty(n, dtype=torch.int32, device=dev)
    segment = torch.empty(n + 1, dtype=torch.int32, device=dev)
    nseg = torch.empty(1, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        check(lib.smlm_b200_merge_segments(req_ids.data_ptr(), req_len.data_ptr(), n, seg_ids.data_ptr(),
                                           seg_len.data_ptr(), segment.data_ptr(), nseg.data_ptr(),
                                           torch.cuda.current_stream(dev).cuda_stream), "smlm_b200_merge_segments")
    return seg_ids, seg_len, segment, nseg


GATHER_MAX_LEN = 8  # rows of a "short" segment at most (the plan builder's rule)


def wants_grouped_plan(seg_lens, seg_ids) -> bool:
    """True when a grouped plan changes anything: some adapter has at least two segments of at most
    ``GATHER_MAX_LEN`` rows (decode tokens that are not neighbours in the batch).  Known on the host
    from the same lists the segment index pointer is built from, so no device round trip is needed;
    batches without such segments keep the ordinary plan and the kernels built for it."""
    seen = set()
    for n, a in zip(seg_lens, seg_ids):
        if 0 < int(n) <= GATHER_MAX_LEN:
            if a in seen:
                return True
            seen.add(a)
    return False
