"""Paged key-value cache of the decode path: the mirror of ``KvPool``, ``KvCache`` and
``BatchedKvCache`` of the reference (kernel_src/src/loquetier/utils/kvcache.py:7-50, 87-141, 143-165)
with the same constructors, properties and methods, plus the three attention-side operators
``batch_prefill``, ``batch_decode``, ``init_kv`` and ``append_kv`` of kernel_src/src/loquetier/ops/__init__.py:18-170
on the B200 kernels.

A page is one tensor ``[num_layers, 2, num_heads, page_len, head_dim]``, as in the reference.  The pool
hands pages out of large slabs instead of one device allocation per page: a slab of 180 GB-class HBM
is cut once, pages are views into it and go back to a free list, so steady-state decoding never calls
the allocator."""
from __future__ import annotations

from collections.abc import Iterable, Sequence
from typing import Any, List, Optional

import torch

from . import cabi
from .cabi import check, lib

_DT = {torch.float16: cabi.SMLM_F16, torch.bfloat16: cabi.SMLM_BF16}


class KvPool:
    def __init__(self, num_layers: int, num_heads: int, head_dim: int, page_len: int, dtype: torch.dtype,
                 device: torch.device, pages_per_slab: int = 256):
        self.num_layers = num_layers
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.page_len = page_len
        self.dtype = dtype
        self.device = torch.device(device)
        self._page_shape = (num_layers, 2, num_heads, page_len, head_dim)
        self._page_meta = torch.empty(self._page_shape, dtype=dtype, device="meta")
        self._pages_per_slab = int(pages_per_slab)
        self._slabs: List[torch.Tensor] = []
        self._free: List[torch.Tensor] = []
        self._allocated = {}

    @property
    def page_meta(self) -> torch.Tensor:
        return self._page_meta

    @property
    def page_nbytes(self) -> int:
        return self._page_meta.nbytes

    @property
    def num_pages(self) -> int:
        return len(self._allocated)

    def allocated_pages(self) -> Iterable[torch.Tensor]:
        return iter(self._allocated.values())

    def alloc_page(self) -> torch.Tensor:
        if not self._free:
            slab = torch.empty((self._pages_per_slab,) + self._page_shape, dtype=self.dtype, device=self.device)
            self._slabs.append(slab)
            self._free.extend(slab[i] for i in range(self._pages_per_slab - 1, -1, -1))
        page = self._free.pop()
        self._allocated[page.data_ptr()] = page
        return page

    def free_page(self, page: torch.Tensor) -> None:
        del self._allocated[page.data_ptr()]
        self._free.append(page)


class GrowableTensor:
    """A 1-D device tensor that grows by doubling (kvcache.py:52-84 of the reference)."""

    def __init__(self, data: Sequence[Any], dtype: Optional[torch.dtype] = None, device=None):
        self._buf = torch.tensor(list(data), dtype=dtype, device=device)
        self._len = len(data)

    def view(self) -> torch.Tensor:
        return self._buf[:self._len]

    def append(self, data: Any) -> None:
        if self._buf.numel() < self._len + 1:
            cap = 1 << max(0, self._len).bit_length()
            new = torch.empty(max(cap, 1), dtype=self._buf.dtype, device=self._buf.device)
            new[:self._len] = self._buf[:self._len]
            self._buf = new
        self._buf[self._len] = data
        self._len += 1

    def clear(self) -> None:
        self._len = 0


class KvCache:
    """Key-value cache for one sequence."""

    def __init__(self, pool: KvPool, init_len: int):
        if init_len < 0:
            raise ValueError("init_len must be non-negative")
        self._pool = pool
        if init_len > 0:
            npages = (init_len + pool.page_len - 1) // pool.page_len
            self._pages = [pool.alloc_page() for _ in range(npages)]
            self._seqlen = init_len
        else:
            self._pages = []
            self._seqlen = 0
        self._ptrs = GrowableTensor([t.data_ptr() for t in self._pages], dtype=torch.int64, device=pool.device)

    pool = property(lambda self: self._pool)
    seqlen = property(lambda self: self._seqlen)
    ptrs = property(lambda self: self._ptrs.view())
    pages = property(lambda self: self._pages)
    num_pages = property(lambda self: len(self._pages))

    def acquire_one(self):
        """Reserve space for one more token."""
        last_page_offset = (self._seqlen - 1) % self._pool.page_len + 1
        if last_page_offset == self._pool.page_len:
            self._pages.append(self._pool.alloc_page())
            self._ptrs.append(self._pages[-1].data_ptr())
        self._seqlen += 1

    def release(self):
        """Release all pages."""
        self._seqlen = 0
        for page in self._pages:
            self._pool.free_page(page)
        self._pages.clear()
        self._ptrs.clear()


class BatchedKvCache:
    """Key-value cache for a batch of sequences: page pointers of all sequences back to back, the page
    index pointer and the number of valid entries of every last page."""

    def __init__(self, kv: Sequence[KvCache]):
        assert len(kv) > 0
        pool = kv[0].pool
        ptrs, indptr, last = [], [0], []
        for c in kv:
            assert c.pool is pool
            assert c.num_pages > 0
            ptrs.append(c.ptrs)
            indptr.append(indptr[-1] + c.num_pages)
            last.append((c.seqlen - 1) % pool.page_len + 1)
        self.pool = pool
        self.ptrs = torch.cat(ptrs)
        self.indptr = torch.tensor(indptr, dtype=torch.int32, device=pool.device)
        self.last_page_offset = torch.tensor(last, dtype=torch.int32, device=pool.device)


# ---------------------------------------------------------------------------
# operators (the reference's loquetier.ops.batch_decode / init_kv / append_kv)
# ---------------------------------------------------------------------------

_WORKSPACES = {}
_WS_SHAPE = {}


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _dtype_code(t):
    try:
        return _DT[t.dtype]
    except KeyError:
        raise RuntimeError(f"No suitable kernel. dtype={t.dtype}") from None


def decode_workspace(device, batch: int, num_qo_heads: int, num_kv_heads: int) -> Optional[torch.Tensor]:
    """Scratch of the decode kernel with its tickets zeroed, cached per device and grown on demand.  The kernel
    leaves the tickets zeroed, but another batch shape moves the boundary between tickets and parked softmax
    states, so the head is cleared again whenever the shape differs from the previous one.  Ask for it right
    before the launch; calls that may overlap on different streams need workspaces of their own."""
    shape = (int(batch), int(num_qo_heads), int(num_kv_heads))
    need = int(lib.smlm_b200_batch_decode_workspace_bytes(*shape))
    ws = _WORKSPACES.get(device)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(max(need, 1 << 16), dtype=torch.uint8, device=device)
        _WORKSPACES[device] = ws
    elif _WS_SHAPE.get(device) != shape:
        tickets = int(lib.smlm_b200_batch_decode_ticket_bytes(int(batch), int(num_kv_heads)))
        if tickets > 0:
            with torch.cuda.device(device):
                ws[:tickets].zero_()
    _WS_SHAPE[device] = shape
    return ws


def batch_decode_into(o, q, kv_ptrs, kv_indptr, last_page_offset, num_layers, layer_idx, num_kv_heads, base, page_size,
                      workspace=None, status_word=None):
    ws = workspace if workspace is not None else decode_workspace(q.device, q.size(0), q.size(1), num_kv_heads)
    with torch.cuda.device(q.device):
        check(lib.smlm_b200_batch_decode(o.data_ptr(), q.data_ptr(), kv_ptrs.data_ptr(), kv_indptr.data_ptr(),
                                         last_page_offset.data_ptr(), ws.data_ptr(), ws.numel(),
                                         None if status_word is None else status_word.data_ptr(),
                                         int(q.size(0)), int(kv_ptrs.numel()), int(q.size(1)), int(num_kv_heads),
                                         int(q.size(2)), int(num_layers), int(layer_idx), int(page_size), float(base),
                                         _dtype_code(q), _stream(q)), "smlm_b200_batch_decode")
    return o


def batch_decode(q: torch.Tensor, kv: BatchedKvCache, base: float, layer_idx: int) -> torch.Tensor:
    """Self-attention with rotary position encoding for a batch of one-token requests.  ``q``
    ``[batch, num_heads, head_dim]`` and the keys in ``kv`` are NOT position encoded.  Returns
    ``[batch, num_heads, head_dim]``."""
    o = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    return batch_decode_into(o, q, kv.ptrs, kv.indptr, kv.last_page_offset, kv.pool.num_layers, layer_idx,
                             kv.pool.num_heads, base, kv.pool.page_len)


_PREFILL_WS = {}


def prefill_workspace(device, total_pages: int, page_size: int, num_kv_heads: int) -> torch.Tensor:
    """Scratch of the prefill kernels (a dense, rotated copy of the batch's keys and values), cached per
    device and grown on demand.  Calls that may overlap on different streams need workspaces of their own."""
    need = int(lib.smlm_b200_batch_prefill_workspace_bytes(int(total_pages), int(page_size), int(num_kv_heads)))
    ws = _PREFILL_WS.get(device)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=device)
        _PREFILL_WS[device] = ws
    return ws


def batch_prefill_into(o, q, qo_indptr, kv_ptrs, kv_indptr, last_page_offset, num_layers, layer_idx, num_kv_heads,
                       base, page_size, workspace=None, status_word=None):
    ws = workspace if workspace is not None else prefill_workspace(q.device, kv_ptrs.numel(), page_size,
                                                                   num_kv_heads)
    with torch.cuda.device(q.device):
        check(lib.smlm_b200_batch_prefill(o.data_ptr(), q.data_ptr(), qo_indptr.data_ptr(), kv_ptrs.data_ptr(),
                                          kv_indptr.data_ptr(), last_page_offset.data_ptr(), ws.data_ptr(),
                                          ws.numel(), None if status_word is None else status_word.data_ptr(),
                                          int(last_page_offset.numel()), int(q.size(0)), int(kv_ptrs.numel()),
                                          int(q.size(1)), int(num_kv_heads), int(q.size(2)), int(num_layers),
                                          int(layer_idx), int(page_size), float(base), _dtype_code(q), _stream(q)),
              "smlm_b200_batch_prefill")
    return o


def batch_prefill(q: torch.Tensor, qo_indptr: torch.Tensor, kv: BatchedKvCache, base: float,
                  layer_idx: int) -> torch.Tensor:
    """Causal self-attention with rotary position encoding for each prompt of the batch
    (batch_prefill, kernel_src/src/loquetier/ops/__init__.py:18-57).  ``q``
    ``[sum(seqlen), num_heads, head_dim]`` and the keys in ``kv`` are NOT position encoded; request b owns
    rows ``qo_indptr[b] .. qo_indptr[b + 1]`` (int32, on the device).  Returns the attention output in the
    shape of ``q``."""
    o = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    return batch_prefill_into(o, q, qo_indptr, kv.ptrs, kv.indptr, kv.last_page_offset, kv.pool.num_layers,
                              layer_idx, kv.pool.num_heads, base, kv.pool.page_len)


def init_kv_raw(kv_ptrs, kv_indptr, last_page_offset, k, v, seqlen_indptr, num_layers, layer_idx, num_kv_heads,
                page_size, status_word=None):
    with torch.cuda.device(k.device):
        check(lib.smlm_b200_init_kv(kv_ptrs.data_ptr(), kv_indptr.data_ptr(), last_page_offset.data_ptr(),
                                    k.data_ptr(), v.data_ptr(), seqlen_indptr.data_ptr(),
                                    None if status_word is None else status_word.data_ptr(),
                                    int(last_page_offset.numel()), int(kv_ptrs.numel()), int(k.size(0)),
                                    int(num_layers), int(layer_idx), int(num_kv_heads), int(k.size(2)),
                                    int(page_size), _dtype_code(k), _stream(k)), "smlm_b200_init_kv")


def init_kv(kv: BatchedKvCache, k: torch.Tensor, v: torch.Tensor, seqlen_indptr: torch.Tensor, layer_idx: int):
    """Copy ``k`` and ``v`` ``[sum(seqlen), num_heads, head_dim]`` to the cache; the pages of each
    sequence are already allocated in ``kv``."""
    init_kv_raw(kv.ptrs, kv.indptr, kv.last_page_offset, k, v, seqlen_indptr, kv.pool.num_layers, layer_idx,
                kv.pool.num_heads, kv.pool.page_len)


def append_kv_raw(kv_ptrs, kv_indptr, last_page_offset, k, v, num_layers, layer_idx, num_kv_heads, page_size,
                  status_word=None):
    with torch.cuda.device(k.device):
        check(lib.smlm_b200_append_kv(kv_ptrs.data_ptr(), kv_indptr.data_ptr(), last_page_offset.data_ptr(),
                                      k.data_ptr(), v.data_ptr(),
                                      None if status_word is None else status_word.data_ptr(), int(k.size(0)),
                                      int(kv_ptrs.numel()), int(num_layers), int(layer_idx), int(num_kv_heads),
                                      int(k.size(2)), int(page_size), _dtype_code(k), _stream(k)),
              "smlm_b200_append_kv")


def append_kv(kv: BatchedKvCache, k: torch.Tensor, v: torch.Tensor, layer_idx: int):
    """Append the new token's ``k`` and ``v`` ``[batch, num_heads, head_dim]``; the page for the new token
    of each sequence is already allocated in ``kv``."""
    append_kv_raw(kv.ptrs, kv.indptr, kv.last_page_offset, k, v, kv.pool.num_layers, layer_idx, kv.pool.num_heads,
                  kv.pool.page_len)
