"""CPU oracle of the paged key-value cache next to the SMLM path: appending keys/values to the pages
and batch decode attention over them.

TEST INFRASTRUCTURE ONLY: the checker the CUDA kernels are compared against.  Nothing in the product
package imports it.

What it restates (paths inside the reference checkout):

* page layout ``[num_layers, 2, num_kv_heads, page_size, head_dim]`` per page and the address arithmetic
  ``get_k_elem_offset_in_page`` / ``kv_offset_delta`` -
  kernel_src/third_party/flashinfer/include/flashinfer/page.cuh:246-251, 291-293;
  sequence length ``(pages - 1) * page_size + last_page_offset`` - page.cuh:377-379;
  the batch description (page pointers, page indptr, last_page_offset = (seqlen - 1) % page_len + 1) -
  kernel_src/src/loquetier/utils/kvcache.py:143-165.
* ``append_kv``  - AppendPagedKVCacheDecodeKernel, page.cuh:368-396: the new token goes to entry
  ``(seq_len - 1) % page_size`` of page ``(seq_len - 1) // page_size``.
* ``init_kv``    - AppendPagedKVCachePrefillKernel, page.cuh:411-444: the run of new tokens fills the
  LAST ``n`` positions of the sequence.
* ``batch_prefill`` - BatchPrefillWithPagedKVCacheKernel, prefill.cuh:904-1060 (causal; query i of a request
  at position ``kv_len - qo_len + i``); same rotation, scale and softmax as below.
* ``batch_decode`` - BatchDecodeWithPagedKVCacheKernel, decode.cuh:451-620, with the settings of
  FlashInferBatchDecodeKernel (kernel_src/csrc/flashinfer_adapter/flashinfer_all.cu:85-108): Llama
  rotary mode, rope scale 1, ``sm_scale = 1 / sqrt(head_dim)`` (decode.cuh:1052); the query is rotated
  at position ``seq_len - 1`` (:489-494), every key at its own position as it is read (:108-111);
  rotation of element i: ``x[i] * cos + (i < d/2 ? -x[i + d/2] : x[i - d/2]) * sin`` with angle
  ``pos * theta ** (-2 * (i % (d/2)) / d)`` (:59-76, :480-483); softmax over all positions; output in
  the storage type.  The reference evaluates sin/cos and the power with fast device intrinsics; the
  oracle evaluates them in float64, which is the value those intrinsics approximate.

Parity pin: the attention code of the reference is vendored third-party CUDA that cannot run in a
CPU-only container and ships no golden vectors; the oracle is pinned on the GPU box against the
reference's own kernels compiled from its headers (``oracle/build_ref.py``, tests in
``tests/test_gpu_ref_cuda.py``), and on the CPU against an independent dense evaluation
(``tests/test_attention_oracle.py``)."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch


def seq_len_of(n_pages: int, last_page_offset: int, page_size: int) -> int:
    return (n_pages - 1) * page_size + last_page_offset if n_pages > 0 else 0


def last_page_offset_of(seqlen: int, page_size: int) -> int:
    """kvcache.py:158: valid entries of the last page, 1 .. page_size."""
    return (seqlen - 1) % page_size + 1


def append_kv(pages: Sequence[torch.Tensor], indptr: Sequence[int], last_page_offset: Sequence[int],
              k: torch.Tensor, v: torch.Tensor, layer_idx: int) -> None:
    """One new token per request; ``pages[i]`` is ``[L, 2, N, P, D]``; k, v ``[B, N, D]``."""
    P = pages[0].shape[3]
    for b in range(len(indptr) - 1):
        n = indptr[b + 1] - indptr[b]
        sl = seq_len_of(n, last_page_offset[b], P)
        page = pages[indptr[b] + (sl - 1) // P]
        e = (sl - 1) % P
        page[layer_idx, 0, :, e, :] = k[b]
        page[layer_idx, 1, :, e, :] = v[b]


def init_kv(pages: Sequence[torch.Tensor], indptr: Sequence[int], last_page_offset: Sequence[int],
            k: torch.Tensor, v: torch.Tensor, seqlen_indptr: Sequence[int], layer_idx: int) -> None:
    """A run of new tokens per request, written to the last positions of its sequence."""
    P = pages[0].shape[3]
    for b in range(len(indptr) - 1):
        sl = seq_len_of(indptr[b + 1] - indptr[b], last_page_offset[b], P)
        a0, a1 = seqlen_indptr[b], seqlen_indptr[b + 1]
        start = sl - (a1 - a0)
        for j in range(a1 - a0):
            pos = start + j
            page = pages[indptr[b] + pos // P]
            page[layer_idx, 0, :, pos % P, :] = k[a0 + j]
            page[layer_idx, 1, :, pos % P, :] = v[a0 + j]


def gather_kv(pages: Sequence[torch.Tensor], p0: int, p1: int, last: int, layer_idx: int):
    """Keys and values of one request as ``[L_seq, N, D]`` float64 tensors."""
    P = pages[0].shape[3]
    sl = seq_len_of(p1 - p0, last, P)
    ks, vs = [], []
    for i in range(p0, p1):
        ks.append(pages[i][layer_idx, 0].permute(1, 0, 2))   # [P, N, D]
        vs.append(pages[i][layer_idx, 1].permute(1, 0, 2))
    if not ks:
        z = torch.zeros((0,) + tuple(pages[0].shape[2:3]) + tuple(pages[0].shape[4:]), dtype=torch.float64)
        return z, z
    return torch.cat(ks)[:sl].to(torch.float64), torch.cat(vs)[:sl].to(torch.float64)


def rope(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """Llama rotary embedding of ``x [..., D]`` (float64) at integer positions ``pos`` broadcastable to
    ``x.shape[:-1]``."""
    D = x.shape[-1]
    half = D // 2
    i = torch.arange(D, dtype=torch.float64)
    freq = torch.tensor(theta, dtype=torch.float64) ** (-2.0 * (i % half) / D)
    ang = pos.to(torch.float64).unsqueeze(-1) * freq
    partner = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * torch.cos(ang) + partner * torch.sin(ang)


def batch_decode(q: torch.Tensor, pages: Sequence[torch.Tensor], indptr: Sequence[int],
                 last_page_offset: Sequence[int], layer_idx: int, rope_theta: float) -> torch.Tensor:
    """``q [B, Nq, D]`` in the storage type; returns ``o [B, Nq, D]`` in the same type."""
    B, Nq, D = q.shape
    N = pages[0].shape[2]
    G = Nq // N
    out = torch.zeros((B, Nq, D), dtype=torch.float64)
    for b in range(B):
        K, V = gather_kv(pages, indptr[b], indptr[b + 1], last_page_offset[b], layer_idx)
        L = K.shape[0]
        if L == 0:
            continue
        qr = rope(q[b].to(torch.float64), torch.full((Nq,), L - 1), rope_theta)          # [Nq, D]
        kr = rope(K.permute(1, 0, 2), torch.arange(L).expand(N, L), rope_theta)           # [N, L, D]
        for h in range(Nq):
            logits = (kr[h // G] @ qr[h]) / np.sqrt(D)
            p = torch.softmax(logits, dim=0)
            out[b, h] = p @ V[:, h // G, :]
    return out.to(q.dtype)


def batch_prefill(q: torch.Tensor, qo_indptr: Sequence[int], pages: Sequence[torch.Tensor], indptr: Sequence[int],
                  last_page_offset: Sequence[int], layer_idx: int, rope_theta: float) -> torch.Tensor:
    """Causal self-attention of a ragged batch of prompts over their paged caches
    (BatchPrefillWithPagedKVCacheKernel, prefill.cuh:904-1060, with the settings of
    FlashInferBatchPrefillKernel, flashinfer_all.cu:48-83: causal, Llama rotary mode, rope scale 1).
    ``q [sum(qo_len), Nq, D]``; request b owns rows ``qo_indptr[b] .. qo_indptr[b + 1]``; its cache already
    holds all ``kv_len >= qo_len`` keys (init_kv ran before).  Query i of a request sits at position
    ``kv_len - qo_len + i`` (prefill.cuh:262) and sees the keys at positions up to its own (:397)."""
    Tq, Nq, D = q.shape
    N = pages[0].shape[2]
    G = Nq // N
    out = torch.zeros((Tq, Nq, D), dtype=torch.float64)
    for b in range(len(qo_indptr) - 1):
        a0, a1 = qo_indptr[b], qo_indptr[b + 1]
        n = a1 - a0
        if n <= 0:
            continue
        K, V = gather_kv(pages, indptr[b], indptr[b + 1], last_page_offset[b], layer_idx)
        L = K.shape[0]
        pos_q = torch.arange(L - n, L)
        qr = rope(q[a0:a1].to(torch.float64).permute(1, 0, 2), pos_q.expand(Nq, n), rope_theta)    # [Nq, n, D]
        kr = rope(K.permute(1, 0, 2), torch.arange(L).expand(N, L), rope_theta)                     # [N, L, D]
        mask = torch.arange(L).unsqueeze(0) > pos_q.unsqueeze(1)                                     # [n, L]
        for h in range(Nq):
            logits = (qr[h] @ kr[h // G].t()) / np.sqrt(D)
            logits = logits.masked_fill(mask, float("-inf"))
            p = torch.softmax(logits, dim=1)
            out[a0:a1, h] = p @ V[:, h // G, :]
    return out.to(q.dtype)


def make_cache(seed: int, seqlens: Sequence[int], num_layers: int, num_kv_heads: int, page_size: int, head_dim: int,
               dtype: torch.dtype, shuffle: bool = True):
    """Seeded synthetic cache: every request gets ceil(seqlen / page_size) pages drawn from a pool in a
    shuffled order (so that neighbouring pages of a request are not neighbours in memory).  Returns
    (pages list, indptr, last_page_offset)."""
    g = torch.Generator().manual_seed(int(seed))
    n_pages = [(s + page_size - 1) // page_size for s in seqlens]
    total = sum(n_pages)
    order = torch.randperm(total, generator=g).tolist() if shuffle else list(range(total))
    pool = [torch.randn((num_layers, 2, num_kv_heads, page_size, head_dim), generator=g).to(dtype) for _ in range(total)]
    pages = [pool[i] for i in order]
    indptr = [0]
    for n in n_pages:
        indptr.append(indptr[-1] + n)
    last = [last_page_offset_of(s, page_size) if s > 0 else 0 for s in seqlens]
    return pages, indptr, last
