"""The paged key-value cache on the GPU through the C ABI: appending keys/values (bit-exact), batch
decode and causal prefill attention (rtol = atol = 1e-2 for 16-bit storage with fp32 arithmetic) against the CPU oracle,
and - where oracle/_ref/libref.so has been built - against the reference's own kernels."""
import os

import numpy as np
import pytest
import torch

import ref_cuda
from helpers import assert_close
from oracle import attention_oracle as A

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
THETA = 10000.0
MORE = max(1, int(os.environ.get("SMLM_RANDOM_SEEDS", "1")))   # multiplies the seeds of the random-shape tests


def _to_dev(pages, indptr, last):
    pd = [p.to(DEV).contiguous() for p in pages]
    ptrs = torch.tensor([p.data_ptr() for p in pd], dtype=torch.int64, device=DEV)
    return pd, ptrs, torch.tensor(indptr, dtype=torch.int32, device=DEV), torch.tensor(last, dtype=torch.int32, device=DEV)


def _decode(q, ptrs, ind, last, Lyr, layer, N, P):
    from loquetier_b200 import kvcache
    o = torch.full(q.shape, 7.0, dtype=q.dtype, device=DEV)
    word = torch.zeros(1, dtype=torch.int32, device=DEV)
    kvcache.batch_decode_into(o, q, ptrs, ind, last, Lyr, layer, N, THETA, P, status_word=word)
    torch.cuda.synchronize()
    assert int(word.item()) == 0, f"fault bits {int(word.item())}"
    return o


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("group,P", [(1, 16), (2, 8), (4, 16), (8, 16), (4, 32), (8, 8)])
def test_decode_matches_oracle_small_batch_many_splits(dtype, group, P):
    N, Lyr, layer = 2, 3, 1
    seqlens = [1, 15, 16, 17, 100, 333, 1000]      # 7 requests x 2 kv heads: the launch cuts them into page ranges
    pages, indptr, last = A.make_cache(11 + group + P, seqlens, Lyr, N, P, 128, dtype)
    g = torch.Generator().manual_seed(group * 31 + P)
    q = torch.randn((len(seqlens), N * group, 128), generator=g).to(dtype)
    pd, ptrs, ind, lst = _to_dev(pages, indptr, last)
    o = _decode(q.to(DEV), ptrs, ind, lst, Lyr, layer, N, P)
    want = A.batch_decode(q, pages, indptr, last, layer, THETA)
    assert_close(o, want, what=f"group {group} page {P}")
    # bit-exact on a second run: the merge order of the page ranges is fixed
    o2 = _decode(q.to(DEV), ptrs, ind, lst, Lyr, layer, N, P)
    assert torch.equal(o, o2)


def test_decode_matches_oracle_large_batch_one_range_per_request():
    """Enough (request, kv head) pairs to fill the machine: no page ranges, no workspace traffic."""
    from loquetier_b200.cabi import lib
    N, group, P, Lyr = 8, 4, 16, 1
    rng = np.random.default_rng(5)
    seqlens = [int(v) for v in rng.integers(1, 200, size=64)]
    assert lib.smlm_b200_batch_decode_workspace_bytes(64, 32, 8) < (2 << 20)   # one range: 132 floats per (request, head)
    pages, indptr, last = A.make_cache(21, seqlens, Lyr, N, P, 128, torch.bfloat16)
    g = torch.Generator().manual_seed(22)
    q = torch.randn((64, N * group, 128), generator=g).to(torch.bfloat16)
    pd, ptrs, ind, lst = _to_dev(pages, indptr, last)
    o = _decode(q.to(DEV), ptrs, ind, lst, Lyr, 0, N, P)
    assert_close(o, A.batch_decode(q, pages, indptr, last, 0, THETA), what="64 requests")


def test_decode_long_sequence_rotation_stays_accurate():
    """8000 positions: the rotation is carried by a recurrence between accurate evaluations."""
    N, group, P = 1, 4, 16
    pages, indptr, last = A.make_cache(31, [8000, 4097], 1, N, P, 128, torch.bfloat16)
    g = torch.Generator().manual_seed(32)
    q = torch.randn((2, 4, 128), generator=g).to(torch.bfloat16)
    pd, ptrs, ind, lst = _to_dev(pages, indptr, last)
    o = _decode(q.to(DEV), ptrs, ind, lst, 1, 0, N, P)
    assert_close(o, A.batch_decode(q, pages, indptr, last, 0, THETA), what="long")


def test_append_and_init_are_bit_exact_and_touch_nothing_else():
    from loquetier_b200 import kvcache
    P, N, Lyr, dt = 16, 4, 2, torch.bfloat16
    seqlens = [17, 3, 32, 16, 1]
    pages, indptr, last = A.make_cache(41, seqlens, Lyr, N, P, 128, dt)
    pd, ptrs, ind, lst = _to_dev(pages, indptr, last)
    g = torch.Generator().manual_seed(42)
    k, v = torch.randn((5, N, 128), generator=g).to(dt), torch.randn((5, N, 128), generator=g).to(dt)
    word = torch.zeros(1, dtype=torch.int32, device=DEV)
    kvcache.append_kv_raw(ptrs, ind, lst, k.to(DEV), v.to(DEV), Lyr, 1, N, P, status_word=word)
    A.append_kv(pages, indptr, last, k, v, 1)
    runs = [4, 3, 20, 16, 1]
    sind = [0] + list(np.cumsum(runs))
    k2, v2 = torch.randn((44, N, 128), generator=g).to(dt), torch.randn((44, N, 128), generator=g).to(dt)
    kvcache.init_kv_raw(ptrs, ind, lst, k2.to(DEV), v2.to(DEV), torch.tensor(sind, dtype=torch.int32, device=DEV), Lyr, 0,
                        N, P, status_word=word)
    A.init_kv(pages, indptr, last, k2, v2, sind, 0)
    torch.cuda.synchronize()
    assert int(word.item()) == 0
    for got, want in zip(pd, pages):
        assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16))


def test_reference_named_operators_and_cache_classes_decode_step():
    """One decode step as the reference's model issues it (mixed_llama.py:176-186 there): reserve a slot per
    sequence, append the new key/value, attend - with the mirrored KvPool / KvCache / BatchedKvCache and
    the operators under the reference's names."""
    from loquetier_b200 import kernels, kvcache
    dt = torch.bfloat16
    Lyr, N, G, P = 2, 2, 4, 16
    pool = kvcache.KvPool(Lyr, N, 128, P, dt, DEV, pages_per_slab=8)
    lens = [5, 16, 31]
    g = torch.Generator().manual_seed(51)
    caches, hist = [], []
    for L in lens:
        c = kvcache.KvCache(pool, L)
        caches.append(c)
        assert c.num_pages == (L + P - 1) // P and c.ptrs.tolist() == [p.data_ptr() for p in c.pages]
    assert pool.num_pages == 1 + 1 + 2
    b0 = kvcache.BatchedKvCache(caches)
    for layer in range(Lyr):
        k0 = torch.randn((sum(lens), N, 128), generator=g).to(dt)
        v0 = torch.randn((sum(lens), N, 128), generator=g).to(dt)
        hist.append((k0, v0))
        kvcache.init_kv(b0, k0.to(DEV), v0.to(DEV), torch.tensor([0, 5, 21, 52], dtype=torch.int32, device=DEV), layer)
    for c in caches:
        c.acquire_one()                       # 16 -> 17 tokens opens a second page
    assert [c.seqlen for c in caches] == [6, 17, 32] and caches[1].num_pages == 2
    b1 = kvcache.BatchedKvCache(caches)
    assert b1.indptr.tolist() == [0, 1, 3, 5] and b1.last_page_offset.tolist() == [6, 1, 16]
    layer = 1
    kn, vn = torch.randn((3, N, 128), generator=g).to(dt), torch.randn((3, N, 128), generator=g).to(dt)
    q = torch.randn((3, N * G, 128), generator=g).to(dt)
    kernels.append_kv(b1.ptrs, b1.indptr, b1.last_page_offset, kn.to(DEV), vn.to(DEV), Lyr, layer, N, P)
    o = kvcache.batch_decode(q.to(DEV), b1, THETA, layer)
    o_named = torch.empty_like(o)
    kernels.batch_decode(o_named, q.to(DEV), b1.ptrs, b1.indptr, b1.last_page_offset,
                         torch.empty(1 << 16, dtype=torch.uint8, device=DEV), Lyr, layer, N, THETA, P)
    torch.cuda.synchronize()
    assert torch.equal(o, o_named)
    # dense answer from the history of that layer
    k0, v0 = hist[layer]
    off, want = 0, []
    for i, L in enumerate(lens):
        K = torch.cat([k0[off:off + L], kn[i:i + 1]]).double()
        V = torch.cat([v0[off:off + L], vn[i:i + 1]]).double()
        off += L
        qr = A.rope(q[i].double(), torch.full((N * G,), L), THETA)
        kr = A.rope(K.permute(1, 0, 2), torch.arange(L + 1).expand(N, L + 1), THETA)
        rows = []
        for h in range(N * G):
            p = torch.softmax((kr[h // G] @ qr[h]) / np.sqrt(128), dim=0)
            rows.append(p @ V[:, h // G, :])
        want.append(torch.stack(rows))
    assert_close(o, torch.stack(want), what="decode step")
    for c in caches:
        c.release()
    assert pool.num_pages == 0
    with pytest.raises(RuntimeError, match="No suitable kernel"):
        kernels.batch_decode(torch.empty((1, 6, 128), dtype=dt, device=DEV), torch.empty((1, 6, 128), dtype=dt, device=DEV),
                             b1.ptrs[:1], b1.indptr[:2], b1.last_page_offset[:1],
                             torch.empty(1 << 16, dtype=torch.uint8, device=DEV), Lyr, 0, 2, THETA, P)   # group 3


def test_bad_page_table_is_reported_not_followed():
    from loquetier_b200 import kvcache
    P, N = 16, 2
    pages, indptr, last = A.make_cache(61, [20, 20], 1, N, P, 128, torch.bfloat16)
    pd, ptrs, ind, lst = _to_dev(pages, indptr, last)
    q = torch.randn((2, 8, 128), device=DEV).to(torch.bfloat16)
    o = torch.zeros_like(q)
    word = torch.zeros(1, dtype=torch.int32, device=DEV)
    bad = torch.tensor([0, 2, 9], dtype=torch.int32, device=DEV)          # reaches past the 4 pages
    kvcache.batch_decode_into(o, q, ptrs, bad, lst, 1, 0, N, THETA, P, status_word=word)
    torch.cuda.synchronize()
    assert int(word.item()) & 1
    word.zero_()
    ptrs2 = ptrs.clone()
    ptrs2[1] = 0                                                           # a null page
    kvcache.batch_decode_into(o, q, ptrs2, ind, lst, 1, 0, N, THETA, P, status_word=word)
    torch.cuda.synchronize()
    assert int(word.item()) & 2


@pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref/libref.so not built")
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("group", [1, 4, 8])
def test_decode_and_append_against_reference_kernels(dtype, group):
    """Three-way: the reference's flashinfer kernels, this library, the oracle (page size 16, head dim 128)."""
    from loquetier_b200 import kvcache
    N, Lyr, layer, P = 2, 2, 1, 16
    seqlens = [1, 16, 17, 250, 1031]
    pages, indptr, last = A.make_cache(71 + group, seqlens, Lyr, N, P, 128, dtype)
    g = torch.Generator().manual_seed(72)
    q = torch.randn((5, N * group, 128), generator=g).to(dtype)
    kn, vn = torch.randn((5, N, 128), generator=g).to(dtype), torch.randn((5, N, 128), generator=g).to(dtype)
    pd_ref, ptrs_ref, ind, lst = _to_dev(pages, indptr, last)
    pd_lib, ptrs_lib, _, _ = _to_dev(pages, indptr, last)
    ref_cuda.append_kv(ptrs_ref, ind, lst, kn.to(DEV), vn.to(DEV), Lyr, layer, N, P)
    kvcache.append_kv_raw(ptrs_lib, ind, lst, kn.to(DEV), vn.to(DEV), Lyr, layer, N, P)
    A.append_kv(pages, indptr, last, kn, vn, layer)
    torch.cuda.synchronize()
    for a, b, c in zip(pd_ref, pd_lib, pages):
        assert torch.equal(a, b) and torch.equal(a.cpu().view(torch.int16), c.view(torch.int16))
    o_ref = torch.zeros((5, N * group, 128), dtype=dtype, device=DEV)
    ref_cuda.batch_decode(o_ref, q.to(DEV), ptrs_ref, ind, lst, Lyr, layer, N, THETA)
    o_lib = _decode(q.to(DEV), ptrs_lib, ind, lst, Lyr, layer, N, P)
    want = A.batch_decode(q, pages, indptr, last, layer, THETA)
    assert_close(o_ref, want, what="reference kernel vs oracle")
    assert_close(o_lib, o_ref, what="library vs reference kernel")


# ---------------------------------------------------------------------------------------------
# prefill
# ---------------------------------------------------------------------------------------------

def _prefill(q, qind, ptrs, ind, last, Lyr, layer, N, P, expect_word=0):
    from loquetier_b200 import kvcache
    o = torch.full(q.shape, 7.0, dtype=q.dtype, device=DEV)
    word = torch.zeros(1, dtype=torch.int32, device=DEV)
    kvcache.batch_prefill_into(o, q, qind, ptrs, ind, last, Lyr, layer, N, THETA, P, status_word=word)
    torch.cuda.synchronize()
    assert int(word.item()) == expect_word, f"fault bits {int(word.item())}"
    return o


def _qind(qlens):
    return [0] + [int(v) for v in np.cumsum(qlens)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("group,P", [(1, 16), (2, 8), (4, 16), (8, 16), (4, 32), (1, 64)])
def test_prefill_matches_oracle(dtype, group, P):
    """Ragged prompts: shorter than a key tile, exactly a tile, ragged query tiles, several query tiles, an
    empty request, and one whose cache already held a prefix (queries are the last positions)."""
    N, Lyr, layer = 2, 2, 1
    seqlens = [1, 5, 64, 65, 130, 300, 0, 200]
    qlens = [1, 5, 64, 65, 130, 300, 0, 77]
    pages, indptr, last = A.make_cache(31 + group + P, seqlens, Lyr, N, P, 128, dtype)
    g = torch.Generator().manual_seed(group * 17 + P)
    qind = _qind(qlens)
    q = torch.randn((qind[-1], N * group, 128), generator=g).to(dtype)
    pd, ptrs, ind, lst = _to_dev(pages, indptr, last)
    o = _prefill(q.to(DEV), torch.tensor(qind, dtype=torch.int32, device=DEV), ptrs, ind, lst, Lyr, layer, N, P)
    want = A.batch_prefill(q, qind, pages, indptr, last, layer, THETA)
    assert_close(o, want, what=f"prefill group {group} page {P}")
    o2 = _prefill(q.to(DEV), torch.tensor(qind, dtype=torch.int32, device=DEV), ptrs, ind, lst, Lyr, layer, N, P)
    assert torch.equal(o, o2)


def test_prefill_long_prompt_and_last_row_is_a_decode_step():
    """2500 positions (40 key tiles, 20 query tiles per head): the running-maximum policy and the barrier
    phases go through many rounds; the last query of a prompt must agree with the decode kernel."""
    N, group, P, Lyr = 2, 4, 16, 1
    seqlens, qlens = [2500, 700], [2500, 700]
    pages, indptr, last = A.make_cache(91, seqlens, Lyr, N, P, 128, torch.bfloat16)
    g = torch.Generator().manual_seed(92)
    qind = _qind(qlens)
    q = (torch.randn((qind[-1], N * group, 128), generator=g) * 1.5).to(torch.bfloat16)
    pd, ptrs, ind, lst = _to_dev(pages, indptr, last)
    o = _prefill(q.to(DEV), torch.tensor(qind, dtype=torch.int32, device=DEV), ptrs, ind, lst, Lyr, 0, N, P)
    sel = list(range(0, 2500, 97)) + [2499, 2500, 2500 + 699]
    want = A.batch_prefill(q, qind, pages, indptr, last, 0, THETA)
    assert_close(o[sel], want[sel], what="long prompt rows")
    assert_close(o, want, what="long prompt")
    last_q = torch.stack([q[qind[1] - 1], q[qind[2] - 1]]).to(DEV)
    od = _decode(last_q, ptrs, ind, lst, Lyr, 0, N, P)
    assert_close(torch.stack([o[qind[1] - 1], o[qind[2] - 1]]), od.cpu(), what="prefill last row vs decode")


def test_prefill_large_scores_raise_the_running_maximum():
    """Scores that grow along the sequence (keys scaled up with their index): every row's maximum is raised
    again and again, so the accumulator in tensor memory is rescaled many times."""
    N, group, P, Lyr = 1, 2, 16, 1
    L = 700
    pages, indptr, last = A.make_cache(55, [L], Lyr, N, P, 128, torch.float16)
    for i, pg in enumerate(pages):
        pg[:, 0] *= 1.0 + 0.1 * i        # keys of later pages are larger
    g = torch.Generator().manual_seed(56)
    q = (torch.randn((L, N * group, 128), generator=g) * 1.5).to(torch.float16)
    pd, ptrs, ind, lst = _to_dev(pages, indptr, last)
    o = _prefill(q.to(DEV), torch.tensor([0, L], dtype=torch.int32, device=DEV), ptrs, ind, lst, Lyr, 0, N, P)
    want = A.batch_prefill(q, [0, L], pages, indptr, last, 0, THETA)
    assert_close(o, want, what="raised maxima")


def test_prefill_named_operator_and_cache_classes():
    """init_kv then batch_prefill through the mirrored classes and through the reference's binding names."""
    from loquetier_b200 import kernels, kvcache
    N, group, P, Lyr, layer = 2, 4, 16, 2, 1
    pool = kvcache.KvPool(num_layers=Lyr, num_heads=N, head_dim=128, page_len=P, dtype=torch.bfloat16, device=DEV)
    lens = [40, 129]
    caches = [kvcache.KvCache(pool, n) for n in lens]
    bkv = kvcache.BatchedKvCache(caches)
    g = torch.Generator().manual_seed(3)
    T = sum(lens)
    k = torch.randn((T, N, 128), generator=g).to(torch.bfloat16)
    v = torch.randn((T, N, 128), generator=g).to(torch.bfloat16)
    q = torch.randn((T, N * group, 128), generator=g).to(torch.bfloat16)
    qind = torch.tensor([0, 40, 169], dtype=torch.int32, device=DEV)
    kvcache.init_kv(bkv, k.to(DEV), v.to(DEV), qind, layer)
    o = kvcache.batch_prefill(q.to(DEV), qind, bkv, THETA, layer)
    o_named = torch.empty_like(o)
    kernels.batch_prefill(o_named, q.to(DEV), qind, bkv.ptrs, bkv.indptr, bkv.last_page_offset,
                          torch.empty(64, dtype=torch.uint8, device=DEV), Lyr, layer, N, THETA, P)
    torch.cuda.synchronize()
    assert torch.equal(o, o_named)
    # dense causal attention of the same k, v
    pages, indptr, last = A.make_cache(0, lens, Lyr, N, P, 128, torch.bfloat16)
    A.init_kv(pages, indptr, last, k, v, [0, 40, 169], layer)
    want = A.batch_prefill(q, [0, 40, 169], pages, indptr, last, layer, THETA)
    assert_close(o, want, what="classes")
    with pytest.raises(RuntimeError, match="No suitable kernel"):
        kernels.batch_prefill(torch.empty((4, 6, 128), dtype=torch.bfloat16, device=DEV),
                              torch.empty((4, 6, 128), dtype=torch.bfloat16, device=DEV),
                              torch.tensor([0, 4], dtype=torch.int32, device=DEV), bkv.ptrs[:1], bkv.indptr[:2],
                              bkv.last_page_offset[:1], torch.empty(64, dtype=torch.uint8, device=DEV), Lyr, layer, 2,
                              THETA, P)   # 6 query heads on 2 kv heads: a group of 3


def test_prefill_more_queries_than_keys_is_reported_not_faulted():
    N, group, P, Lyr = 1, 1, 16, 1
    pages, indptr, last = A.make_cache(8, [10], Lyr, N, P, 128, torch.bfloat16)
    q = torch.randn((20, 1, 128)).to(torch.bfloat16)
    pd, ptrs, ind, lst = _to_dev(pages, indptr, last)
    o = _prefill(q.to(DEV), torch.tensor([0, 20], dtype=torch.int32, device=DEV), ptrs, ind, lst, Lyr, 0, N, P,
                 expect_word=1)
    assert torch.isfinite(o.float()).all()
    assert float(o[:10].float().abs().max()) == 0.0     # positions -10 .. -1 see no key


@pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref/libref.so not built")
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("group", [1, 4, 8])
def test_prefill_against_reference_kernel(dtype, group):
    """Three-way: the reference's flashinfer prefill kernel, this library, the oracle (page 16, head dim 128)."""
    N, Lyr, layer, P = 2, 2, 1, 16
    seqlens = [3, 64, 100, 517]
    qlens = [3, 64, 100, 517]
    pages, indptr, last = A.make_cache(171 + group, seqlens, Lyr, N, P, 128, dtype)
    g = torch.Generator().manual_seed(172)
    qind = _qind(qlens)
    q = torch.randn((qind[-1], N * group, 128), generator=g).to(dtype)
    pd, ptrs, ind, lst = _to_dev(pages, indptr, last)
    qi = torch.tensor(qind, dtype=torch.int32, device=DEV)
    o_ref = torch.zeros(q.shape, dtype=dtype, device=DEV)
    ref_cuda.batch_prefill(o_ref, q.to(DEV), qi, ptrs, ind, lst, Lyr, layer, N, THETA)
    o_lib = _prefill(q.to(DEV), qi, ptrs, ind, lst, Lyr, layer, N, P)
    want = A.batch_prefill(q, qind, pages, indptr, last, layer, THETA)
    assert_close(o_ref, want, what="reference kernel vs oracle")
    assert_close(o_lib, o_ref, what="library vs reference kernel")



def test_prefill_many_short_requests():
    """More requests than one pass of the kernels' request scan covers (32 per pass), some of them empty."""
    N, group, P, Lyr = 2, 4, 16, 1
    rng = np.random.default_rng(77)
    seqlens = [int(v) for v in rng.integers(0, 41, size=70)]
    seqlens[33] = 0
    qlens = list(seqlens)
    pages, indptr, last = A.make_cache(401, seqlens, Lyr, N, P, 128, torch.bfloat16)
    g = torch.Generator().manual_seed(402)
    qind = _qind(qlens)
    q = torch.randn((qind[-1], N * group, 128), generator=g).to(torch.bfloat16)
    pd, ptrs, ind, lst = _to_dev(pages, indptr, last)
    o = _prefill(q.to(DEV), torch.tensor(qind, dtype=torch.int32, device=DEV), ptrs, ind, lst, Lyr, 0, N, P)
    want = A.batch_prefill(q, qind, pages, indptr, last, 0, THETA)
    assert_close(o, want, what="70 short requests")


@pytest.mark.parametrize("seed", list(range(12 * MORE)))
def test_prefill_random_shapes(seed):
    """Seeded random batches: group size, page size, kv heads, layers, batch size, cached prefix lengths and
    storage type all vary; every row against the oracle."""
    rng = np.random.default_rng(9000 + seed)
    group = int(rng.choice([1, 2, 4, 8]))
    P = int(rng.choice([8, 16, 32, 64]))
    N = int(rng.integers(1, 4))
    Lyr = int(rng.integers(1, 3))
    layer = int(rng.integers(0, Lyr))
    dtype = torch.bfloat16 if seed % 2 == 0 else torch.float16
    B = int(rng.integers(1, 10))
    seqlens = [int(v) for v in rng.integers(0, 260, size=B)]
    qlens = [int(rng.integers(0, L + 1)) if rng.random() < 0.4 else L for L in seqlens]
    if sum(qlens) == 0:
        seqlens[0], qlens[0] = 70, 70
    pages, indptr, last = A.make_cache(9100 + seed, seqlens, Lyr, N, P, 128, dtype)
    g = torch.Generator().manual_seed(9200 + seed)
    qind = _qind(qlens)
    q = torch.randn((qind[-1], N * group, 128), generator=g).to(dtype)
    pd, ptrs, ind, lst = _to_dev(pages, indptr, last)
    o = _prefill(q.to(DEV), torch.tensor(qind, dtype=torch.int32, device=DEV), ptrs, ind, lst, Lyr, layer, N, P)
    want = A.batch_prefill(q, qind, pages, indptr, last, layer, THETA)
    assert_close(o, want, what=f"seed {seed}: group {group} page {P} heads {N} batch {B} {dtype}")


@pytest.mark.parametrize("seed", list(range(8 * MORE)))
def test_decode_random_shapes(seed):
    """Seeded random decode batches (group size, page size, kv heads, layers, batch size, context lengths,
    storage type), every row against the oracle; small batches are cut into key ranges, large ones are not."""
    rng = np.random.default_rng(9500 + seed)
    group = int(rng.choice([1, 2, 4, 8]))
    P = int(rng.choice([8, 16, 32, 64]))
    N = int(rng.integers(1, 5))
    Lyr = int(rng.integers(1, 3))
    layer = int(rng.integers(0, Lyr))
    dtype = torch.bfloat16 if seed % 2 == 0 else torch.float16
    B = int(rng.choice([1, 3, 17, 130]))
    hi = 1200 if B < 20 else 90
    seqlens = [int(v) for v in rng.integers(1, hi, size=B)]
    pages, indptr, last = A.make_cache(9600 + seed, seqlens, Lyr, N, P, 128, dtype)
    g = torch.Generator().manual_seed(9700 + seed)
    q = torch.randn((B, N * group, 128), generator=g).to(dtype)
    pd, ptrs, ind, lst = _to_dev(pages, indptr, last)
    o = _decode(q.to(DEV), ptrs, ind, lst, Lyr, layer, N, P)
    want = A.batch_decode(q, pages, indptr, last, layer, THETA)
    assert_close(o, want, what=f"seed {seed}: group {group} page {P} heads {N} batch {B} {dtype}")
