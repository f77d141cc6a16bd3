"""CPU checks of the attention oracle: the paged evaluation against an independent dense one (contiguous
K/V, rotation written with complex numbers, softmax by hand), and the append bookkeeping."""
import numpy as np
import torch

from oracle import attention_oracle as A


def _dense(q, K, V, theta):
    """q [Nq, D], K/V [L, N, D] float64: rotate pairs (i, i + D/2) as complex numbers."""
    Nq, D = q.shape
    L, N, _ = K.shape
    half = D // 2
    freq = theta ** (-2.0 * np.arange(half) / D)

    def rot(x, pos):
        z = x[..., :half] + 1j * x[..., half:]
        z = z * np.exp(1j * pos[..., None] * freq)
        return np.concatenate([z.real, z.imag], axis=-1)

    qr = rot(q, np.full((Nq,), L - 1.0))
    kr = rot(K, np.arange(L, dtype=np.float64)[:, None].repeat(N, 1))
    out = np.zeros((Nq, D))
    G = Nq // N
    for h in range(Nq):
        s = kr[:, h // G, :] @ qr[h] / np.sqrt(D)
        p = np.exp(s - s.max())
        out[h] = (p / p.sum()) @ V[:, h // G, :]
    return out


def test_paged_decode_equals_dense_attention():
    for seed, seqlens, N, G, P in ((1, [1, 16, 17, 40], 2, 4, 16), (2, [5, 33], 1, 8, 8), (3, [64], 4, 1, 32)):
        D, Lyr = 128, 3
        pages, indptr, last = A.make_cache(seed, seqlens, Lyr, N, P, D, torch.float32)
        g = torch.Generator().manual_seed(seed + 100)
        q = torch.randn((len(seqlens), N * G, D), generator=g)
        for layer in (0, 2):
            o = A.batch_decode(q, pages, indptr, last, layer, 10000.0)
            for b, L in enumerate(seqlens):
                K, V = A.gather_kv(pages, indptr[b], indptr[b + 1], last[b], layer)
                assert K.shape == (L, N, D)
                want = _dense(q[b].double().numpy(), K.numpy(), V.numpy(), 10000.0)
                assert np.allclose(o[b].double().numpy(), want, rtol=1e-5, atol=1e-6)


def test_append_and_init_fill_the_last_positions():
    P, N, D, Lyr = 16, 2, 128, 2
    seqlens = [17, 3, 32]
    pages, indptr, last = A.make_cache(4, seqlens, Lyr, N, P, D, torch.float32)
    before = [p.clone() for p in pages]
    g = torch.Generator().manual_seed(5)
    k, v = torch.randn((3, N, D), generator=g), torch.randn((3, N, D), generator=g)
    A.append_kv(pages, indptr, last, k, v, 1)
    for b, L in enumerate(seqlens):
        K, V = A.gather_kv(pages, indptr[b], indptr[b + 1], last[b], 1)
        assert torch.equal(K[-1].float(), k[b]) and torch.equal(V[-1].float(), v[b])
        K0, _ = A.gather_kv(before, indptr[b], indptr[b + 1], last[b], 1)
        assert torch.equal(K[:-1], K0[:-1])                          # nothing else of the layer moved
    for i in range(len(pages)):
        assert torch.equal(pages[i][0], before[i][0])                # the other layer is untouched
    # a run of tokens per request lands behind what the cache already holds
    runs = [4, 3, 20]
    ind = [0, 4, 7, 27]
    k2, v2 = torch.randn((27, N, D), generator=g), torch.randn((27, N, D), generator=g)
    A.init_kv(pages, indptr, last, k2, v2, ind, 0)
    for b, L in enumerate(seqlens):
        K, V = A.gather_kv(pages, indptr[b], indptr[b + 1], last[b], 0)
        assert torch.equal(K[L - runs[b]:].float(), k2[ind[b]:ind[b + 1]])
        assert torch.equal(V[L - runs[b]:].float(), v2[ind[b]:ind[b + 1]])
        K0, _ = A.gather_kv(before, indptr[b], indptr[b + 1], last[b], 0)
        assert torch.equal(K[:L - runs[b]], K0[:L - runs[b]])
    assert A.last_page_offset_of(16, 16) == 16 and A.last_page_offset_of(17, 16) == 1


def test_paged_prefill_equals_dense_causal_attention_and_decode_of_its_last_row():
    P, N, G, D = 16, 2, 4, 128
    seqlens = [5, 16, 40]          # keys in the cache
    qlens = [5, 9, 40]             # the last qlens[b] positions are the prompt being prefilled
    pages, indptr, last = A.make_cache(7, seqlens, 1, N, P, D, torch.float32)
    g = torch.Generator().manual_seed(8)
    qind = [0] + list(np.cumsum(qlens))
    q = torch.randn((qind[-1], N * G, D), generator=g)
    o = A.batch_prefill(q, qind, pages, indptr, last, 0, 10000.0)
    for b, (L, n) in enumerate(zip(seqlens, qlens)):
        K, V = A.gather_kv(pages, indptr[b], indptr[b + 1], last[b], 0)
        for i in range(n):
            pos = L - n + i
            want = _dense(q[qind[b] + i].double().numpy(), K.numpy()[:pos + 1], V.numpy()[:pos + 1], 10000.0)
            assert np.allclose(o[qind[b] + i].double().numpy(), want, rtol=1e-5, atol=1e-6)
    # the last query of every prompt sees the whole cache: it is a decode step
    last_q = torch.stack([q[qind[b + 1] - 1] for b in range(3)])
    od = A.batch_decode(last_q, pages, indptr, last, 0, 10000.0)
    for b in range(3):
        assert torch.allclose(od[b], o[qind[b + 1] - 1], rtol=1e-5, atol=1e-6)
