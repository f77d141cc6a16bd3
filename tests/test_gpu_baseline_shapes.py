"""Parity at the sizes of the benchmark configurations: forward and backward of
the mixed Llama-2-7B q_proj batch, the decode sweep, one Llama-3-8B projection and
one fine-tune-heavy partition, each against the CPU oracle on the same seeded
inputs, plus size-independent properties (linearity in x, segment independence)."""
import numpy as np
import pytest
import torch

from helpers import assert_close
from oracle import smlm_oracle as O

pytestmark = pytest.mark.gpu


def _case(seed, lens, n_ad, h_in, h_out, rank, dtype, ids=None):
    rng = np.random.default_rng(seed)
    ids = list(rng.integers(0, n_ad, size=len(lens))) if ids is None else ids
    return O.make_case(seed, lens, [int(i) for i in ids], n_ad, h_in, h_out, rank, dtype)


def test_c2_llama2_qproj_mixed_batch_fwd_bwd():
    from gpu_util import check_forward
    from test_gpu_parity import _grad_close, _oracle_bwd, _run_bwd
    lens = [1024, 1024] + [512] * 4 + [1] * 64
    c = _case(2000, lens, 32, 4096, 4096, 16, torch.float16)
    check_forward(c)
    # backward over the two fine-tune segments
    part = [0, 1024, 2048]
    cb = dict(c)
    cb["wa"] = [c["wa"][c["ids"][0]], c["wa"][c["ids"][1]]]
    cb["wb"] = [c["wb"][c["ids"][0]], c["wb"][c["ids"][1]]]
    dx, dA, dB = _run_bwd(cb, part)
    gx, gA, gB = _oracle_bwd(cb, part)
    _grad_close(dx[:2048], gx[:2048], "dX")
    for p in range(2):
        _grad_close(dA[p], gA[p], f"dA{p}")
        _grad_close(dB[p], gB[p], f"dB{p}")


@pytest.mark.parametrize("h_in,h_out", [(4096, 11008), (11008, 4096)])
def test_c4_decode_sweep(h_in, h_out):
    from gpu_util import check_forward
    c = _case(4000, [1] * 1024, 256, h_in, h_out, 32, torch.bfloat16)
    check_forward(c, indexed=True)


def test_c3_llama3_down_proj_zipf_segments():
    from gpu_util import check_forward
    rng = np.random.default_rng(3000)
    lens, tot = [], 0
    while tot < 8192:
        n = int(min(2048, max(1, rng.zipf(1.2))))
        n = min(n, 8192 - tot)
        lens.append(n)
        tot += n
    c = _case(3000, lens, 128, 14336, 4096, 16, torch.bfloat16)
    check_forward(c, indexed=True, scale=[2.0] * 128)


def test_c5_finetune_partition_rank64():
    from test_gpu_parity import _grad_close, _oracle_bwd, _run_bwd
    c = _case(5000, [4096], 2, 4096, 14336, 64, torch.bfloat16, ids=[0])
    part = [0, 2048, 4096]
    dx, dA, dB = _run_bwd(c, part)
    gx, gA, gB = _oracle_bwd(c, part)
    _grad_close(dx, gx, "dX")
    for p in range(2):
        _grad_close(dA[p], gA[p], f"dA{p}")
        _grad_close(dB[p], gB[p], f"dB{p}")


def test_linearity_and_segment_independence():
    """y(2x) == 2 y(x) bit-exactly (scaling by two is exact in binary floating
    point), and a segment's rows do not depend on what other segments hold."""
    from gpu_util import run_forward
    c = _case(77, [300, 1, 1, 700, 64, 5], 8, 2048, 1536, 16, torch.bfloat16)
    y1, v1 = run_forward(c)
    c2 = dict(c)
    c2["x"] = (c["x"].float() * 2).to(torch.bfloat16)
    y2, v2 = run_forward(c2)
    assert torch.equal((y1.float() * 2).to(torch.bfloat16), y2)
    c3 = dict(c)
    x3 = c["x"].clone()
    x3[301:] = 0
    c3["x"] = x3
    y3, _ = run_forward(c3)
    assert torch.equal(y3[:301], y1[:301])
    assert (y3[301:] == 0).all()
