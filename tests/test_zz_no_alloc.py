"""The weight-gradient entry point that brings its own scratch.

Some users of the library cannot give it device memory: a serving loop that split up
the whole GPU at start-up and keeps the allocator off the request path, a plugin that
is handed tensors by its host and has no allocator of its own.  For them
``smlm_b200_wgrad_static`` keeps the kernel's workspace in a fixed 16 MiB array inside
the library.  These tests call it through the C ABI, twice in a row and on different
problems (the array is shared and keeps what the previous call left in it), and compare
with ``smlm_b200_wgrad``, which takes the workspace from the caller.

This file sorts last on purpose: a run that stops at the first failure has then
already been through every other test."""
import ctypes

import numpy as np
import pytest
import torch



def _problem(seed, part, h, rank, dtype, dev):
    g = torch.Generator().manual_seed(seed)
    T = part[-1] + 3
    p = (torch.randn((T, rank), generator=g) * 0.5).to(dtype).to(dev)
    q = torch.randn((T, h), generator=g).to(dtype).to(dev)
    return p, q, torch.tensor(part, dtype=torch.int32, device=dev)


def _run_both(seed, part, h, rank, dtype, transposed, grad_fp32):
    from loquetier_b200 import cabi, ops
    dev = torch.device("cuda:0")
    p, q, pd = _problem(seed, part, h, rank, dtype, dev)
    npart = len(part) - 1
    plan = ops.Plan(pd, part[-1])
    shape = (h, rank) if transposed else (rank, h)
    gdt = torch.float32 if grad_fp32 else dtype
    scale = torch.tensor(np.linspace(0.5, 2.0, npart), dtype=torch.float32, device=dev)

    def outputs():
        gs = [torch.full(shape, 9.0, dtype=gdt, device=dev) for _ in range(npart)]
        return gs, torch.tensor([t.data_ptr() for t in gs], dtype=torch.int64, device=dev)

    want, want_t = outputs()
    ops.wgrad(want_t, p, q, pd, plan, transposed=transposed, part_scale=scale, grad_fp32=grad_fp32)
    got, got_t = outputs()
    stream = torch.cuda.current_stream().cuda_stream
    rc = cabi.lib.smlm_b200_wgrad_static(got_t.data_ptr(), p.data_ptr(), q.data_ptr(), pd.data_ptr(),
                                         scale.data_ptr(), plan.buf.data_ptr(), npart, part[-1], rank, h,
                                         cabi.SMLM_BF16 if dtype == torch.bfloat16 else cabi.SMLM_F16,
                                         int(transposed), 0, int(grad_fp32), stream)
    assert rc == 0, cabi.lib.smlm_b200_status_string(rc)
    torch.cuda.synchronize()
    plan.raise_if_failed()
    for i, (g_, w_) in enumerate(zip(got, want)):
        # the same kernel adds the same partial sums in the same order whichever workspace it is given
        assert torch.equal(g_, w_), f"partition {i}: built-in scratch and caller workspace disagree"
        assert not (g_ == 9.0).all() or part[i + 1] == part[i]


@pytest.mark.gpu
def test_static_scratch_matches_caller_workspace_two_calls_in_a_row():
    # a long partition that is spread over several CTAs (parked partial sums and tickets
    # are really used), short ones, and an empty one
    _run_both(11, [0, 700, 700, 733, 1500], 1024, 16, torch.bfloat16, transposed=True, grad_fp32=False)
    # straight after it, a different problem on the same shared array
    _run_both(12, [0, 5, 1300], 1536, 32, torch.float16, transposed=False, grad_fp32=True)
    # rank 64 runs the tcgen05 variant of the kernel, with its own cut of the shared array
    _run_both(13, [0, 400, 400, 690], 1024, 64, torch.bfloat16, transposed=True, grad_fp32=False)
    # and the first one again: leftovers of the other calls must not matter
    _run_both(11, [0, 700, 700, 733, 1500], 1024, 16, torch.bfloat16, transposed=True, grad_fp32=False)


def test_static_scratch_refuses_problems_beyond_its_size():
    """Checked on the host before any CUDA call, so it needs no GPU."""
    from loquetier_b200 import cabi
    L = cabi.lib
    need = L.smlm_b200_wgrad_workspace_bytes(32768, 16, 64, 14336, 0)
    assert need > (16 << 20)
    rc = L.smlm_b200_wgrad_static(16, 16, 16, 16, None, 16, 16, 32768, 64, 14336, cabi.SMLM_BF16, 0, 0, 0, None)
    assert rc == 11
    assert b"16 MiB" in L.smlm_b200_status_string(rc)
