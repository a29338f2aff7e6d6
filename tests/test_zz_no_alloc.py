"""`ms_stats_forward_static`: the statistics entry point for callers that cannot allocate.

Some users of the library sit where device allocation is not available to them: a plugin inside
an application that owns the allocator and passes only input/output buffers, or a latency-bound
loop where cudaMalloc's implicit synchronisation is unacceptable.  For them the library carries
its own scratch (a fixed 16 MiB buffer in the library image) and this entry point uses it instead
of a caller workspace.  The test drives it through the C ABI, twice in a row with different
inputs (the buffer is shared between calls and keeps old contents), and requires the same packed
statistics as the workspace-taking entry point; it also checks that an over-sized shape is refused
with the dedicated status instead of launching.

The file name makes pytest collect it last, so a run that stops at the first failure has already
executed every other test.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

from conftest import rel_l2
from oracle import memsolve_oracle as O

pytestmark = pytest.mark.gpu

MS_ERR_STATIC_SCRATCH = 7


def _inputs(seed, batch, tokens, heads, rank, head_dim):
    gen = torch.Generator().manual_seed(seed)
    proj = torch.randn(batch, tokens, heads * (rank + head_dim), generator=gen).bfloat16().cuda()
    pos = torch.arange(tokens)[None].float()
    freq = 10000.0 ** (-torch.arange(0, head_dim, 2).float() / head_dim)
    ang = pos[..., None] * freq
    return proj, ang.cos().contiguous().cuda(), ang.sin().contiguous().cuda()


def test_static_scratch_entry_matches_workspace_entry():
    from memsolve_b200.ball import cuda
    cuda.load()
    lib = cuda._LIB
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row; the second has a different shape so stale partials of the first call
    # sit in the shared buffer beyond and between the new ones
    for seed, (batch, tokens, heads, rank, head_dim) in enumerate([(2, 5000, 4, 32, 64), (1, 3001, 3, 16, 24)]):
        proj, cos, sin = _inputs(seed, batch, tokens, heads, rank, head_dim)
        shape = cuda._Shape(batch, tokens, heads, rank, head_dim, 0, 1, 0)
        floats = lib.ms_packed_stats_floats(ctypes.byref(shape), 0)
        want = torch.empty(floats, device="cuda")
        got = torch.full((floats,), float("nan"), device="cuda")
        ws = torch.empty(lib.ms_workspace_bytes(ctypes.byref(shape)), dtype=torch.uint8, device="cuda")
        assert lib.ms_stats_forward(ctypes.byref(shape), proj.data_ptr(), cos.data_ptr(), sin.data_ptr(), None,
                                    ws.data_ptr(), ws.numel(), want.data_ptr(), stream) == 0
        assert lib.ms_stats_forward_static(ctypes.byref(shape), proj.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                           None, got.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        # same kernels and summation order: the tolerance of the statistics tests (1e-5 relative
        # L2) is met with room to spare, in fact bit for bit
        err = float((got.double() - want.double()).norm() / want.double().norm())
        assert err <= 1e-5
        assert torch.equal(got, want)
        # and against the FP64 oracle, at the limit of the statistics tests
        g64, q64 = O.stage_stats(proj.cpu(), heads, rank, None, cos.cpu(), sin.cpu())
        pk = got.view(batch * heads, rank * rank + rank * head_dim).cpu()
        assert rel_l2(pk[:, : rank * rank].reshape(batch, heads, rank, rank), g64) <= 1e-5
        assert rel_l2(pk[:, rank * rank:].reshape(batch, heads, rank, head_dim), q64) <= 1e-5
        # "allocates nothing": the device's free memory is the same before and after another call
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        assert lib.ms_stats_forward_static(ctypes.byref(shape), proj.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                           None, got.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.equal(got, want)


def test_static_scratch_entry_rejects_oversized_shapes():
    from memsolve_b200.ball import cuda
    cuda.load()
    lib = cuda._LIB
    # 64 samples x 16 heads of rank 64, head dimension 512: the partial sums alone exceed 16 MiB
    shape = cuda._Shape(64, 4096, 16, 64, 512, 0, 0, 0)
    dummy = torch.zeros(16, device="cuda")
    status = lib.ms_stats_forward_static(ctypes.byref(shape), dummy.data_ptr(), None, None, None, dummy.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream)
    assert status == MS_ERR_STATIC_SCRATCH
    assert b"static" in lib.ms_status_string(status)
    assert lib.ms_stats_forward_static(ctypes.byref(shape), dummy.data_ptr(), None, None, None, None, None) == 1
