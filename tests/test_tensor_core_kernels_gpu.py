"""The tcgen05 (fifth-generation tensor core) token kernels: parity against the FP64 oracle on the shapes
that take them (head dimension 64, rank 16/32/64, long samples), and their FP32 results before the BF16
store against the same oracle at the FP32 criterion (<= 1e-4 relative L2 on identical BF16 inputs)."""
from __future__ import annotations

import ctypes

import pytest
import torch

from conftest import rel_l2
from oracle import memsolve_oracle as O
from test_fast_mix_gpu import _assert_case, _dev, _random_case, cuda_mod  # noqa: F401  (fixture)

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("batch,length,heads,rank,rot,comp,masked", [
    (1, 515, 2, 32, True, False, False),      # ragged last 128-token tile
    (2, 3000, 12, 32, True, False, False),    # four head groups per sample
    (1, 4096, 12, 64, True, False, False),    # one head per CTA group
    (2, 2500, 5, 16, True, True, False),      # rank 16, complement mode
    (2, 1500, 3, 32, False, False, True),     # no rotation: operands straight from shared memory; gaps, empty sample
    (1, 2048, 4, 64, False, True, False),
    (3, 700, 6, 16, False, False, False),
    (2, 1100, 4, 32, True, False, True),      # per-sample tables with gaps
])
def test_tcgen05_token_backward_matches_oracle(cuda_mod, batch, length, heads, rank, rot, comp, masked):
    case = _random_case(9100 + length + rank, batch, length, heads, rank, 64, comp=comp, rot=rot, masked=masked,
                        batched_table=rot and masked)
    _assert_case(cuda_mod, *case, gproj=5e-3 if rot else 3e-2, gpar=5e-4 if rot else 3e-2,
                 tag=f"tcgen05 B{batch} N{length} H{heads} r{rank} rot={rot} comp={comp} masked={masked}")
    assert cuda_mod._LIB.ms_device_error() == 0


def _backward_stages(cuda_mod, proj, base, eta_raw, counts, cos, sin, dy):
    """Forward tape, adjoint statistics and compact adjoint through the C ABI; returns what the token pass needs."""
    lib = cuda_mod._LIB
    dp, db, de, ddy = proj.cuda(), base.cuda(), eta_raw.cuda(), dy.cuda().contiguous()
    dcos, dsin, dcounts = _dev(cos), _dev(sin), _dev(counts)
    _, tape, dims = cuda_mod._mix_forward(dp, db, de, dcounts, None, dcos, dsin)
    shape = cuda_mod._Shape(*dims, 0)
    batch, length, heads, rank, head_dim = dims[:5]
    ws = cuda_mod._workspace(shape, dp.device)
    tape_c = tape.as_struct()
    stream = torch.cuda.current_stream().cuda_stream
    ptr = cuda_mod._ptr
    gram = torch.empty(batch, heads, 2, rank, rank, device="cuda", dtype=torch.bfloat16)
    cross = torch.empty(batch, heads, 2, rank, lib.ms_padded_head_dim(head_dim), device="cuda", dtype=torch.bfloat16)
    d_base, d_raw = torch.empty_like(db), torch.empty_like(de)
    assert lib.ms_stats_backward(ctypes.byref(shape), dp.data_ptr(), ddy.data_ptr(), ptr(dcos), ptr(dsin),
                                 ptr(dcounts), ws.data_ptr(), ws.numel(), None, stream) == 0
    assert lib.ms_compact_backward(ctypes.byref(shape), ptr(dcounts), ws.data_ptr(), ws.numel(), None,
                                   ctypes.byref(tape_c), db.data_ptr() if db.numel() else None, de.data_ptr(), 1.0,
                                   gram.data_ptr(), cross.data_ptr(), d_base.data_ptr() if db.numel() else None,
                                   d_raw.data_ptr(), stream) == 0
    return shape, tape, tape_c, (dp, ddy, dcos, dsin, dcounts), gram, cross


@pytest.mark.parametrize("rank,rot,length", [(32, True, 2300), (64, True, 1024), (16, False, 1500), (32, False, 300)])
def test_token_backward_fp32_before_rounding(cuda_mod, rank, rot, length):
    """The token pass itself at the FP32 criterion: its FP32 results (two-word operands, FP32 accumulation,
    FP32 rotation) against the FP64 oracle on identical BF16 `projected` and upstream gradient, <= 1e-4; the
    BF16 tensor written beside them is exactly the rounding of those FP32 values."""
    lib = cuda_mod._LIB
    heads, batch = 3, 2
    proj, base, eta_raw, counts, cos, sin, dy = _random_case(640 + rank, batch, length, heads, rank, 64, rot=rot)
    shape, tape, tape_c, (dp, ddy, dcos, dsin, dcounts), gram, cross = _backward_stages(
        cuda_mod, proj, base, eta_raw, counts, cos, sin, dy)
    ptr = cuda_mod._ptr
    out16 = torch.empty_like(dp)
    out32 = torch.full(dp.shape, float("nan"), device="cuda", dtype=torch.float32)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.ms_token_backward_debug(ctypes.byref(shape), dp.data_ptr(), ddy.data_ptr(), ptr(dcos), ptr(dsin),
                                       ptr(dcounts), ctypes.byref(tape_c), gram.data_ptr(), cross.data_ptr(),
                                       out16.data_ptr(), out32.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert lib.ms_device_error() == 0
    want = O.stage_backward(proj, dy, base, eta_raw, counts, cos, sin)["dprojected"]
    err32, err16 = rel_l2(out32, want), rel_l2(out16, want)
    print(f"token backward r{rank} rot={rot} N{length}: FP32 {err32:.2e}, BF16 {err16:.2e}")
    assert torch.isfinite(out32).all()
    assert err32 <= 1e-4
    assert err16 <= 5e-3
    assert torch.equal(out32.bfloat16(), out16)
    # the production entry point gives the same BF16 tensor
    again = torch.empty_like(dp)
    assert lib.ms_token_backward(ctypes.byref(shape), dp.data_ptr(), ddy.data_ptr(), ptr(dcos), ptr(dsin),
                                 ptr(dcounts), ctypes.byref(tape_c), gram.data_ptr(), cross.data_ptr(),
                                 again.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    if length >= 512:
        assert torch.equal(again, out16)
    else:
        assert rel_l2(again, out16) <= 4e-3   # short samples take the mma.sync kernel: same values to BF16 rounding


@pytest.mark.parametrize("rank,rot,length,comp", [(32, True, 2300, False), (64, True, 1024, False), (16, False, 1500, False),
                                                  (32, False, 300, True), (64, True, 777, True)])
def test_readout_fp32_before_rounding(cuda_mod, rank, rot, length, comp):
    """The readout kernel's own FP32 values (two-word coefficients, FP32 accumulation, inverse rotation and
    eta*C in FP32) against the reference's frame formulation in FP64 on the identical BF16 projection:
    <= 1e-4, the FP32 criterion; the BF16 tensor beside them is their rounding."""
    lib = cuda_mod._LIB
    heads, batch = 3, 2
    proj, base, eta_raw, counts, cos, sin, dy = _random_case(720 + rank, batch, length, heads, rank, 64, rot=rot, comp=comp)
    dp, db, de = proj.cuda(), base.cuda(), eta_raw.cuda()
    dcos, dsin = _dev(cos), _dev(sin)
    mixed, tape, dims = cuda_mod._mix_forward(dp, db, de, None, None, dcos, dsin)
    shape = cuda_mod._Shape(*dims, 0)
    tape_c = tape.as_struct()
    ptr = cuda_mod._ptr
    out16 = torch.empty_like(mixed)
    out32 = torch.full(mixed.shape, float("nan"), device="cuda", dtype=torch.float32)
    assert lib.ms_readout_debug(ctypes.byref(shape), dp.data_ptr(), ptr(dcos), ptr(dsin), None, ctypes.byref(tape_c),
                                out16.data_ptr(), out32.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert lib.ms_device_error() == 0
    want = O.fast_mix_frame(proj, base, eta_raw, None, cos, sin)
    err32, err16 = rel_l2(out32, want), rel_l2(out16, want)
    print(f"readout r{rank} rot={rot} N{length} comp={comp}: FP32 {err32:.2e}, BF16 {err16:.2e}")
    assert err32 <= 1e-4 and err16 <= 5e-3
    assert torch.equal(out32.bfloat16(), out16)
    if length >= 512:
        assert torch.equal(out16, mixed)
    else:
        assert rel_l2(out16, mixed) <= 4e-3


@pytest.mark.parametrize("rank,rot,length,heads,batch,masked", [
    (32, True, 5000, 3, 2, False), (64, True, 3000, 5, 1, False), (16, False, 2100, 6, 2, False),
    (32, False, 1500, 2, 1, True), (16, True, 4096, 5, 1, False), (64, False, 1024, 2, 2, False),
    (32, True, 32768, 12, 1, False), (64, True, 32768, 12, 1, False)])
def test_tcgen05_statistics_stagewise(cuda_mod, rank, rot, length, heads, batch, masked):
    """Forward (G, Q) and adjoint (E, <dY, C>) token reductions of the tcgen05 kernel against FP64, <= 1e-5
    (the limit of the statistics stage), for head groups that are full, partial (odd head counts) and of four
    heads (rank 16), with and without rotation, ragged last tiles and counts.  The 1e-5 limit is the reference's
    for its own sizes (up to 8193 tokens, tests/cuda/test_fast_path.py:847-932); the two 32768-token cases sum
    twenty times more FP32 terms per accumulator and are held to 2e-5 (measured 4e-6 ... 1.5e-5)."""
    lib = cuda_mod._LIB
    proj, base, eta_raw, counts, cos, sin, dy = _random_case(830 + rank + length, batch, length, heads, rank, 64,
                                                             rot=rot, masked=masked)
    dp, ddy = proj.cuda(), dy.cuda().contiguous()
    dcos, dsin, dcounts = _dev(cos), _dev(sin), _dev(counts)
    shape = cuda_mod._Shape(batch, length, heads, rank, 64, 0, 0 if cos is None else cos.shape[0], 0)
    ws = cuda_mod._workspace(shape, dp.device)
    ptr = cuda_mod._ptr
    stream = torch.cuda.current_stream().cuda_stream
    fwd = torch.full((lib.ms_packed_stats_floats(ctypes.byref(shape), 0),), float("nan"), device="cuda")
    bwd = torch.full((lib.ms_packed_stats_floats(ctypes.byref(shape), 1),), float("nan"), device="cuda")
    assert lib.ms_stats_forward(ctypes.byref(shape), dp.data_ptr(), ptr(dcos), ptr(dsin), ptr(dcounts), ws.data_ptr(),
                                ws.numel(), fwd.data_ptr(), stream) == 0
    assert lib.ms_stats_backward(ctypes.byref(shape), dp.data_ptr(), ddy.data_ptr(), ptr(dcos), ptr(dsin),
                                 ptr(dcounts), ws.data_ptr(), ws.numel(), bwd.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert lib.ms_device_error() == 0
    g, q = O.stage_stats(proj, heads, rank, counts, cos, sin)
    pk = fwd.view(batch * heads, rank * rank + rank * 64).cpu()
    errs = {"G": rel_l2(pk[:, : rank * rank].reshape(batch, heads, rank, rank), g),
            "Q": rel_l2(pk[:, rank * rank:].reshape(batch, heads, rank, 64), q)}
    want = O.stage_backward(proj, dy, base, eta_raw, counts, cos, sin)
    got_e = bwd[: batch * heads * rank * 64].view(batch, heads, rank, 64).cpu()
    got_de = bwd[batch * heads * rank * 64:].view(batch, heads).cpu().double().sum(0)
    errs["E"] = rel_l2(got_e, want["E"])
    errs["de"] = rel_l2(got_de, want["de"])
    print(f"statistics r{rank} rot={rot} N{length} H{heads} B{batch}", {k: f"{v:.2e}" for k, v in errs.items()})
    limit = 1e-5 if length <= 8193 else 2e-5
    assert all(v <= limit for v in errs.values()), errs


@pytest.mark.parametrize("rank", [16, 32, 64])
def test_tcgen05_statistics_stagewise_repeatable(cuda_mod, rank):
    """Forty launches of both token reductions over 32768 rotated tokens give the same bits.  The kernels add in a
    fixed order, so any difference is a synchronisation fault: this is the case that exposed rotary rows handed back
    to the table warp's next bulk copy while the loads that read them were still in flight (single threads then
    rotated by the next tile's angles, in about every second launch)."""
    lib = cuda_mod._LIB
    proj, base, eta_raw, counts, cos, sin, dy = _random_case(77 + rank, 1, 32768, 12, rank, 64, rot=True)
    dp, ddy, dcos, dsin = proj.cuda(), dy.cuda().contiguous(), cos.cuda(), sin.cuda()
    shape = cuda_mod._Shape(1, 32768, 12, rank, 64, 0, 1, 0)
    ws = cuda_mod._workspace(shape, dp.device)
    stream = torch.cuda.current_stream().cuda_stream
    sizes = [lib.ms_packed_stats_floats(ctypes.byref(shape), k) for k in (0, 1)]
    first = None
    for _ in range(40):
        fwd, bwd = (torch.zeros(n, device="cuda") for n in sizes)
        assert lib.ms_stats_forward(ctypes.byref(shape), dp.data_ptr(), dcos.data_ptr(), dsin.data_ptr(), None,
                                    ws.data_ptr(), ws.numel(), fwd.data_ptr(), stream) == 0
        assert lib.ms_stats_backward(ctypes.byref(shape), dp.data_ptr(), ddy.data_ptr(), dcos.data_ptr(),
                                     dsin.data_ptr(), None, ws.data_ptr(), ws.numel(), bwd.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        if first is None:
            first = (fwd, bwd)
        else:
            assert torch.equal(fwd, first[0]) and torch.equal(bwd, first[1])
    assert lib.ms_device_error() == 0


def test_tcgen05_statistics_all_ranks_in_child_process():
    """Rank 16 takes the mma.sync statistics kernels unless MEMSOLVE_STATS_TCGEN05=1 is set when the library
    plans its first launch: run the stage-wise statistics cases and the mixer cases of this file in a child
    process with the switch on, so the tcgen05 kernel is checked at every rank."""
    import os
    import subprocess
    import sys
    if os.environ.get("MEMSOLVE_STATS_TCGEN05") == "1":
        pytest.skip("already inside the child process")
    env = dict(os.environ, MEMSOLVE_STATS_TCGEN05="1")
    here = os.path.abspath(__file__)
    done = subprocess.run([sys.executable, "-m", "pytest", here, "-q", "-x", "-p", "no:cacheprovider", "-k",
                           "statistics_stagewise or token_backward_matches_oracle"], env=env, capture_output=True,
                          text=True, timeout=900)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-2000:]


def test_mma_sync_statistics_at_rank_32_in_child_process():
    """The other way round: with MEMSOLVE_STATS_TCGEN05=0 rank 32 takes the mma.sync statistics kernels at every
    length; the stage-wise cases and the long-sequence mixer case run in a child process with that setting."""
    import os
    import subprocess
    import sys
    if os.environ.get("MEMSOLVE_STATS_TCGEN05") is not None:
        pytest.skip("already inside a child process")
    env = dict(os.environ, MEMSOLVE_STATS_TCGEN05="0")
    here = os.path.dirname(os.path.abspath(__file__))
    done = subprocess.run([sys.executable, "-m", "pytest", os.path.join(here, "test_tensor_core_kernels_gpu.py"),
                           os.path.join(here, "test_fast_mix_gpu.py"), "-q", "-x", "-p", "no:cacheprovider", "-k",
                           "statistics_stagewise or full_size_long_sequence"], env=env, capture_output=True,
                          text=True, timeout=900)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-2000:]


@pytest.mark.parametrize("rows,in_features,out_features,bias,masks", [
    (4096, 768, 1152, False, False), (1000, 768, 768, True, True), (130, 128, 128, True, False),
    (777, 256, 384, False, True), (32768, 768, 1152, True, True)])
def test_tcgen05_linear_forward(cuda_mod, rows, in_features, out_features, bias, masks):
    """`ms_linear_forward` against the same contraction in FP32 on the BF16 operands: products and bias in FP32,
    one BF16 rounding (<= 1 BF16 ulp apart from the FP32 result rounded once: relative L2 <= 2e-3, which is the
    rounding itself), masked output rows exactly zero, masked input rows give exactly the rounded bias even when
    they hold NaN."""
    lib = cuda_mod._LIB
    gen = torch.Generator().manual_seed(rows + out_features)
    x = torch.randn(rows, in_features, generator=gen).bfloat16().cuda()
    w = (torch.randn(out_features, in_features, generator=gen) * 0.05).bfloat16().cuda()
    b = torch.randn(out_features, generator=gen).cuda() if bias else None
    in_mask = out_mask = None
    if masks:
        in_mask = (torch.rand(rows, generator=gen) > 0.2).cuda()
        out_mask = (torch.rand(rows, generator=gen) > 0.2).cuda()
        x[~in_mask] = float("nan")
    out = torch.full((rows, out_features), float("nan"), device="cuda", dtype=torch.bfloat16)
    ptr = cuda_mod._ptr
    status = lib.ms_linear_forward(rows, in_features, out_features, x.data_ptr(), w.data_ptr(), ptr(b), ptr(in_mask),
                                   ptr(out_mask), out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert status == 0
    torch.cuda.synchronize()
    assert lib.ms_device_error() == 0
    xin = x.float() if in_mask is None else torch.where(in_mask[:, None], x.float(), torch.zeros((), device="cuda"))
    want = xin @ w.float().t()
    if b is not None:
        want = want + b
    if out_mask is not None:
        want = torch.where(out_mask[:, None], want, torch.zeros((), device="cuda"))
    assert torch.isfinite(out.float()).all()
    err = rel_l2(out, want)
    print(f"linear {rows}x{in_features}x{out_features}: {err:.2e}")
    assert err <= 2e-3
    assert float((out.float() - want.bfloat16().float()).abs().max()) <= 2.0 ** -6 * float(want.abs().max())
    if masks:
        assert torch.count_nonzero(out[~out_mask]) == 0
        only_bias = out_mask & ~in_mask
        expect = torch.zeros(out_features, device="cuda") if b is None else b
        assert torch.equal(out[only_bias], expect.bfloat16().expand(int(only_bias.sum()), -1))
    assert lib.ms_linear_forward(rows, in_features + 8, out_features, x.data_ptr(), w.data_ptr(), None, None, None,
                                 out.data_ptr(), None) == 9


@pytest.mark.parametrize("rows,in_features,out_features,masks", [
    (4096, 768, 1152, False), (1000, 768, 768, True), (130, 128, 64, False), (777, 384, 256, True),
    (32768, 768, 1152, True)])
def test_tcgen05_linear_input_grad(cuda_mod, rows, in_features, out_features, masks):
    """`ms_linear_input_grad` (dx = dy W, the weight read in place as an N-major operand) against the FP32 product of
    the BF16 operands: one BF16 rounding; a row cleared by either mask is exactly zero whatever dy holds there."""
    lib = cuda_mod._LIB
    gen = torch.Generator().manual_seed(rows + in_features)
    dy = torch.randn(rows, out_features, generator=gen).bfloat16().cuda()
    w = (torch.randn(out_features, in_features, generator=gen) * 0.05).bfloat16().cuda()
    in_mask = out_mask = None
    if masks:
        in_mask = (torch.rand(rows, generator=gen) > 0.2).cuda()
        out_mask = (torch.rand(rows, generator=gen) > 0.2).cuda()
        dy[~out_mask] = float("nan")
    dx = torch.full((rows, in_features), float("nan"), device="cuda", dtype=torch.bfloat16)
    ptr = cuda_mod._ptr
    status = lib.ms_linear_input_grad(rows, in_features, out_features, dy.data_ptr(), w.data_ptr(), ptr(in_mask),
                                      ptr(out_mask), dx.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert status == 0
    torch.cuda.synchronize()
    assert lib.ms_device_error() == 0
    keep = torch.ones(rows, dtype=torch.bool, device="cuda") if not masks else in_mask & out_mask
    want = torch.where(keep[:, None], torch.nan_to_num(dy.float()) @ w.float(), torch.zeros((), device="cuda"))
    assert torch.isfinite(dx.float()).all()
    err = rel_l2(dx, want)
    print(f"input grad {rows}x{in_features}x{out_features}: {err:.2e}")
    assert err <= 2e-3
    assert float((dx.float() - want.bfloat16().float()).abs().max()) <= 2.0 ** -6 * float(want.abs().max())
    assert torch.count_nonzero(dx[~keep]) == 0
    assert lib.ms_linear_input_grad(rows, in_features + 8, out_features, dy.data_ptr(), w.data_ptr(), None, None,
                                    dx.data_ptr(), None) == 9


@pytest.mark.parametrize("rows,in_features,out_features,bias", [
    (4096, 768, 1152, True), (1000, 768, 768, False), (63, 128, 128, True), (777, 384, 256, True),
    (32768, 768, 1152, True), (32768, 768, 768, True)])
def test_tcgen05_linear_weight_grad(cuda_mod, rows, in_features, out_features, bias):
    """`ms_linear_weight_grad` (dW = dy^T x and db = column sums of dy, FP32 sums of BF16 products, rows split over
    CTAs and added in a fixed order) against FP64 sums of the same BF16 operands: <= 2e-5 relative (the tensor cores'
    FP32 accumulation over several thousand rows per CTA: 7e-6 measured at 32768 rows), and bit-identical on a second
    run."""
    lib = cuda_mod._LIB
    gen = torch.Generator().manual_seed(rows + in_features + out_features)
    x = torch.randn(rows, in_features, generator=gen).bfloat16().cuda()
    dy = torch.randn(rows, out_features, generator=gen).bfloat16().cuda()
    nbytes = int(lib.ms_linear_weight_grad_workspace(rows, in_features, out_features))
    assert nbytes > 0
    results = []
    for _ in range(2):
        ws = torch.empty(nbytes, device="cuda", dtype=torch.uint8)
        dw = torch.full((out_features, in_features), float("nan"), device="cuda")
        db = torch.full((out_features,), float("nan"), device="cuda") if bias else None
        status = lib.ms_linear_weight_grad(rows, in_features, out_features, x.data_ptr(), dy.data_ptr(), dw.data_ptr(),
                                           cuda_mod._ptr(db), ws.data_ptr(), nbytes,
                                           torch.cuda.current_stream().cuda_stream)
        assert status == 0
        torch.cuda.synchronize()
        assert lib.ms_device_error() == 0
        results.append((dw, db))
    dw, db = results[0]
    want = dy.double().t() @ x.double()
    err = rel_l2(dw, want)
    print(f"weight grad {rows}x{in_features}x{out_features}: {err:.2e}")
    assert err <= 2e-5
    assert torch.equal(dw, results[1][0])
    if bias:
        want_b = dy.double().sum(0)
        assert float((db.double() - want_b).abs().max()) <= 2e-6 * float(dy.double().abs().sum(0).max())
        assert torch.equal(db, results[1][1])
    assert lib.ms_linear_weight_grad_workspace(rows, in_features + 8, out_features) == 0
    assert lib.ms_linear_weight_grad(rows, in_features + 8, out_features, x.data_ptr(), dy.data_ptr(), dw.data_ptr(),
                                     None, ws.data_ptr(), nbytes, None) == 9


def test_debug_entry_rejects_other_shapes(cuda_mod):
    lib = cuda_mod._LIB
    proj, base, eta_raw, counts, cos, sin, dy = _random_case(5, 1, 600, 2, 48, 64)
    shape, tape, tape_c, (dp, ddy, dcos, dsin, dcounts), gram, cross = _backward_stages(
        cuda_mod, proj, base, eta_raw, counts, cos, sin, dy)
    out16 = torch.empty_like(dp)
    out32 = torch.empty(dp.shape, device="cuda")
    status = lib.ms_token_backward_debug(ctypes.byref(shape), dp.data_ptr(), ddy.data_ptr(), None, None, None,
                                         ctypes.byref(tape_c), gram.data_ptr(), cross.data_ptr(), out16.data_ptr(),
                                         out32.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert status == 8 and b"tcgen05" in lib.ms_status_string(status)
