"""GPU parity of the mixer kernels (called through the C-ABI library) against the CPU oracle
and the committed golden vectors.  Metric: relative L2, as in the reference's own CUDA tests
(tests/cuda/test_fast_path.py:85-99); limits follow those tests (forward 5e-3, gradients 3e-2,
rotary dprojected 5e-3) and are written at each assertion."""
from __future__ import annotations

import ctypes

import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import memsolve_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda_mod():
    from memsolve_b200.ball import cuda
    cuda.load()
    assert cuda.is_available()
    return cuda


def _dev(t):
    return None if t is None else t.cuda()


def _run_fast(cuda_mod, proj, base, eta_raw, counts, cos, sin, dy):
    ins = [proj.cuda().requires_grad_(), base.cuda().requires_grad_(), eta_raw.cuda().requires_grad_()]
    y = cuda_mod.fast_mix(ins[0], ins[1], ins[2], _dev(counts), rotary_cos=_dev(cos), rotary_sin=_dev(sin))
    grads = torch.autograd.grad((y.float() * dy.cuda().float()).sum(), ins, allow_unused=True)
    torch.cuda.synchronize()
    return y, grads


def _run_oracle(proj, base, eta_raw, counts, cos, sin, dy):
    ins = [proj.double().requires_grad_(), base.double().requires_grad_(), eta_raw.double().requires_grad_()]
    y = O.fast_mix_frame(ins[0], ins[1], ins[2], counts, cos, sin)
    wanted = [ins[0], ins[2]] if base.numel() == 0 else ins
    g = torch.autograd.grad((y * dy.double()).sum(), wanted)
    gp, ge = g[0], g[-1]
    gb = g[1] if base.numel() else torch.zeros_like(base, dtype=torch.float64)
    return y, (gp, gb, ge)


def _assert_case(cuda_mod, proj, base, eta_raw, counts, cos, sin, dy, *, fwd=5e-3, gproj=3e-2, gpar=3e-2,
                 expected=None, tag=""):
    y, grads = _run_fast(cuda_mod, proj, base, eta_raw, counts, cos, sin, dy)
    ey, eg = expected if expected is not None else _run_oracle(proj, base, eta_raw, counts, cos, sin, dy)
    assert y.dtype == torch.bfloat16 and torch.isfinite(y.float()).all()
    errs = {"y": rel_l2(y, ey), "dproj": rel_l2(grads[0], eg[0]), "deta": rel_l2(grads[2], eg[2])}
    if base.numel():
        errs["dbase"] = rel_l2(grads[1], eg[1])
    print(tag, {k: f"{v:.2e}" for k, v in errs.items()})
    assert errs["y"] <= fwd, errs
    assert errs["dproj"] <= gproj, errs
    assert errs["deta"] <= gpar, errs
    if base.numel():
        assert errs["dbase"] <= gpar, errs
    return errs


GOLDEN = ["mix_r16_plain", "mix_r32_rot", "mix_r16_comp_rot_mask", "mix_r48_strong", "mix_r64_rot_mask",
          "mix_r16_short"]


@pytest.mark.parametrize("name", GOLDEN)
def test_golden_vectors(cuda_mod, name):
    g = load_golden(name + ".npz")
    expected = (g["y"], (g["d_projected"], g["d_base"], g["d_eta_raw"]))
    _assert_case(cuda_mod, g["projected"].bfloat16(), g["base"], g["eta_raw"], g.get("counts"), g.get("cos"),
                 g.get("sin"), g["dy"].bfloat16(), expected=expected, tag=name)


def _random_case(seed, b, n, h, r, d, *, comp=False, rot=False, masked=False, base_scale=0.1, rel_scale=1.0,
                 batched_table=False):
    gen = torch.Generator().manual_seed(seed)
    proj = torch.randn(b, n, h * r + h * d, generator=gen)
    proj[..., : h * r] *= rel_scale
    counts = None
    if masked:
        mask = torch.rand(b, n, generator=gen) > 0.3
        mask[-1] = False if b > 1 else mask[-1]
        proj = torch.where(mask[:, :, None], proj, torch.zeros_like(proj))
        counts = mask.sum(-1).float().clamp_min(1.0)
    proj = proj.bfloat16()
    base = torch.randn(h, r, 0 if comp else r, generator=gen) * base_scale
    eta_raw = torch.randn(h, generator=gen) * 0.5
    dy = torch.randn(b, n, h * d, generator=gen).bfloat16()
    if masked:
        dy = torch.where(mask[:, :, None], dy, torch.zeros_like(dy))
    cos = sin = None
    if rot:
        if batched_table:
            pos = torch.stack([torch.arange(n) + 3 * i for i in range(b)])
        else:
            pos = torch.arange(n)[None]
        cos, sin = O.rotary_tables(pos, head_dim=d, train_length=16, context_length=n)
    return proj, base, eta_raw, counts, cos, sin, dy


@pytest.mark.parametrize("length", (31, 33, 64, 65, 127, 128, 129, 257, 513))
def test_lengths_around_tile_edges(cuda_mod, length):
    """Shapes of tests/cuda/test_fast_path.py:692-743 (B=1, H=2, D=32, r=16)."""
    case = _random_case(19 + length, 1, length, 2, 16, 16)
    _assert_case(cuda_mod, *case, tag=f"N={length}")


@pytest.mark.parametrize(
    ("batch", "rank", "heads", "head_dim", "length"),
    [(1, 16, 1, 1, 31), (1, 16, 1, 17, 31), (1, 16, 1, 33, 33), (1, 16, 1, 257, 33), (1, 32, 2, 48, 31),
     (2, 32, 3, 17, 35), (1, 48, 2, 96, 33), (1, 64, 1, 33, 33), (1, 64, 1, 17, 2017), (1, 32, 8, 32, 4096),
     (1, 16, 4, 32, 4776), (1, 32, 1, 17, 8193), (3, 32, 2, 64, 197), (2, 64, 2, 64, 300)],
)
def test_generic_shapes(cuda_mod, batch, rank, heads, head_dim, length):
    """Head dims off the 8/16/64 grids, all ranks, multi-chunk lengths
    (tests/cuda/test_fast_path.py:847-932)."""
    case = _random_case(71 + batch + rank + head_dim, batch, length, heads, rank, head_dim, base_scale=0.05)
    _assert_case(cuda_mod, *case, tag=f"B{batch} r{rank} H{heads} d{head_dim} N{length}")


@pytest.mark.parametrize("comp", [False, True])
@pytest.mark.parametrize("rank", [16, 32, 48, 64])
@pytest.mark.parametrize("length,head_dim", [(7, 8), (129, 64), (200, 18)])
def test_rotary_modes_ranks(cuda_mod, comp, rank, length, head_dim):
    """RoVE on every rank and both core modes (tests/cuda/test_fast_path.py:1805-1866); the
    reference bounds the rotary forward and dprojected at 5e-3."""
    case = _random_case(500 + rank + length, 2, length, 2, rank, head_dim, comp=comp, rot=True,
                        batched_table=(length == 129))
    _assert_case(cuda_mod, *case, gproj=5e-3, gpar=5e-4, tag=f"rot comp={comp} r{rank} N{length} d{head_dim}")


@pytest.mark.parametrize("comp", [False, True])
@pytest.mark.parametrize("rank", [16, 32, 48, 64])
@pytest.mark.parametrize("length", [7, 129])
def test_rotary_parameter_gradients_hold_reference_limit(cuda_mod, comp, rank, length):
    """The reference's own RoVE case (tests/cuda/test_fast_path.py:1805-1838): two samples of two heads,
    head dimension 64, random gaps in sample 0, sample 1 empty, positions of sample 1 shifted by 321,
    eta_raw = (0.8, 1.4).  Limits as there: forward and dprojected 5e-3, d_core_base_raw and
    d_eta_raw 5e-4."""
    gen = torch.Generator().manual_seed(277 + rank + length)
    batch, heads, head_dim = 2, 2, 64
    valid = torch.rand(batch, length, generator=gen) > 0.2
    valid[1] = False
    proj = (torch.randn(batch, length, heads * (rank + head_dim), generator=gen) * valid[..., None]).bfloat16()
    base = torch.randn(heads, rank, 0 if comp else rank, generator=gen) * 0.1
    eta_raw = torch.tensor([0.8, 1.4])
    counts = valid.sum(-1).float().clamp_min(1.0)
    positions = torch.arange(length)[None] + torch.tensor([[0], [321]])
    phases = positions[..., None].float() * 10000.0 ** (-torch.arange(0, head_dim, 2).float() / head_dim)
    cos, sin = phases.cos().contiguous(), phases.sin().contiguous()
    dy = (torch.randn(batch, length, heads * head_dim, generator=gen) * valid[..., None]).bfloat16()
    y, _ = _run_fast(cuda_mod, proj, base, eta_raw, counts, cos, sin, dy)
    _assert_case(cuda_mod, proj, base, eta_raw, counts, cos, sin, dy, gproj=5e-3, gpar=5e-4,
                 tag=f"reference RoVE case comp={comp} r{rank} N{length}")
    assert torch.count_nonzero(y[~valid.cuda()]) == 0


@pytest.mark.parametrize("rank,head_dim,length", [(16, 17, 35), (32, 64, 35), (64, 257, 35), (64, 17, 2017)])
def test_masked_rows_and_empty_samples(cuda_mod, rank, head_dim, length):
    """Gapped masks and a fully masked sample (tests/cuda/test_fast_path.py:936-1024)."""
    case = _random_case(97 + rank + head_dim, 2, length, 2, rank, head_dim, masked=True, base_scale=0.05)
    proj, base, eta_raw, counts, cos, sin, dy = case
    _assert_case(cuda_mod, *case, tag=f"masked r{rank} d{head_dim} N{length}")
    y = cuda_mod.fast_mix(proj.cuda(), base.cuda(), eta_raw.cuda(), counts.cuda())
    assert torch.count_nonzero(y[1]) == 0  # all-masked sample: zero rows stay zero


@pytest.mark.parametrize("rel_scale,eta_value,base_scale", [(64.0, 9.5, 4.0), (0.001, -9.5, 0.0), (8.0, 0.3, 1.0)])
def test_numerical_boundaries(cuda_mod, rel_scale, eta_value, base_scale):
    """Strong relations, saturated eta, large core (tests/cuda/test_fast_path.py:1385-1427)."""
    proj, base, eta_raw, counts, cos, sin, dy = _random_case(7, 2, 150, 2, 32, 32, rel_scale=rel_scale,
                                                             base_scale=base_scale)
    eta_raw = torch.full_like(eta_raw, eta_value)
    y, grads = _run_fast(cuda_mod, proj, base, eta_raw, counts, cos, sin, dy)
    ey, eg = _run_oracle(proj, base, eta_raw, counts, cos, sin, dy)
    assert all(torch.isfinite(g).all() for g in grads)
    assert rel_l2(y, ey) <= 1.5e-2
    assert rel_l2(grads[0], eg[0]) <= 3.5e-2
    # the Cayley map of a large core (entries of U up to ~12, J = L L^T + Omega far from the identity) is where an
    # inverse of I + J without row exchanges would lose accuracy first: F against FP64, and the gradients that
    # pass through its adjoint
    _, tape, _ = cuda_mod._mix_forward(proj.cuda(), base.cuda(), eta_raw.cuda(), None, None, None, None)
    torch.cuda.synchronize()
    want_f = O.cayley(O.generator(base.double()))
    errs = {"core_map": rel_l2(tape.core_map, want_f), "dbase": rel_l2(grads[1], eg[1]),
            "deta": rel_l2(grads[2], eg[2])}
    print(f"boundaries rel_scale={rel_scale} eta_raw={eta_value} base_scale={base_scale}",
          {k: f"{v:.2e}" for k, v in errs.items()})
    assert int(tape.core_info.abs().sum()) == 0
    if base_scale > 0:
        assert errs["core_map"] <= 2e-5, errs
        assert errs["dbase"] <= 3e-2, errs
    else:   # U = 0 gives J = I and F = 0 exactly
        assert float(tape.core_map.abs().max()) <= 1e-6
    if abs(eta_value) < 5:   # a saturated eta has a vanishing slope: its gradient is below FP32 resolution
        assert errs["deta"] <= 3e-2, errs


@pytest.mark.parametrize("length", [1, 2, 7, 16, 17])
@pytest.mark.parametrize("rank", [16, 64])
@pytest.mark.parametrize("rel_scale", [1.0, 32.0])
def test_fewer_tokens_than_rank(cuda_mod, length, rank, rel_scale):
    """N <= r, where the reference switches to a token-space system (memsolve/ball/cuda.py:3230-3926; its tests
    use N = 1 and 7, tests/cuda/test_fast_path.py:1805-1838).  Under strong relations (entries of A up to ~100)
    and N < r the rank-space form eta (C - P P^T C) of the output is a small difference of large terms, and so is
    d_eta = <dY, C> - tr dF (the rank-space kernels lose d_eta_raw there: 8e-2 at N = 2, rank 64, relations x 32).
    The library evaluates the eta term in token space for N <= r, so every gradient holds the same limits as at
    long lengths: forward 5e-3, dprojected 5e-3 (3e-2 under strong relations, BF16 storage of large values),
    parameters 3e-2.  N = 17 at rank 16 is the first length of the rank-space path."""
    case = _random_case(3300 + 7 * length + rank, 2, length, 2, rank, 64, rot=True, rel_scale=rel_scale,
                        base_scale=0.3)
    _assert_case(cuda_mod, *case, gproj=5e-3 if rel_scale == 1.0 else 3e-2, gpar=3e-2,
                 tag=f"short N={length} r{rank} relations x{rel_scale}")


@pytest.mark.parametrize("rank,d,length,rot,complement,masked", [
    (32, 64, 32, True, False, False),    # N = r exactly
    (64, 64, 64, True, False, True),     # N = r = 64, padded samples
    (48, 72, 5, False, False, False),    # rank 48, two channel blocks (64 + 8), no rotary
    (16, 130, 9, True, False, True),     # three channel blocks, the last of 2 channels
    (32, 64, 3, True, True, False),      # complement mode: F = 0, the eta term is all there is
    (64, 128, 40, True, True, True),
])
def test_short_sequences_shapes(cuda_mod, rank, d, length, rot, complement, masked):
    """The token-space kernels over the shape envelope of the library: all ranks, head widths that are not a
    multiple of 64, padded samples (counts), complement mode, with and without rotary tables."""
    case = list(_random_case(4100 + rank + d + length, 3, length, 2, rank, d, rot=rot, rel_scale=8.0,
                             base_scale=0.3, comp=complement, masked=masked))
    _assert_case(cuda_mod, *case, gproj=2e-2, gpar=3e-2, tag=f"short shapes r{rank} d{d} N={length}")


def test_correction_term_alone(cuda_mod):
    """mixed - eta*C isolates the compact path, which is only a few percent of `mixed`
    at default initialisation."""
    proj, base, eta_raw, counts, cos, sin, dy = _random_case(11, 1, 1024, 4, 32, 64, rot=True)
    heads, rank, d = 4, 32, 64
    y = cuda_mod.fast_mix(proj.cuda(), base.cuda(), eta_raw.cuda(), rotary_cos=cos.cuda(), rotary_sin=sin.cuda())
    ey = O.fast_mix_frame(proj, base, eta_raw, None, cos, sin)
    eta = O.bounded_eta(eta_raw.double())
    content = proj[..., heads * rank:].double().reshape(1, 1024, heads, d) * eta.view(1, 1, heads, 1)
    content = content.reshape(1, 1024, heads * d)
    got = y.double().cpu() - content
    want = ey - content
    # the BF16 store of `mixed` dominates: its rounding is ~2^-9 of |mixed| ~ 20x the correction
    assert rel_l2(got, want) <= 8e-2


def test_bitwise_repeatability(cuda_mod):
    """Two evaluations give identical bits (fixed-order reductions, no atomics)."""
    proj, base, eta_raw, counts, cos, sin, dy = _random_case(5, 2, 3000, 3, 32, 64, rot=True)
    a = _run_fast(cuda_mod, proj, base, eta_raw, counts, cos, sin, dy)
    b = _run_fast(cuda_mod, proj, base, eta_raw, counts, cos, sin, dy)
    assert torch.equal(a[0], b[0])
    for ga, gb in zip(a[1], b[1]):
        assert torch.equal(ga, gb)


@pytest.mark.parametrize("rank", [32, 64])
def test_bitwise_repeatability_long_sequence(cuda_mod, rank):
    """Twelve forward + backward passes over 32768 rotated tokens (the tcgen05 readout, token backward and, at
    rank 64, statistics kernels, all with TMA-staged rotary rows) give identical bits every time."""
    case = _random_case(23 + rank, 1, 32768, 12, rank, 64, rot=True)
    first = _run_fast(cuda_mod, *case)
    for _ in range(11):
        again = _run_fast(cuda_mod, *case)
        assert torch.equal(again[0], first[0])
        for ga, gb in zip(again[1], first[1]):
            assert torch.equal(ga, gb)


_PLAIN_LAUNCH_CHILD = """
import sys, torch
sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r})
import test_fast_mix_gpu as T
from memsolve_b200.ball import cuda
cuda.load()
out = {{}}
for k, (rank, d, n, rot) in enumerate({cases!r}):
    y, grads = T._run_fast(cuda, *T._random_case(11 + k, 2, n, 3, rank, d, rot=rot))
    out[k] = [y.cpu()] + [g.cpu() for g in grads]
torch.save(out, {path!r})
"""


def test_chained_launches_match_plain_launches(cuda_mod, tmp_path):
    """`ms_mix_forward` / `ms_mix_backward` chain their second and third launch to the kernel before
    (programmatic dependent launch); a child process with MEMSOLVE_NO_CHAIN=1 launches the same kernels
    the plain way and must produce identical bits (TMA kernels, generic kernels, rank 64)."""
    import os
    import subprocess
    import sys
    cases = [(32, 64, 3000, True), (64, 64, 700, False), (16, 24, 130, True), (48, 40, 257, False)]
    here = os.path.dirname(os.path.abspath(__file__))
    path = str(tmp_path / "plain.pt")
    code = _PLAIN_LAUNCH_CHILD.format(root=os.path.dirname(here), tests=here, cases=cases, path=path)
    env = dict(os.environ, MEMSOLVE_NO_CHAIN="1")
    subprocess.run([sys.executable, "-c", code], check=True, env=env, timeout=600)
    plain = torch.load(path)
    for k, (rank, d, n, rot) in enumerate(cases):
        y, grads = _run_fast(cuda_mod, *_random_case(11 + k, 2, n, 3, rank, d, rot=rot))
        mine = [y.cpu()] + [g.cpu() for g in grads]
        for a, b in zip(mine, plain[k]):
            assert torch.equal(a, b), (rank, d, n, rot)


def test_inputs_are_not_mutated(cuda_mod):
    proj, base, eta_raw, counts, cos, sin, dy = _random_case(3, 1, 200, 2, 16, 32, rot=True)
    dev = [t.cuda() for t in (proj, base, eta_raw, cos, sin)]
    keep = [t.clone() for t in dev]
    p = dev[0].requires_grad_()
    y = cuda_mod.fast_mix(p, dev[1], dev[2], rotary_cos=dev[3], rotary_sin=dev[4])
    y.backward(dy.cuda())
    for a, b in zip(dev, keep):
        assert torch.equal(a.detach(), b)


# ---------------------------------------------------------------------------------------
# stage-wise checks straight through ctypes
# ---------------------------------------------------------------------------------------
def _stage_buffers(cuda_mod, proj, base, cos):
    shape, dims = cuda_mod._make_shape(proj, base, cos)
    tape = cuda_mod._alloc_tape(dims, proj.device)
    ws = cuda_mod._workspace(shape, proj.device)
    return shape, dims, tape, ws


@pytest.mark.parametrize("rank,head_dim,length,rot", [(32, 64, 5000, True), (64, 64, 777, False), (16, 24, 130, True),
                                                      (48, 70, 333, True)])
def test_stagewise_forward(cuda_mod, rank, head_dim, length, rot):
    """Statistics <= 1e-5, inverse factor <= 2e-6, coefficients <= 2e-5 against FP64
    (limits of tests/cuda/test_fast_path.py:1752, 2122-2123 for the compact stages)."""
    lib = cuda_mod._LIB
    heads, batch = 2, 2
    proj, base, eta_raw, counts, cos, sin, dy = _random_case(900 + rank, batch, length, heads, rank, head_dim, rot=rot)
    dp, db, de = proj.cuda(), base.cuda(), eta_raw.cuda()
    dcos, dsin = _dev(cos), _dev(sin)
    shape, dims, tape, ws = _stage_buffers(cuda_mod, dp, db, dcos)
    tape_c = tape.as_struct()
    stream = torch.cuda.current_stream().cuda_stream
    packed = torch.empty(lib.ms_packed_stats_floats(ctypes.byref(shape), 0), device="cuda")
    ptr = cuda_mod._ptr
    assert lib.ms_core_forward(ctypes.byref(shape), db.data_ptr(), de.data_ptr(), ctypes.byref(tape_c), stream) == 0
    assert lib.ms_stats_forward(ctypes.byref(shape), dp.data_ptr(), ptr(dcos), ptr(dsin), None, ws.data_ptr(),
                                ws.numel(), packed.data_ptr(), stream) == 0
    assert lib.ms_compact_forward(ctypes.byref(shape), None, ws.data_ptr(), ws.numel(), None,
                                  ctypes.byref(tape_c), stream) == 0
    torch.cuda.synchronize()
    g, q = O.stage_stats(proj, heads, rank, None, cos, sin)
    t, z, f, eta, w = O.stage_compact(g, q, base, eta_raw)
    pk = packed.view(batch * heads, rank * rank + rank * head_dim).cpu()
    got_g = pk[:, : rank * rank].reshape(batch, heads, rank, rank)
    got_q = pk[:, rank * rank:].reshape(batch, heads, rank, head_dim)
    assert rel_l2(got_g, g) <= 1e-5 and rel_l2(got_q, q) <= 1e-5
    assert rel_l2(tape.core_map, f) <= 2e-5
    assert rel_l2(tape.eta, eta) <= 1e-6
    assert int(tape.core_info.abs().sum()) == 0
    assert rel_l2(tape.inverse, t) <= 2e-6
    assert rel_l2(tape.state, z) <= 1e-5
    coeff = tape.coeff.float().sum(dim=2)[..., :head_dim]
    assert rel_l2(coeff, w) <= 2e-5
    # the same compact result from the packed (all-reduce) path
    tape2 = cuda_mod._alloc_tape(dims, dp.device)
    t2c = tape2.as_struct()
    assert lib.ms_core_forward(ctypes.byref(shape), db.data_ptr(), de.data_ptr(), ctypes.byref(t2c), stream) == 0
    assert lib.ms_compact_forward(ctypes.byref(shape), None, None, 0, packed.data_ptr(), ctypes.byref(t2c), stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(tape2.inverse, tape.inverse) and torch.equal(tape2.coeff, tape.coeff)


@pytest.mark.parametrize("rank,head_dim,length", [(32, 64, 5000), (64, 64, 777), (16, 24, 130)])
def test_exchange_entry_points_single_rank(cuda_mod, rank, head_dim, length):
    """ms_stats_exchange with one rank (no peer) must give the library's own reduction of the partials
    bit for bit, forward and adjoint, call after call (both parities of the double buffer);
    ms_peer_sum with one rank leaves the values unchanged."""
    lib = cuda_mod._LIB
    heads, batch = 2, 2
    proj, base, eta_raw, counts, cos, sin, dy = _random_case(70 + rank, batch, length, heads, rank, head_dim, rot=True)
    dp, db, ddy = proj.cuda(), base.cuda(), dy.bfloat16().cuda().contiguous()
    dcos, dsin = _dev(cos), _dev(sin)
    shape, dims, tape, ws = _stage_buffers(cuda_mod, dp, db, dcos)
    stream = torch.cuda.current_stream().cuda_stream
    area_bytes = int(lib.ms_exchange_area_bytes(ctypes.byref(shape)))
    assert area_bytes > 0
    area = torch.zeros(area_bytes // 4 + 64, device="cuda")
    areas = (ctypes.c_void_p * 1)(area.data_ptr())
    for backward in (0, 1, 0, 1, 1, 0):
        want = torch.empty(lib.ms_packed_stats_floats(ctypes.byref(shape), backward), device="cuda")
        got = torch.full_like(want, float("nan"))
        if backward:
            assert lib.ms_stats_backward(ctypes.byref(shape), dp.data_ptr(), ddy.data_ptr(), dcos.data_ptr(),
                                         dsin.data_ptr(), None, ws.data_ptr(), ws.numel(), want.data_ptr(),
                                         stream) == 0
        else:
            assert lib.ms_stats_forward(ctypes.byref(shape), dp.data_ptr(), dcos.data_ptr(), dsin.data_ptr(), None,
                                        ws.data_ptr(), ws.numel(), want.data_ptr(), stream) == 0
        assert lib.ms_stats_exchange(ctypes.byref(shape), backward, ws.data_ptr(), ws.numel(), None, areas,
                                     area_bytes, 1, 0, got.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    # argument checks
    assert lib.ms_stats_exchange(ctypes.byref(shape), 0, ws.data_ptr(), ws.numel(), None, areas, 64, 1, 0,
                                 got.data_ptr(), stream) != 0
    assert lib.ms_stats_exchange(ctypes.byref(shape), 0, ws.data_ptr(), ws.numel(), None, areas, area_bytes, 9, 0,
                                 got.data_ptr(), stream) != 0

    values = torch.randn(4096 + 4 * rank, device="cuda")
    keep = values.clone()
    sum_bytes = int(lib.ms_peer_sum_area_bytes(values.numel()))
    sum_area = torch.zeros(sum_bytes // 4 + 64, device="cuda")
    sum_areas = (ctypes.c_void_p * 1)(sum_area.data_ptr())
    for _ in range(3):
        assert lib.ms_peer_sum(values.data_ptr(), values.numel(), sum_areas, sum_bytes, 1, 0, stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(values, keep)
    assert lib.ms_peer_sum(values.data_ptr(), values.numel() - 1, sum_areas, sum_bytes, 1, 0, stream) != 0
    assert lib.ms_device_error() == 0


def test_peer_wait_runs_out_without_hanging(cuda_mod):
    """A rank whose peer never arrives: `world_size = 2` with both exchange areas in this GPU's memory and
    nobody raising the second rank's flags.  With the wait limit set to 50 ms the kernels must return by
    themselves, record 0x200 in the device error word and hand back NaN instead of partial sums; the next
    call with a peer-free world works again."""
    lib = cuda_mod._LIB
    heads, batch, rank, head_dim, length = 2, 1, 32, 64, 700
    proj, base, eta_raw, counts, cos, sin, dy = _random_case(77, batch, length, heads, rank, head_dim, rot=True)
    dp, db = proj.cuda(), base.cuda()
    dcos, dsin = _dev(cos), _dev(sin)
    shape, dims, tape, ws = _stage_buffers(cuda_mod, dp, db, dcos)
    stream = torch.cuda.current_stream().cuda_stream
    area_bytes = int(lib.ms_exchange_area_bytes(ctypes.byref(shape)))
    mine, absent = (torch.zeros(area_bytes // 4 + 64, device="cuda") for _ in range(2))
    areas = (ctypes.c_void_p * 2)(mine.data_ptr(), absent.data_ptr())
    want = torch.empty(lib.ms_packed_stats_floats(ctypes.byref(shape), 0), device="cuda")
    got = torch.zeros_like(want)
    assert lib.ms_device_error() == 0
    assert lib.ms_set_peer_wait_ms(0) != 0
    assert lib.ms_set_peer_wait_ms(50) == 0
    try:
        assert lib.ms_stats_forward(ctypes.byref(shape), dp.data_ptr(), dcos.data_ptr(), dsin.data_ptr(), None,
                                    ws.data_ptr(), ws.numel(), want.data_ptr(), stream) == 0
        assert lib.ms_stats_exchange(ctypes.byref(shape), 0, ws.data_ptr(), ws.numel(), None, areas, area_bytes,
                                     2, 0, got.data_ptr(), stream) == 0
        torch.cuda.synchronize()        # returns: the wait is bounded
        assert lib.ms_device_error() == 0x200
        assert lib.ms_device_error() == 0        # reading clears the word
        assert torch.isnan(got).all()

        values = torch.randn(1 << 16, device="cuda")
        sum_bytes = int(lib.ms_peer_sum_area_bytes(values.numel()))
        a0, a1 = (torch.zeros(sum_bytes // 4 + 64, device="cuda") for _ in range(2))
        sum_areas = (ctypes.c_void_p * 2)(a0.data_ptr(), a1.data_ptr())
        assert lib.ms_peer_sum(values.data_ptr(), values.numel(), sum_areas, sum_bytes, 2, 0, stream) == 0
        torch.cuda.synchronize()
        assert lib.ms_device_error() == 0x200
        assert torch.isnan(values).all()
    finally:
        assert lib.ms_set_peer_wait_ms(20000) == 0
    # the library is usable afterwards
    solo = torch.zeros(area_bytes // 4 + 64, device="cuda")
    solo_areas = (ctypes.c_void_p * 1)(solo.data_ptr())
    assert lib.ms_stats_exchange(ctypes.byref(shape), 0, ws.data_ptr(), ws.numel(), None, solo_areas, area_bytes,
                                 1, 0, got.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(got, want) and lib.ms_device_error() == 0


def test_fp32_readout_before_rounding(cuda_mod):
    """On an identical BF16 projection the coefficients W in FP32 reproduce the reference's
    frame formulation to <= 1e-4 (the FP32 criterion), checked before the BF16 store by
    evaluating eta*C + A W with the kernel's W on the host."""
    heads, rank, d, n = 3, 32, 64, 4096
    proj, base, eta_raw, counts, cos, sin, dy = _random_case(31, 1, n, heads, rank, d, rot=True)
    dp, db, de = proj.cuda(), base.cuda(), eta_raw.cuda()
    shape, dims, tape, ws = _stage_buffers(cuda_mod, dp, db, cos.cuda())
    mixed = cuda_mod.fast_mix(dp, db, de, rotary_cos=cos.cuda(), rotary_sin=sin.cuda())
    # recover W from a fresh forward tape
    y2, tape, dims = cuda_mod._mix_forward(dp, db, de, None, None, cos.cuda(), sin.cuda())
    torch.cuda.synchronize()
    w = tape.coeff.float().sum(dim=2)[..., :d].cpu()
    y32 = O.stage_readout(proj, w, tape.eta.cpu(), heads, rank, None, cos, sin, dtype=torch.float32)
    want = O.fast_mix_frame(proj, base, eta_raw, None, cos, sin)
    assert rel_l2(y32, want) <= 1e-4
    assert rel_l2(mixed, want) <= 5e-3
    assert torch.equal(mixed, y2)


@pytest.mark.parametrize("rank", [32, 64])
def test_full_size_long_sequence(cuda_mod, rank):
    """One sequence of 32768 tokens, 12 heads of dimension 64, rotary, rank 32 (the headline benchmark shape)
    and rank 64 (one GPU's share of the 262144-token sequence-parallel shape): direct comparison with the
    FP64 oracle at full size, forward and all gradients; parameter gradients to the reference's RoVE limit."""
    heads, d, n = 12, 64, 32768
    gen = torch.Generator().manual_seed(0)
    proj = (torch.randn(1, n, heads * (rank + d), generator=gen) * 0.6).bfloat16()
    base = torch.randn(heads, rank, rank, generator=gen) * 0.1
    eta_raw = torch.full((heads,), 1.4722) + torch.randn(heads, generator=gen) * 0.1
    dy = torch.randn(1, n, heads * d, generator=gen).bfloat16()
    cos, sin = O.rotary_tables(torch.arange(n)[None], head_dim=d, train_length=128, context_length=n)
    _assert_case(cuda_mod, proj, base, eta_raw, None, cos, sin, dy, gproj=5e-3, gpar=5e-4,
                 tag=f"32768 tokens rank {rank}")
    assert cuda_mod._LIB.ms_device_error() == 0


@pytest.mark.parametrize("rank,length", [(32, 32768), (64, 262144)])
def test_full_size_properties(cuda_mod, rank, length):
    """Size-independent properties at the benchmark sizes (32768 tokens at rank 32; the whole 262144-token sequence
    of the sequence-parallel configuration at rank 64, where an FP64 oracle run would take minutes).  For fixed
    relations A the mixer is LINEAR in the content: mix(A, C1 + C2) = mix(A, C1) + mix(A, C2), also through the
    rotation; and with eta -> 1 and a zero core the update vanishes in the limit of weak relations:
    mix(0, C) = eta C.  Limits are those of the BF16 stores (three roundings in the sum: 8e-3)."""
    heads, d = 12, 64
    gen = torch.Generator().manual_seed(length + rank)
    rel = (torch.randn(1, length, heads * rank, generator=gen) * 0.6).bfloat16()
    # contents on a coarse grid, so that C1 + C2 is exact in BF16
    c1 = (torch.randint(-8, 9, (1, length, heads * d), generator=gen).float() / 8).bfloat16()
    c2 = (torch.randint(-8, 9, (1, length, heads * d), generator=gen).float() / 8).bfloat16()
    base = (torch.randn(heads, rank, rank, generator=gen) * 0.1).cuda()
    eta_raw = (torch.full((heads,), 1.4722) + torch.randn(heads, generator=gen) * 0.1).cuda()
    cos, sin = O.rotary_tables(torch.arange(length)[None], head_dim=d, train_length=128, context_length=length)
    cos, sin = cos.cuda(), sin.cuda()

    def mix(content, relations=rel):
        proj = torch.cat([relations, content], dim=-1).cuda().contiguous()
        with torch.no_grad():
            return cuda_mod.fast_mix(proj, base, eta_raw, rotary_cos=cos, rotary_sin=sin).float()

    y1, y2, y12 = mix(c1), mix(c2), mix((c1.float() + c2.float()).bfloat16())
    err = rel_l2(y12, y1 + y2)
    print(f"linearity at {length} tokens, rank {rank}: {err:.2e}")
    assert err <= 8e-3
    y0 = mix(c1, torch.zeros_like(rel))
    eta = O.bounded_eta(eta_raw.double().cpu())
    want = (c1.double().reshape(1, length, heads, d) * eta.view(1, 1, heads, 1)).reshape(1, length, heads * d)
    assert rel_l2(y0.cpu(), want) <= 5e-3
    assert cuda_mod._LIB.ms_device_error() == 0


@pytest.mark.parametrize("rank,length", [(32, 32768), (64, 262144)])
def test_full_size_adjoint_identity(cuda_mod, rank, length):
    """For fixed relations the mixer is a linear map of the content, so forward and backward must be adjoint:
    <mix(A, C), dY> = <C, dC>, with dC the content part of the backward pass for the upstream gradient dY.  With
    dY = mix(A, C) itself both sides are |Y|^2, a sum of 2e7 ... 2e8 positive terms against which the BF16
    rounding of Y and dC averages out: 2e-4 relative."""
    heads, d = 12, 64
    gen = torch.Generator().manual_seed(3 * length + rank)
    proj = (torch.randn(1, length, heads * (rank + d), generator=gen) * 0.6).bfloat16().cuda().requires_grad_()
    base = (torch.randn(heads, rank, rank, generator=gen) * 0.1).cuda()
    eta_raw = (torch.full((heads,), 1.4722) + torch.randn(heads, generator=gen) * 0.1).cuda()
    cos, sin = O.rotary_tables(torch.arange(length)[None], head_dim=d, train_length=128, context_length=length)
    y = cuda_mod.fast_mix(proj, base, eta_raw, rotary_cos=cos.cuda(), rotary_sin=sin.cuda())
    dy = y.detach().clone()
    y.backward(dy)
    content = proj.detach()[..., heads * rank:].double()
    d_content = proj.grad[..., heads * rank:].double()
    left = float((y.detach().double() * dy.double()).sum())
    right = float((content * d_content).sum())
    print(f"adjoint identity at {length} tokens, rank {rank}: {left:.8e} vs {right:.8e} ({abs(left - right) / left:.1e})")
    assert abs(left - right) <= 2e-4 * left
    assert cuda_mod._LIB.ms_device_error() == 0


@pytest.mark.parametrize("batch,length,heads,rank,head_dim,rot", [
    (1, 16 * 37 + 5, 12, 32, 64, True), (3, 197, 6, 32, 64, False), (2, 1000, 3, 64, 128, True),
    (1, 50, 2, 16, 64, True), (2, 4100, 16, 32, 64, True)])
def test_tma_kernel_shapes(cuda_mod, batch, length, heads, rank, head_dim, rot):
    """Shapes that take the TMA kernels (head_dim % 64 == 0, rank 16/32/64): ragged last slice,
    several samples, head groups that do not fit shared memory at once, two channel blocks."""
    case = _random_case(4000 + length, batch, length, heads, rank, head_dim, rot=rot, batched_table=rot and batch > 1)
    _assert_case(cuda_mod, *case, gproj=5e-3 if rot else 3e-2, gpar=5e-4 if rot else 3e-2,
                 tag=f"tma B{batch} N{length} H{heads} r{rank} d{head_dim}")
    assert cuda_mod._LIB.ms_device_error() == 0


@pytest.mark.parametrize("batch,length,heads,rank,head_dim,rot,masked", [
    (40, 197, 4, 32, 64, True, False), (26, 128, 6, 32, 64, False, True), (80, 50, 2, 16, 128, True, True),
    (50, 130, 3, 64, 64, False, False), (150, 7, 1, 32, 64, True, False)])
def test_many_short_sequences(cuda_mod, batch, length, heads, rank, head_dim, rot, masked):
    """At least one (sample, head) system per SM and one token chunk per system: the statistics kernels
    switch to the variant in which every warp reduces one whole system (ragged and empty samples, two
    channel blocks, rank 64 adjoint, fewer tokens than the rank)."""
    case = _random_case(7000 + length, batch, length, heads, rank, head_dim, rot=rot, masked=masked,
                        batched_table=rot and masked)
    _assert_case(cuda_mod, *case, gproj=5e-3 if rot else 3e-2,
                 tag=f"short B{batch} N{length} H{heads} r{rank} d{head_dim}")
    assert cuda_mod._LIB.ms_device_error() == 0


def test_rejects_bad_inputs(cuda_mod):
    proj, base, eta_raw, counts, cos, sin, dy = _random_case(1, 1, 40, 2, 16, 8)
    with pytest.raises(RuntimeError, match="mixed precision CUDA contract"):
        cuda_mod.fast_mix(proj.cuda().float(), base.cuda(), eta_raw.cuda())
    with pytest.raises(RuntimeError, match="rank in"):
        cuda_mod.fast_mix(torch.zeros(1, 40, 2 * 8 + 16, device="cuda", dtype=torch.bfloat16),
                          torch.zeros(2, 8, 8, device="cuda"), eta_raw.cuda())
    with pytest.raises(ValueError, match="supplied together"):
        cuda_mod.fast_mix(proj.cuda(), base.cuda(), eta_raw.cuda(), rotary_cos=torch.zeros(1, 40, 4, device="cuda"))
    lib = cuda_mod._LIB
    shape, dims = cuda_mod._make_shape(proj.cuda(), base.cuda(), None)
    assert lib.ms_stats_forward(ctypes.byref(shape), proj.cuda().data_ptr(), None, None, None, None, 0, None,
                                None) == 3  # MS_ERR_WORKSPACE
