"""The mixer as registered torch.library operators: direct calls, operator checks and
torch.compile(fullgraph=True) against the eager path (the reference registers `memsolve::fast_mix_*`
custom ops for the same purpose, memsolve/ball/cuda.py:4164-5003)."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(rank=32, heads=3, d=64, batch=2, length=300, rotary=True, seed=5):
    from memsolve_b200.ball.rotary import rotary_position_factors
    g = torch.Generator().manual_seed(seed)
    projected = (torch.randn(batch, length, heads * (rank + d), generator=g) * 0.5).bfloat16().cuda()
    base = (torch.randn(heads, rank, rank, generator=g) * 0.1).cuda()
    raw = (torch.randn(heads, generator=g) * 0.3).cuda()
    cos = sin = None
    if rotary:
        cos, sin = rotary_position_factors(torch.arange(length, device="cuda")[None], head_dim=d, base=10000.0,
                                           train_length=128, context_length=length, scaling="yarn")
    upstream = torch.randn(batch, length, heads * d, generator=g).bfloat16().cuda()
    return projected, base, raw, cos, sin, upstream


def _grads(fn, projected, base, raw, upstream):
    leaves = [t.detach().clone().requires_grad_() for t in (projected, base, raw)]
    out = fn(*leaves)
    out.backward(upstream)
    return out.detach(), [t.grad for t in leaves]


def test_operator_equals_eager_path():
    from memsolve_b200.ball import cuda
    cuda.load()
    projected, base, raw, cos, sin, upstream = _inputs()
    eager = lambda p, b, r: cuda.fast_mix(p, b, r, rotary_cos=cos, rotary_sin=sin)
    op = lambda p, b, r: torch.ops.memsolve_b200.fast_mix_fwd(p, b, r, None, cos, sin)[0]
    y0, g0 = _grads(eager, projected, base, raw, upstream)
    y1, g1 = _grads(op, projected, base, raw, upstream)
    assert torch.equal(y0, y1)
    for a, b in zip(g0, g1):
        assert torch.equal(a, b)


def test_opcheck():
    from memsolve_b200.ball import cuda
    cuda.load()
    projected, base, raw, cos, sin, _ = _inputs(length=96)
    args = (projected.requires_grad_(), base.requires_grad_(), raw.requires_grad_(), None, cos, sin)
    torch.library.opcheck(torch.ops.memsolve_b200.fast_mix_fwd.default, args,
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))


@pytest.mark.parametrize("rotary", [False, True])
def test_compile_fullgraph_mixer(rotary):
    from memsolve_b200.ball import cuda
    cuda.load()
    projected, base, raw, cos, sin, upstream = _inputs(rotary=rotary)
    counts = torch.full((projected.shape[0],), float(projected.shape[1]), device="cuda")

    def mix(p, b, r):
        return cuda.fast_mix(p, b, r, counts, rotary_cos=cos, rotary_sin=sin)

    compiled = torch.compile(mix, fullgraph=True, backend="aot_eager")
    y0, g0 = _grads(mix, projected, base, raw, upstream)
    y1, g1 = _grads(compiled, projected, base, raw, upstream)
    assert torch.equal(y0, y1)
    for a, b in zip(g0, g1):
        assert torch.equal(a, b)


def test_compile_fullgraph_layer():
    from memsolve_b200 import MemSolve, MemSolveConfig
    from memsolve_b200.ball import cuda
    cuda.load()
    torch.manual_seed(3)
    layer = MemSolve(MemSolveConfig(128, 2, rank=16, rotary=True, recompute_readout=False)).cuda()
    with torch.no_grad():
        layer.core_base_raw.normal_(std=0.1)
    x = torch.randn(2, 200, 128).bfloat16().cuda()
    upstream = torch.randn(2, 200, 128).bfloat16().cuda()
    factors = layer._rotary_factors(x, None, None, None)

    def run(module):
        module.zero_grad(set_to_none=True)
        xin = x.clone().requires_grad_()
        out = module(xin, implementation="cuda", rotary_factors=factors)
        out.backward(upstream)
        return out.detach(), xin.grad, [p.grad.clone() for p in layer.parameters()]

    y0, dx0, g0 = run(layer)
    compiled = torch.compile(layer, fullgraph=True, backend="aot_eager")
    y1, dx1, g1 = run(compiled)
    assert torch.equal(y0, y1) and torch.equal(dx0, dx1)
    for a, b in zip(g0, g1):
        assert torch.equal(a, b)
