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


def test_compile_inference_operator():
    """Traced without gradients the mixer is `memsolve_b200::fast_mix_infer` (no tape kept); same bits as eager."""
    from memsolve_b200.ball import cuda
    cuda.load()
    projected, base, raw, cos, sin, _ = _inputs(length=200)
    torch.library.opcheck(torch.ops.memsolve_b200.fast_mix_infer.default, (projected, base, raw, None, cos, sin),
                          test_utils=("test_schema", "test_faketensor"))

    def mix(p, b, r):
        return cuda.fast_mix(p, b, r, rotary_cos=cos, rotary_sin=sin)

    with torch.no_grad():
        want = mix(projected, base, raw)
        got = torch.compile(mix, fullgraph=True, backend="aot_eager")(projected, base, raw)
    assert torch.equal(want, got)


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


def test_projection_operators_opcheck():
    """`memsolve_b200::tensor_core_linear` and `memsolve_b200::fast_mix_output_linear_fwd` (the reference registers
    `memsolve::tensor_core_linear[_backward]` and `memsolve::fast_mix_output_linear_fwd/_bwd`,
    memsolve/ball/cuda.py:1104-1304, 4422-4882): schema, fake kernels and autograd registration."""
    from memsolve_b200.ball import cuda
    cuda.load()
    g = torch.Generator().manual_seed(2)
    x = torch.randn(200, 128, generator=g).bfloat16().cuda().requires_grad_()
    w = (torch.randn(256, 128, generator=g) * 0.05).cuda().requires_grad_()
    b = torch.randn(256, generator=g).cuda().requires_grad_()
    mask = (torch.rand(200, generator=g) > 0.2).cuda()
    checks = ("test_schema", "test_faketensor", "test_autograd_registration")
    torch.library.opcheck(torch.ops.memsolve_b200.tensor_core_linear.default, (x, w, b, mask, mask, 2),
                          test_utils=checks)
    torch.library.opcheck(torch.ops.memsolve_b200.tensor_core_linear.default, (x, w, None, None, None, 1),
                          test_utils=checks)
    projected, base, raw, cos, sin, _ = _inputs(length=96)
    wo = (torch.randn(128, 3 * 64, generator=g) * 0.05).cuda().requires_grad_()
    bo = torch.randn(128, generator=g).cuda().requires_grad_()
    args = (projected.requires_grad_(), base.requires_grad_(), raw.requires_grad_(), None, cos, sin, wo, bo, None, 2)
    torch.library.opcheck(torch.ops.memsolve_b200.fast_mix_output_linear_fwd.default, args, test_utils=checks)


@pytest.mark.parametrize("bias,masked", [(False, False), (True, True)])
def test_projection_operator_equals_eager_path(bias, masked):
    """The registered projection against the eager autograd nodes: identical bits for the output and all three
    gradients, with and without bias and row masks (which select the fused tcgen05 kernels)."""
    from memsolve_b200.ball import cuda
    cuda.load()
    g = torch.Generator().manual_seed(4)
    x0 = torch.randn(3, 130, 128, generator=g).bfloat16().cuda()
    w0 = (torch.randn(256, 128, generator=g) * 0.05).cuda()
    b0 = torch.randn(256, generator=g).cuda() if bias else None
    mask = (torch.rand(3, 130, generator=g) > 0.2).cuda() if masked else None
    upstream = torch.randn(3, 130, 256, generator=g).bfloat16().cuda()

    def run(traced):
        x, w = x0.clone().requires_grad_(), w0.clone().requires_grad_()
        b = None if b0 is None else b0.clone().requires_grad_()
        if traced:
            flat_mask = None if mask is None else mask.reshape(-1)
            out = torch.ops.memsolve_b200.tensor_core_linear(x.reshape(-1, 128), w, b, flat_mask, flat_mask, 2)
            out = out.reshape(3, 130, 256)
        else:
            out = cuda.tensor_core_linear(x, w, b, output_dtype=torch.bfloat16, output_mask=mask, input_mask=mask)
        out.backward(upstream)
        return [out.detach(), x.grad, w.grad] + ([] if b is None else [b.grad])

    for a, c in zip(run(False), run(True)):
        assert torch.equal(a, c)


@pytest.mark.parametrize("length", [700, 9])
def test_compile_fullgraph_layer_with_readout_recompute(length):
    """A traced layer with recompute_readout=True runs mixer + output projection as one registered operator that
    keeps the compact tape; outputs and gradients equal the eager layer's bit for bit.  Bias on: the projections take
    the fused tcgen05 kernels, which a tracer reaches only through the registered operators."""
    from memsolve_b200 import MemSolve, MemSolveConfig
    from memsolve_b200.ball import cuda
    cuda.load()
    torch.manual_seed(7)
    layer = MemSolve(MemSolveConfig(128, 2, rank=16, rotary=True, bias=True, recompute_readout=True)).cuda()
    with torch.no_grad():
        layer.core_base_raw.normal_(std=0.1)
    x = torch.randn(2, length, 128).bfloat16().cuda()
    upstream = torch.randn(2, length, 128).bfloat16().cuda()
    factors = layer._rotary_factors(x, None, None, None)

    def run(module):
        layer.zero_grad(set_to_none=True)
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
