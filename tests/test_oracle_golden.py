"""Pin the CPU oracle against vectors produced by the reference implementation."""
from __future__ import annotations

import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import memsolve_oracle as O

MIX_CASES = ["mix_r16_plain", "mix_r32_rot", "mix_r16_comp_rot_mask", "mix_r48_strong",
             "mix_r64_rot_mask", "mix_r16_short"]


def _mix_inputs(g):
    proj = g["projected"].bfloat16()
    return (proj, g["base"], g["eta_raw"], g.get("counts"), g.get("cos"), g.get("sin"), g["dy"])


@pytest.mark.parametrize("name", MIX_CASES)
def test_frame_mix_matches_reference_fp64(name):
    g = load_golden(name + ".npz")
    proj, base, eta_raw, counts, cos, sin, dy = _mix_inputs(g)
    ins = [proj.double().requires_grad_(), base.double().requires_grad_(), eta_raw.double().requires_grad_()]
    y = O.fast_mix_frame(ins[0], ins[1], ins[2], counts, cos, sin)
    assert rel_l2(y, g["y"]) < 1e-12
    wanted = [ins[0], ins[2]] if base.numel() == 0 else ins
    grads = torch.autograd.grad((y * dy.double()).sum(), wanted)
    assert rel_l2(grads[0], g["d_projected"]) < 1e-11
    assert rel_l2(grads[-1], g["d_eta_raw"]) < 1e-11
    if base.numel():
        assert rel_l2(grads[1], g["d_base"]) < 1e-11


@pytest.mark.parametrize("name", MIX_CASES)
def test_rankspace_stages_match_reference_fp64(name):
    """The Cholesky (no-frame) formulation and its analytic backward reproduce the
    reference's frame formulation and autograd gradients."""
    g = load_golden(name + ".npz")
    proj, base, eta_raw, counts, cos, sin, dy = _mix_inputs(g)
    y = O.fast_mix_rankspace(proj, base, eta_raw, counts, cos, sin)
    assert rel_l2(y, g["y"]) < 1e-10
    bw = O.stage_backward(proj, dy, base, eta_raw, counts, cos, sin)
    assert rel_l2(bw["sym_lower_check"], 0.5 * (torch.tril(bw["sym_lower_check"]) * 2)) >= 0  # shape sanity
    assert rel_l2(bw["dprojected"], g["d_projected"]) < 1e-9
    assert rel_l2(bw["d_eta_raw"], g["d_eta_raw"]) < 1e-9
    if base.numel():
        assert rel_l2(bw["d_base"], g["d_base"]) < 1e-9


def test_small_maps_match_reference():
    g = load_golden("small_maps.npz")
    pos = g["pos"]
    c, s = O.rotary_tables(pos, head_dim=64, base=10000.0, train_length=128, context_length=32768, scaling="yarn")
    assert torch.equal(c, g["c1"]) and torch.equal(s, g["s1"])
    c, s = O.rotary_tables(pos, head_dim=24, base=500.0, train_length=64,
                           context_length=torch.tensor([40, 400]), scaling="yarn")
    assert torch.equal(c, g["c2"]) and torch.equal(s, g["s2"])
    c, s = O.rotary_tables(pos, head_dim=8, base=10000.0, train_length=128, context_length=999, scaling="none")
    assert torch.equal(c, g["c3"]) and torch.equal(s, g["s3"])
    assert rel_l2(O.generator(g["raw"]), g["gen"]) < 1e-14
    raw = g["eta_in"].clone().requires_grad_()
    eta = O.bounded_eta(raw)
    assert torch.equal(eta.detach(), g["eta"])
    (de,) = torch.autograd.grad(eta.sum(), raw)
    assert torch.allclose(de, g["deta"], rtol=1e-6, atol=0)
    assert rel_l2(O.soft_frame(g["rel"]), g["frame"]) < 1e-12


def _layer_params(g, dtype):
    meta = g["meta"].tolist()
    dim, heads, rank = meta[0], meta[1], meta[2]
    p = O.LayerParams(
        w_bc=g["p_w_bc_weight"], w_o=g["p_w_o_weight"],
        core_base_raw=g.get("p_core_base_raw"), eta_raw=g["p_eta_raw"],
        b_bc=g.get("p_w_bc_bias"), b_o=g.get("p_w_o_bias"), heads=heads, rank=rank,
    ).to(dtype)
    for t in p.tensors():
        t.requires_grad_()
    return p


@pytest.mark.parametrize("name", ["layer_small_eq", "layer_small_rot", "layer_small_comp"])
@pytest.mark.parametrize("tag", ["f32", "f64"])
def test_layer_matches_reference_module(name, tag):
    g = load_golden(name + ".npz")
    dtype = torch.float64 if tag == "f64" else torch.float32
    p = _layer_params(g, dtype)
    x = g["x"]
    bf16_in = name == "layer_small_rot"
    if tag == "f64":
        x = x.double()
    elif bf16_in:
        x = x.bfloat16()
    x = x.clone().requires_grad_()
    mask = g.get("mask")
    cos, sin = g.get("cos"), g.get("sin")
    if tag == "f64" and cos is not None:
        # the FP64 reference module builds FP64 tables; rebuild them the same way
        n = x.shape[1]
        cos, sin = O.rotary_tables(torch.arange(n)[None], head_dim=p.w_o.shape[0] // p.heads,
                                   context_length=n, dtype=torch.float64)
    y = O.layer_forward(p, x, mask, cos, sin)
    y.backward(g["dout"].to(y.dtype))
    tol = 1e-10 if tag == "f64" else 2e-3
    assert rel_l2(y, g[f"y_{tag}"]) < (1e-10 if tag == "f64" else 1e-2)
    assert rel_l2(x.grad, g[f"dx_{tag}"]) < max(tol, 2e-2 if tag == "f32" else 0)
    names = {"w_bc": "d_w_bc_weight", "w_o": "d_w_o_weight", "eta_raw": "d_eta_raw",
             "core_base_raw": "d_core_base_raw", "b_bc": "d_w_bc_bias", "b_o": "d_w_o_bias"}
    for attr, key in names.items():
        t = getattr(p, attr)
        if t is None:
            continue
        assert rel_l2(t.grad, g[f"{key}_{tag}"]) < (1e-9 if tag == "f64" else 3e-2), attr


def test_layer_config1_matches_reference_module():
    """The reference's CPU-runnable small case: dim 384, 6 heads, rank 32, x [4,196,384] FP32, seed 0."""
    from memsolve_b200 import MemSolve, MemSolveConfig

    g = load_golden("layer_config1.npz")
    torch.manual_seed(0)
    layer = MemSolve(MemSolveConfig(dim=384, num_heads=6, rank=32))
    x = torch.randn(4, 196, 384)
    same = (abs(float(x.double().sum()) - float(g["x_sum"])) < 1e-9
            and abs(float(layer.w_bc.weight.double().abs().sum()) - float(g["w_bc_abs"])) < 1e-9
            and abs(float(layer.w_o.weight.double().abs().sum()) - float(g["w_o_abs"])) < 1e-9)
    if not same:
        pytest.skip("seeded inputs differ from the ones the fixture was made with (different torch RNG)")
    p = O.LayerParams(layer.w_bc.weight, layer.w_o.weight, layer.core_base_raw, layer.eta_raw,
                      heads=6, rank=32)
    y32 = O.layer_forward(p.to(torch.float32), x)
    y64 = O.layer_forward(p.to(torch.float64), x.double())
    assert rel_l2(y64[:, ::4], g["y_f64_sub"]) < 1e-6      # fixture stored as float32
    assert rel_l2(y32[:, ::4], g["y_f32_sub"]) < 5e-3      # both BF16-rounded paths
