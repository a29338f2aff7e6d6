"""Generate golden vectors by running the reference implementation itself.

Run in a container where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/MemSolve

It imports the reference's ``memsolve`` package read-only, evaluates its CPU
path on small seeded cases, and writes ``tests/golden/*.npz``.  The fixtures are
committed; the tests never import the reference.

Every array is stored as float32/float64/bool/int64 (BF16 values are stored as
float32, which holds them exactly).
"""
from __future__ import annotations

import argparse
import copy
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _np(t):
    if t is None:
        return None
    t = t.detach()
    if t.dtype == torch.bfloat16:
        t = t.float()
    return t.cpu().numpy()


def _save(name, **arrays):
    arrays = {k: v for k, v in arrays.items() if v is not None}
    np.savez_compressed(os.path.join(HERE, name), **arrays)
    print("wrote", name, {k: getattr(v, "shape", None) for k, v in arrays.items()})


def fast_mix_cases(ref):
    """FP64 frame-formulation value + gradients of the mix on a packed BF16 projection."""
    from memsolve.ball import reference as R

    def oracle(projected, base, eta_raw, counts, cos, sin):
        # composition used by the reference's own CUDA tests
        projected = projected.double()
        heads, rank = base.shape[:2]
        b, n, w = projected.shape
        dim = w - heads * rank
        cnt = torch.full((b,), float(n), dtype=torch.float64) if counts is None else counts.double()
        rel, con = projected.split((heads * rank, dim), dim=-1)
        rel = rel.view(b, n, heads, rank).transpose(1, 2) / cnt.sqrt().view(b, 1, 1, 1)
        con = con.view(b, n, heads, dim // heads).transpose(1, 2)
        frame = R.qr_soft_frame(rel)
        if cos is None:
            state = frame.mT @ con
            kw = {}
        else:
            cos, sin = cos.double(), sin.double()
            state = frame.mT @ R.rotate_content(con, cos, sin)
            kw = {"rotary_cos": cos, "rotary_sin": sin}
        gen = None if base.numel() == 0 else R.accretive_generator(base.double())
        y = R.accretive_equilibrium_mix(frame, gen, state, con, R.bounded_complement(eta_raw.double()), **kw)
        return y.transpose(1, 2).contiguous().view(b, n, dim)

    cases = [
        # name, B, N, H, r, d, complement, rotary, masked, rel_scale
        ("mix_r16_plain", 2, 40, 2, 16, 8, False, False, False, 1.0),
        ("mix_r32_rot", 1, 67, 2, 32, 16, False, True, False, 1.0),
        ("mix_r16_comp_rot_mask", 2, 33, 1, 16, 6, True, True, True, 1.0),
        ("mix_r48_strong", 1, 70, 1, 48, 10, False, False, False, 8.0),
        ("mix_r64_rot_mask", 2, 90, 2, 64, 12, False, True, True, 1.0),
        ("mix_r16_short", 1, 7, 2, 16, 4, False, True, False, 1.0),
    ]
    for seed, (name, b, n, h, r, d, comp, rot, masked, scale) in enumerate(cases):
        torch.manual_seed(1000 + seed)
        proj = torch.randn(b, n, h * r + h * d)
        proj[..., : h * r] *= scale
        counts = None
        if masked:
            mask = torch.rand(b, n) > 0.3
            mask[-1, n // 2:] = False
            proj = torch.where(mask[:, :, None], proj, torch.zeros_like(proj))
            counts = mask.sum(-1).float().clamp_min(1.0)
        proj = proj.bfloat16()
        base = torch.randn(h, r, 0 if comp else r) * 0.1
        eta_raw = torch.randn(h) * 0.5
        dy = torch.randn(b, n, h * d).bfloat16()
        cos = sin = None
        if rot:
            pos = torch.arange(n)[None]
            cos, sin = R.rotary_position_factors(pos, head_dim=d, base=10000.0, train_length=16,
                                                 context_length=n, scaling="yarn", dtype=torch.float32)
        ins = [proj.double().requires_grad_(), base.double().requires_grad_(), eta_raw.double().requires_grad_()]
        y = oracle(ins[0], ins[1], ins[2], counts, cos, sin)
        if comp:
            gp, ge = torch.autograd.grad((y * dy.double()).sum(), (ins[0], ins[2]))
            gb = torch.zeros_like(base, dtype=torch.float64)
        else:
            gp, gb, ge = torch.autograd.grad((y * dy.double()).sum(), ins)
        _save(name + ".npz", projected=_np(proj), base=_np(base), eta_raw=_np(eta_raw), dy=_np(dy),
              counts=_np(counts), cos=_np(cos), sin=_np(sin), y=_np(y), d_projected=_np(gp),
              d_base=_np(gb), d_eta_raw=_np(ge),
              meta=np.array([b, n, h, r, d, int(comp), int(rot), int(masked)], dtype=np.int64))


def layer_cases(ref):
    """Whole-layer forward/backward through the reference module's own CPU path."""
    from memsolve import MemSolve, MemSolveConfig, CoreMode

    cases = [
        # name, dim, heads, rank, B, N, mode, rotary, bias, masked, dtype
        ("layer_small_eq", 32, 2, 16, 2, 37, "equilibrium", False, True, True, torch.float32),
        ("layer_small_rot", 48, 3, 16, 2, 150, "equilibrium", True, False, False, torch.bfloat16),
        ("layer_small_comp", 32, 2, 16, 1, 50, "complement", True, True, True, torch.float32),
    ]
    for seed, (name, dim, heads, rank, b, n, mode, rot, bias, masked, dt) in enumerate(cases):
        torch.manual_seed(2000 + seed)
        layer = MemSolve(MemSolveConfig(dim=dim, num_heads=heads, rank=rank, core_mode=CoreMode(mode),
                                        rotary=rot, bias=bias))
        with torch.no_grad():
            if layer.core_base_raw is not None:
                layer.core_base_raw.normal_(std=0.1)
            layer.eta_raw.add_(torch.randn(heads) * 0.2)
        x = torch.randn(b, n, dim).to(dt)
        dout = torch.randn(b, n, dim).to(dt)
        mask = None
        if masked:
            mask = torch.rand(b, n) > 0.25
            mask[0, :3] = True
        out = {}
        for tag, mod, xx in (("f32", layer, x), ("f64", copy.deepcopy(layer).double(), x.double())):
            mod.zero_grad(set_to_none=True)
            xin = xx.clone().requires_grad_()
            y = mod(xin, mask, implementation="reference")
            y.backward(dout.to(y.dtype))
            out[f"y_{tag}"] = _np(y)
            out[f"dx_{tag}"] = _np(xin.grad)
            for pname, p in mod.named_parameters():
                out[f"d_{pname.replace('.', '_')}_{tag}"] = _np(p.grad)
        cos, sin = layer._rotary_factors(x, mask, None, None)
        params = {f"p_{k.replace('.', '_')}": _np(v) for k, v in layer.named_parameters()}
        _save(name + ".npz", x=_np(x), dout=_np(dout), mask=_np(mask), cos=_np(cos), sin=_np(sin),
              meta=np.array([dim, heads, rank, b, n, int(mode == "complement"), int(rot), int(bias)], dtype=np.int64),
              **params, **out)

    # the CPU-runnable small case: dim 384, 6 heads, rank 32, x [4,196,384] fp32, seed 0, default init.
    torch.manual_seed(0)
    layer = MemSolve(MemSolveConfig(dim=384, num_heads=6, rank=32))
    x = torch.randn(4, 196, 384)
    with torch.no_grad():
        y = layer(x, implementation="reference")
        y64 = copy.deepcopy(layer).double()(x.double(), implementation="reference")
    # Inputs and weights are reproducible from the seed (same construction order as the
    # reference module); only checksums and a token-subsampled output are stored.
    _save("layer_config1.npz",
          x_sum=np.array(float(x.double().sum())), x_abs=np.array(float(x.double().abs().sum())),
          w_bc_sum=np.array(float(layer.w_bc.weight.double().sum())),
          w_bc_abs=np.array(float(layer.w_bc.weight.double().abs().sum())),
          w_o_sum=np.array(float(layer.w_o.weight.double().sum())),
          w_o_abs=np.array(float(layer.w_o.weight.double().abs().sum())),
          y_f32_sub=_np(y[:, ::4]), y_f64_sub=_np(y64[:, ::4]).astype(np.float32),
          meta=np.array([384, 6, 32, 4, 196], dtype=np.int64))


def table_cases(ref):
    from memsolve.ball import reference as R

    pos = torch.arange(5, 300, 7)[None]
    c1, s1 = R.rotary_position_factors(pos, head_dim=64, base=10000.0, train_length=128,
                                       context_length=32768, scaling="yarn")
    c2, s2 = R.rotary_position_factors(pos, head_dim=24, base=500.0, train_length=64,
                                       context_length=torch.tensor([40, 400]), scaling="yarn")
    c3, s3 = R.rotary_position_factors(pos, head_dim=8, base=10000.0, train_length=128,
                                       context_length=999, scaling="none")
    torch.manual_seed(7)
    raw = torch.randn(3, 16, 16, dtype=torch.float64) * 0.3
    gen = R.accretive_generator(raw)
    eta_in = torch.tensor([-9.5, -1.0, -1e-3, 0.0, 0.4, 3.0, 9.5], dtype=torch.float32, requires_grad=True)
    eta = R.bounded_complement(eta_in)
    (deta,) = torch.autograd.grad(eta.sum(), eta_in)
    rel = torch.randn(2, 2, 30, 16, dtype=torch.float64) * 2.0
    frame = R.qr_soft_frame(rel)
    _save("small_maps.npz", pos=_np(pos), c1=_np(c1), s1=_np(s1), c2=_np(c2), s2=_np(s2), c3=_np(c3), s3=_np(s3),
          raw=_np(raw), gen=_np(gen), eta_in=_np(eta_in), eta=_np(eta), deta=_np(deta),
          rel=_np(rel), frame=_np(frame))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (the directory that holds memsolve/)")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    sys.dont_write_bytecode = True
    import memsolve  # noqa: F401  (the reference package)

    torch.set_num_threads(4)
    fast_mix_cases(memsolve)
    layer_cases(memsolve)
    table_cases(memsolve)


if __name__ == "__main__":
    main()
