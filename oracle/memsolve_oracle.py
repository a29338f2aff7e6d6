"""CPU oracle for the MemSolve layer (TEST INFRASTRUCTURE, not a product path).

This file restates, on plain CPU torch tensors, the algorithm of the reference
PyTorch implementation of the MemSolve token mixer.  It exists only so that the
CUDA kernels can be checked against it and so that the benchmark can time a CPU
baseline.  Nothing in the shipped package imports it; only the tests, the smoke
entry and the benchmark's CPU-baseline / reference arm do.

Parity status: PINNED.  ``tests/golden/*.npz`` were produced by importing the
reference itself (``tests/golden/make_golden.py``) and ``tests/test_oracle_golden.py``
checks every function below against those vectors.

Each function names the reference lines it follows (paths are relative to the
reference project root).

Two families live here:

* the *frame* formulation, which is what the reference's CPU path computes
  (thin QR of ``[A; I]`` -> soft frame ``P``), used for whole-layer parity and for
  the timed CPU baseline;
* the *rank-space* formulation (Cholesky of ``I + A^T A``; no ``N x r`` frame), which
  is what the reference's CUDA path computes, written out stage by stage with its
  analytic backward so that each CUDA kernel has its own check.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

SOFTPLUS_SHIFT = math.log(math.expm1(1.0))  # reference.py:11


def _calc_dtype(t: torch.Tensor) -> torch.dtype:
    # reference.py:14-15
    return torch.float64 if t.dtype == torch.float64 else torch.float32


# ----------------------------------------------------------------------------
# scalar / small maps
# ----------------------------------------------------------------------------
class _Eta(torch.autograd.Function):
    """eta = (1 - eps) tanh(raw) with the exponential-form derivative.

    Follows memsolve/ball/reference.py:392-409.
    """

    @staticmethod
    def forward(ctx, raw):
        ctx.save_for_backward(raw)
        return (1.0 - torch.finfo(raw.dtype).eps) * torch.tanh(raw)

    @staticmethod
    def backward(ctx, g):
        (raw,) = ctx.saved_tensors
        q = torch.exp(-2.0 * raw.abs())
        return g * (1.0 - torch.finfo(raw.dtype).eps) * 4.0 * q / (1.0 + q) ** 2


def bounded_eta(raw: torch.Tensor) -> torch.Tensor:
    """memsolve/ball/reference.py:412-426."""
    return _Eta.apply(raw.to(_calc_dtype(raw)))


def core_factor(raw: torch.Tensor) -> torch.Tensor:
    """L = tril(U,-1) + diag(softplus(diag U + c0)); reference.py:446-449."""
    diag = torch.diagonal(raw, dim1=-2, dim2=-1)
    return torch.tril(raw, -1) + torch.diag_embed(
        torch.nn.functional.softplus(diag + SOFTPLUS_SHIFT)
    )


def generator(raw: torch.Tensor) -> torch.Tensor:
    """J = L L^T + (triu(U,1) - triu(U,1)^T); reference.py:429-454."""
    raw = raw.to(_calc_dtype(raw))
    fac = core_factor(raw)
    up = torch.triu(raw, 1)
    return fac @ fac.mT + (up - up.mT)


def cayley(gen: torch.Tensor) -> torch.Tensor:
    """F = (I + J)^-1 (I - J); reference.py:542-550."""
    eye = torch.eye(gen.shape[-1], dtype=gen.dtype)
    return torch.linalg.solve(eye + gen, eye - gen)


# ----------------------------------------------------------------------------
# rotary value transport
# ----------------------------------------------------------------------------
def rotary_tables(
    positions: torch.Tensor,
    *,
    head_dim: int,
    base: float = 10000.0,
    train_length: int = 128,
    context_length=None,
    scaling: str = "yarn",
    dtype: torch.dtype = torch.float32,
):
    """cos/sin tables [rows, N, head_dim/2]; reference.py:272-313."""
    cd = torch.float64 if dtype == torch.float64 else torch.float32
    half = head_dim // 2
    idx = torch.arange(half, dtype=cd)
    freq = base ** (-2.0 * idx / head_dim)
    if scaling == "yarn":
        if isinstance(context_length, torch.Tensor):
            scale = (context_length.to(cd) / train_length).clamp_min(1.0).reshape(-1, 1)
        else:
            scale = max(1.0, context_length / train_length)
        lo = max(0, math.floor(head_dim * math.log(train_length / (2 * math.pi * 32)) / (2 * math.log(base))))
        hi = min(half - 1, math.ceil(head_dim * math.log(train_length / (2 * math.pi)) / (2 * math.log(base))))
        ramp = ((idx - lo) / max(hi - lo, 1e-4)).clamp(0, 1)
        freq = freq * (1.0 - ramp + ramp / scale)
    elif scaling != "none":
        raise ValueError("rotary scaling must be 'none' or 'yarn'")
    if freq.ndim == 1:
        freq = freq[None]
    ang = positions.to(cd)[..., None] * freq[:, None, :]
    return ang.cos().contiguous(), ang.sin().contiguous()


def rotate(content: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, inverse: bool = False):
    """Adjacent-pair planar rotation of [B,H,N,d]; reference.py:335-350."""
    v = content.to(_calc_dtype(content))
    c, s = cos[:, None], sin[:, None]
    if inverse:
        s = -s
    ev, od = v[..., 0::2], v[..., 1::2]
    return torch.stack((ev * c - od * s, ev * s + od * c), dim=-1).flatten(-2)


# ----------------------------------------------------------------------------
# frame formulation (what the reference CPU path evaluates)
# ----------------------------------------------------------------------------
def soft_frame(relation: torch.Tensor) -> torch.Tensor:
    """P = A R^-1 via a thin QR of [A; I]; reference.py:353-389."""
    v = relation.to(_calc_dtype(relation))
    n, r = v.shape[-2:]
    scale = v.abs().amax(dim=(-2, -1), keepdim=True).clamp_min(1.0).detach()
    eye = torch.eye(r, dtype=v.dtype).expand(v.shape[:-2] + (r, r))
    q, fac = torch.linalg.qr(torch.cat((v / scale, eye / scale), dim=-2), mode="reduced")
    d = torch.diagonal(fac, dim1=-2, dim2=-1)
    sign = torch.where(d < 0, -torch.ones_like(d), torch.ones_like(d)).detach()
    return (q * sign.unsqueeze(-2))[..., :n, :]


def frame_mix(frame, gen, state, content, eta, cos=None, sin=None):
    """Y = eta C + rot^-1(P (F - eta I) Z); reference.py:457-569 (gen None -> F = 0)."""
    h = frame.shape[1]
    e = eta.view(1, h, 1, 1)
    if gen is None:
        compact = -e * state
    else:
        compact = cayley(gen) @ state - e * state
    corr = frame @ compact
    if cos is not None:
        corr = rotate(corr, cos, sin, inverse=True)
    return e * content + corr


def split_projected(projected, heads: int, rank: int):
    """[B,N,H*r+D] -> relation [B,H,N,r], content [B,H,N,d]; model.py:400-408."""
    b, n, w = projected.shape
    dim = w - heads * rank
    rel, con = projected.split((heads * rank, dim), dim=-1)
    rel = rel.reshape(b, n, heads, rank).transpose(1, 2)
    con = con.reshape(b, n, heads, dim // heads).transpose(1, 2)
    return rel, con


def fast_mix_frame(projected, base_raw, eta_raw, counts=None, cos=None, sin=None,
                   dtype: torch.dtype = torch.float64):
    """Frame-formulation value of ``fast_mix`` on a given packed projection.

    Same composition the reference's CUDA tests use as their FP64 oracle
    (tests/cuda/test_fast_path.py:33-82): split, scale by 1/sqrt(n), QR frame,
    Z = P^T rot(C), shared generator, mix, concatenate heads.
    ``base_raw`` with a zero last dimension selects complement mode.
    """
    projected = projected.to(dtype)
    heads, rank = base_raw.shape[:2]
    b, n, w = projected.shape
    cnt = torch.full((b,), float(n), dtype=dtype) if counts is None else counts.to(dtype)
    rel, con = split_projected(projected, heads, rank)
    frame = soft_frame(rel / cnt.sqrt().view(b, 1, 1, 1))
    if cos is not None:
        cos, sin = cos.to(dtype), sin.to(dtype)
        state = frame.mT @ rotate(con, cos, sin)
    else:
        state = frame.mT @ con
    gen = None if base_raw.numel() == 0 else generator(base_raw.to(dtype))
    y = frame_mix(frame, gen, state, con, bounded_eta(eta_raw.to(dtype)), cos, sin)
    return y.transpose(1, 2).reshape(b, n, w - heads * rank)


# ----------------------------------------------------------------------------
# whole layer (projection -> mix -> projection), as the reference CPU path
# ----------------------------------------------------------------------------
@dataclass
class LayerParams:
    """Plain container for one layer's tensors (model.py:44-71)."""

    w_bc: torch.Tensor            # [H*r + D, D]
    w_o: torch.Tensor             # [D, D]
    core_base_raw: torch.Tensor | None  # [H, r, r] or None (complement mode)
    eta_raw: torch.Tensor         # [H]
    b_bc: torch.Tensor | None = None
    b_o: torch.Tensor | None = None
    heads: int = 1
    rank: int = 16

    def to(self, dtype):
        def cv(t):
            return None if t is None else t.detach().to(dtype)
        return LayerParams(cv(self.w_bc), cv(self.w_o), cv(self.core_base_raw), cv(self.eta_raw),
                           cv(self.b_bc), cv(self.b_o), self.heads, self.rank)

    def tensors(self):
        return [t for t in (self.w_bc, self.b_bc, self.w_o, self.b_o, self.core_base_raw, self.eta_raw)
                if t is not None]


def _linear(x, w, b, out_dtype):
    # CPU branch of tensor_core_linear: FP32 (or FP64) matmul, bias, one cast
    # (reference.py:93-94, 262-269).
    cd = torch.float64 if (x.dtype == torch.float64 or w.dtype == torch.float64) else torch.float32
    y = x.to(cd) @ w.to(cd).mT
    if b is not None:
        y = y + b.to(y.dtype)
    return y if out_dtype is None else y.to(out_dtype)


def layer_forward(p: LayerParams, x: torch.Tensor, mask: torch.Tensor | None = None,
                  cos=None, sin=None) -> torch.Tensor:
    """Reference-path layer forward; model.py:358-448 and 594-624.

    For non-FP64 input the packed projection and the mixed readout are rounded to
    BF16 exactly where the reference rounds them (model.py:398, 614-615).
    """
    b, n, _ = x.shape
    fp64 = x.dtype == torch.float64
    cd = torch.float64 if fp64 else torch.float32
    xs = x if mask is None else torch.where(mask[:, :, None], x, torch.zeros_like(x))
    projected = _linear(xs, p.w_bc, p.b_bc, torch.float64 if fp64 else torch.bfloat16)
    rel, con = split_projected(projected, p.heads, p.rank)
    if mask is not None:
        act = mask[:, None, :, None]
        rel = torch.where(act, rel, torch.zeros_like(rel))
        con = torch.where(act, con, torch.zeros_like(con))
    rel, con = rel.to(cd), con.to(cd)
    cnt = (torch.full((b,), float(n), dtype=cd) if mask is None
           else mask.sum(-1).to(cd).clamp_min(1.0))
    frame = soft_frame(rel / cnt.sqrt().view(b, 1, 1, 1))
    moved = con if cos is None else rotate(con, cos.to(cd), sin.to(cd))
    state = frame.mT @ moved
    gen = None if p.core_base_raw is None else generator(p.core_base_raw.to(cd))
    eta = bounded_eta(p.eta_raw.to(cd))
    y = frame_mix(frame, gen, state, con, eta,
                  None if cos is None else cos.to(cd), None if sin is None else sin.to(cd))
    if not fp64:
        y = y.to(torch.bfloat16)
    y = y.transpose(1, 2).reshape(b, n, -1)
    out = _linear(y, p.w_o, p.b_o, x.dtype)
    return out if mask is None else torch.where(mask[:, :, None], out, torch.zeros_like(out))


# ----------------------------------------------------------------------------
# rank-space formulation, stage by stage (what the CUDA path evaluates)
# ----------------------------------------------------------------------------
def stage_stats(projected, heads, rank, counts=None, cos=None, sin=None, dtype=torch.float64):
    """G = A^T A / n, Q = A^T rot(C) / sqrt(n); memsolve/ball/cuda.py:1542-1667, 2058-2090."""
    projected = projected.to(dtype)
    b, n, _ = projected.shape
    cnt = torch.full((b,), float(n), dtype=dtype) if counts is None else counts.to(dtype)
    rel, con = split_projected(projected, heads, rank)
    moved = con if cos is None else rotate(con, cos.to(dtype), sin.to(dtype))
    g = rel.mT @ rel / cnt.view(b, 1, 1, 1)
    q = rel.mT @ moved / cnt.sqrt().view(b, 1, 1, 1)
    return g, q


def stage_compact(g, q, base_raw, eta_raw):
    """T = chol(I+G)^-1 (lower), Z = T Q, F, eta, W = T^T (F - eta I) Z.

    docs/CUDA_CONTRACT.md:21-35; memsolve/ball/cuda.py:2843-2880, 2580-2681.
    """
    dtype = g.dtype
    r = g.shape[-1]
    eye = torch.eye(r, dtype=dtype)
    low = torch.linalg.cholesky(eye + 0.5 * (g + g.mT))
    t = torch.linalg.solve_triangular(low, eye.expand_as(low), upper=False)
    z = t @ q
    eta = bounded_eta(eta_raw.to(dtype))
    if base_raw.numel() == 0:
        f = torch.zeros(base_raw.shape[0], r, r, dtype=dtype)
    else:
        f = cayley(generator(base_raw.to(dtype)))
    m = f - eta.view(-1, 1, 1) * eye
    w = t.mT @ (m @ z)
    return t, z, f, eta, w


def stage_readout(projected, w, eta, heads, rank, counts=None, cos=None, sin=None, dtype=torch.float64):
    """Y = eta C + rot^-1(A_raw W)/sqrt(n); memsolve/ball/cuda.py:1670-1764."""
    projected = projected.to(dtype)
    b, n, width = projected.shape
    cnt = torch.full((b,), float(n), dtype=dtype) if counts is None else counts.to(dtype)
    rel, con = split_projected(projected, heads, rank)
    corr = rel @ w.to(dtype) / cnt.sqrt().view(b, 1, 1, 1)
    if cos is not None:
        corr = rotate(corr, cos.to(dtype), sin.to(dtype), inverse=True)
    y = eta.to(dtype).view(1, heads, 1, 1) * con + corr
    return y.transpose(1, 2).reshape(b, n, width - heads * rank)


def fast_mix_rankspace(projected, base_raw, eta_raw, counts=None, cos=None, sin=None, dtype=torch.float64):
    """Whole rank-space forward; equals ``fast_mix_frame`` in exact arithmetic
    (identity exercised by the reference at tests/core/test_reference.py:777-818)."""
    heads, rank = base_raw.shape[:2]
    g, q = stage_stats(projected, heads, rank, counts, cos, sin, dtype)
    _t, _z, _f, eta, w = stage_compact(g, q, base_raw, eta_raw)
    return stage_readout(projected, w, eta, heads, rank, counts, cos, sin, dtype)


def stage_backward(projected, dy, base_raw, eta_raw, counts=None, cos=None, sin=None, dtype=torch.float64):
    """Analytic rank-space backward, every intermediate returned.

    docs/CUDA_CONTRACT.md:39-50; memsolve/ball/cuda.py:2883-2987 (compact adjoint),
    2306-2343 (core adjoint), 1767-1922 (token pass), 2517-2527 (eta).
    """
    heads, rank = base_raw.shape[:2]
    projected = projected.to(dtype)
    dy = dy.to(dtype)
    b, n, width = projected.shape
    d = (width - heads * rank) // heads
    cnt = torch.full((b,), float(n), dtype=dtype) if counts is None else counts.to(dtype)
    s = 1.0 / cnt.sqrt().view(b, 1, 1, 1)
    if cos is not None:
        cos, sin = cos.to(dtype), sin.to(dtype)
    rel, con = split_projected(projected, heads, rank)
    dyh = dy.reshape(b, n, heads, d).transpose(1, 2)
    g, q = stage_stats(projected, heads, rank, counts, cos, sin, dtype)
    t, z, f, eta, w = stage_compact(g, q, base_raw, eta_raw)
    eye = torch.eye(rank, dtype=dtype)
    m = f - eta.view(-1, 1, 1) * eye
    rdy = dyh if cos is None else rotate(dyh, cos, sin)
    rc = con if cos is None else rotate(con, cos, sin)
    e = s * (rel.mT @ rdy)                       # [B,H,r,d]
    de = (dyh * con).sum(dim=(0, 2, 3))           # [H]
    u = t @ e
    hmat = u @ z.mT
    d_f = hmat.sum(0)
    d_eta = de - torch.diagonal(d_f, dim1=-2, dim2=-1).sum(-1)
    d_q = t.mT @ (m.mT @ u)
    x = -(m @ hmat.mT) - (m.mT @ hmat)
    sym_lower = 0.5 * (torch.tril(x) + torch.tril(x, -1).mT)
    # the reference keeps tril(x)/2 with the diagonal halved again and adds the transpose
    low = torch.tril(x, -1) * 0.5 + torch.diag_embed(torch.diagonal(x, dim1=-2, dim2=-1)) * 0.25
    sym = low + low.mT
    d_g = t.mT @ sym @ t
    out = {"G": g, "Q": q, "T": t, "Z": z, "F": f, "eta": eta, "W": w, "E": e, "de": de,
           "U": u, "H": hmat, "dF": d_f, "dQ": d_q, "dG": d_g, "sym_lower_check": sym_lower}
    # core adjoint
    raw = eta_raw.to(dtype)
    qq = torch.exp(-2.0 * raw.abs())
    out["d_eta_raw"] = d_eta * (1.0 - torch.finfo(dtype).eps) * 4.0 * qq / (1.0 + qq) ** 2
    if base_raw.numel():
        base = base_raw.to(dtype)
        gen = generator(base)
        v = torch.linalg.solve((eye + gen).mT, d_f)
        d_j = -(v @ (f + eye).mT)
        fac = core_factor(base)
        d_l = (d_j + d_j.mT) @ fac
        diag = torch.diagonal(base, dim1=-2, dim2=-1) + SOFTPLUS_SHIFT
        out["d_base"] = (torch.tril(d_l, -1)
                         + torch.diag_embed(torch.diagonal(d_l, dim1=-2, dim2=-1) * torch.sigmoid(diag))
                         + torch.triu(d_j - d_j.mT, 1))
    else:
        # complement mode: F = 0 is not a parameter; d_eta keeps the same trace term
        out["d_base"] = torch.zeros_like(base_raw, dtype=dtype)
    # token pass
    sg = d_g + d_g.mT
    da = s * (s * (rel @ sg) + rdy @ w.mT + rc @ d_q.mT)
    corr = rel @ d_q
    if cos is not None:
        corr = rotate(corr, cos, sin, inverse=True)
    dc = eta.view(1, heads, 1, 1) * dyh + s * corr
    dproj = torch.cat((da.transpose(1, 2).reshape(b, n, heads * rank),
                       dc.transpose(1, 2).reshape(b, n, heads * d)), dim=-1)
    out["dprojected"] = dproj
    return out
