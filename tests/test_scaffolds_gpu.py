"""The encoder scaffolds (many short sequences around the MemSolve layer): the mixer call at the vision and
text shapes against the CPU oracle, padding behaviour, and one training step of each scaffold."""
from __future__ import annotations

import pytest
import torch

from conftest import rel_l2
from oracle import memsolve_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def scaffolds():
    from memsolve_b200.ball import cuda
    from memsolve_b200.integrations import scaffolds as S
    cuda.load()
    return S


def _oracle_params(mixer):
    m = mixer.mixer
    cfg = m.config
    return O.LayerParams(m.w_bc.weight.detach().cpu().double(), m.w_o.weight.detach().cpu().double(),
                         m.core_base_raw.detach().cpu().double(), m.eta_raw.detach().cpu().double(),
                         heads=cfg.num_heads, rank=cfg.rank)


@pytest.mark.parametrize("batch,tokens,dim,heads,ragged", [(6, 197, 384, 6, False), (5, 128, 768, 12, True)])
def test_mixer_call_matches_oracle(scaffolds, batch, tokens, dim, heads, ragged):
    """Vision shape (197 tokens, 6 heads of 64) and text shape (128 tokens, 12 heads, ragged padding):
    output and all gradients against the FP64 oracle layer; limits 2e-2 (output) and 3e-2 (gradients)."""
    torch.manual_seed(3)
    call = scaffolds.MixerCall(dim, heads, 32).cuda()
    with torch.no_grad():
        call.mixer.core_base_raw.normal_(std=0.1)
    x = torch.randn(batch, tokens, dim).bfloat16()
    dout = torch.randn(batch, tokens, dim).bfloat16()
    mask = None
    if ragged:
        lengths = torch.tensor([tokens, 1, 37, tokens - 1, 64][:batch])
        mask = torch.arange(tokens)[None] < lengths[:, None]
    xg = x.cuda().requires_grad_()
    counts = None if mask is None else mask.cuda().sum(-1, dtype=torch.float32).clamp_min_(1)
    y = call(xg, None if mask is None else mask.cuda(), counts)
    y.backward(dout.cuda())

    p = _oracle_params(call)
    for t in p.tensors():
        t.requires_grad_()
    xo = x.double().requires_grad_()
    yo = O.layer_forward(p, xo, mask)
    yo.backward(dout.double() if mask is None else torch.where(mask[..., None], dout.double(), 0.0))
    assert rel_l2(y.float().cpu(), yo.detach()) <= 2e-2
    if mask is not None:
        assert torch.count_nonzero(y[~mask.cuda()]) == 0
        assert torch.count_nonzero(xg.grad[~mask.cuda()]) == 0
    m = call.mixer
    assert rel_l2(xg.grad.float().cpu(), xo.grad) <= 3e-2
    assert rel_l2(m.w_bc.weight.grad.cpu(), p.w_bc.grad) <= 3e-2
    assert rel_l2(m.w_o.weight.grad.cpu(), p.w_o.grad) <= 3e-2
    assert rel_l2(m.core_base_raw.grad.cpu(), p.core_base_raw.grad) <= 3e-2
    assert rel_l2(m.eta_raw.grad.cpu(), p.eta_raw.grad) <= 3e-2


def test_vision_scaffold_training_step(scaffolds):
    torch.manual_seed(0)
    model = scaffolds.VisionScaffold(image_size=64, num_classes=10, dim=128, depth=2, heads=2, rank=16).cuda()
    assert model.tokens == 17
    images = torch.randn(4, 3, 64, 64, device="cuda")
    labels = torch.randint(0, 10, (4,), device="cuda")
    with torch.autocast("cuda", dtype=torch.bfloat16):
        logits = model(images)
        loss = torch.nn.functional.cross_entropy(logits.float(), labels)
    loss.backward()
    assert logits.shape == (4, 10) and torch.isfinite(loss)
    missing = [n for n, p in model.named_parameters() if p.grad is None or not torch.isfinite(p.grad).all()]
    assert not missing
    # without autocast the mixer still receives BF16 activations
    assert torch.isfinite(model(images)).all()


def test_text_scaffold_padding_and_training_step(scaffolds):
    torch.manual_seed(0)
    model = scaffolds.TextScaffold(vocab_size=500, dim=128, depth=2, heads=2, rank=16, ffn=256,
                                   max_positions=64).cuda()
    gen = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 500, (3, 48), generator=gen).cuda()
    lengths = torch.tensor([48, 20, 33], device="cuda")
    attention = torch.arange(48, device="cuda")[None] < lengths[:, None]
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        first = model.encode(ids, attention)
        other = ids.clone()
        other[~attention] = 7                      # padded positions must not reach the valid ones
        second = model.encode(other, attention)
    assert torch.equal(first[attention], second[attention])
    labels = torch.where(torch.rand(ids.shape, generator=gen).cuda() < 0.3, ids, torch.full_like(ids, -100))
    labels = torch.where(attention, labels, torch.full_like(labels, -100))
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss = model(ids, attention, labels=labels)
    loss.backward()
    assert torch.isfinite(loss)
    missing = [n for n, p in model.named_parameters() if p.grad is None or not torch.isfinite(p.grad).all()]
    assert not missing
    # the same loss with the target positions given as indices (the form a CUDA graph can capture)
    positions = (labels.reshape(-1) != -100).nonzero().squeeze(1)
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        again = model.masked_lm_loss(ids, positions, labels.reshape(-1)[positions], attention)
    assert torch.equal(again, loss.detach())
    with pytest.raises(ValueError, match="2D padding mask"):
        model.encode(ids, attention[:, None, :])
