"""Self-contained encoder scaffolds around the MemSolve layer.

The reference ships its vision and masked-language models as adapters on top of timm and
Hugging Face transformers (integrations/timm.py:181-207, 284-334; integrations/transformers.py:
191-223, 298-334).  Neither library is a dependency here, so these two plain `torch.nn` encoders
reproduce what those adapters do around the layer -- and nothing else:

* the activations are cast to the autocast dtype (BF16 without autocast) right before the mixer,
  so that both backends see the same rounding (timm.py:196-198, transformers.py:214-218);
* the padding mask becomes `valid_mask`, and `valid_counts` is computed ONCE per forward and handed
  to every layer (transformers.py:318-321);
* every layer is called as `mixer(x, valid_mask, implementation="cuda", valid_counts=...)`.

`VisionScaffold` is a ViT-Small-shaped classifier (patch 16, 224x224: 196 patch tokens and a class
token, pre-norm blocks, GELU MLP of ratio 4).  `TextScaffold` is a BERT-base-shaped masked-language
model (post-norm blocks, FFN 3072, learned absolute positions, tied decoder).  Everything outside the
mixer is stock PyTorch; the mixer is the sm_100a path of this package.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from ..ball.config import MemSolveConfig
from ..ball.model import MemSolve

__all__ = ["MixerCall", "VisionScaffold", "TextScaffold"]


class MixerCall(nn.Module):
    """One MemSolve layer called the way the reference adapters call it."""

    def __init__(self, dim: int, heads: int, rank: int, *, bias: bool = False, core_mode: str = "equilibrium"):
        super().__init__()
        self.mixer = MemSolve(MemSolveConfig(dim=dim, num_heads=heads, rank=rank, core_mode=core_mode,
                                             bias=bias, rotary=False))

    def forward(self, x: torch.Tensor, valid_mask: torch.Tensor | None = None,
                valid_counts: torch.Tensor | None = None) -> torch.Tensor:
        if x.is_cuda and torch.is_autocast_enabled("cuda"):
            x = x.to(torch.get_autocast_dtype("cuda"))
        elif x.dtype not in (torch.float16, torch.bfloat16):
            x = x.to(torch.bfloat16)
        return self.mixer(x, valid_mask, implementation="cuda", valid_counts=valid_counts)


def _counts(valid_mask: torch.Tensor | None) -> torch.Tensor | None:
    if valid_mask is None:
        return None
    return valid_mask.sum(-1, dtype=torch.float32).clamp_min_(1)


class _Mlp(nn.Module):
    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.up = nn.Linear(dim, hidden)
        self.down = nn.Linear(hidden, dim)

    def forward(self, x):
        return self.down(F.gelu(self.up(x)))


class _PreNormBlock(nn.Module):
    """x + mixer(norm(x)); x + mlp(norm(x)) -- the vision block."""

    def __init__(self, dim, heads, rank, hidden, eps):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim, eps=eps)
        self.attn = MixerCall(dim, heads, rank)
        self.norm2 = nn.LayerNorm(dim, eps=eps)
        self.mlp = _Mlp(dim, hidden)

    def forward(self, x, valid_mask=None, valid_counts=None):
        x = x + self.attn(self.norm1(x), valid_mask, valid_counts).to(x.dtype)
        return x + self.mlp(self.norm2(x))


class VisionScaffold(nn.Module):
    """ViT-Small-shaped classifier: patch embedding, class token, learned positions, pre-norm blocks."""

    def __init__(self, *, image_size: int = 224, patch_size: int = 16, num_classes: int = 1000, dim: int = 384,
                 depth: int = 12, heads: int = 6, rank: int = 32, mlp_ratio: float = 4.0,
                 class_token: bool = True, norm_eps: float = 1e-6):
        super().__init__()
        if image_size % patch_size:
            raise ValueError("image_size must be a multiple of patch_size")
        grid = image_size // patch_size
        self.patch_embed = nn.Conv2d(3, dim, patch_size, stride=patch_size)
        self.cls_token = nn.Parameter(torch.zeros(1, 1, dim)) if class_token else None
        self.tokens = grid * grid + int(class_token)
        self.pos_embed = nn.Parameter(torch.randn(1, self.tokens, dim) * 0.02)
        self.blocks = nn.ModuleList(_PreNormBlock(dim, heads, rank, int(dim * mlp_ratio), norm_eps)
                                    for _ in range(depth))
        self.norm = nn.LayerNorm(dim, eps=norm_eps)
        self.head = nn.Linear(dim, num_classes)

    def forward_features(self, images: torch.Tensor) -> torch.Tensor:
        x = self.patch_embed(images).flatten(2).transpose(1, 2)
        if self.cls_token is not None:
            x = torch.cat([self.cls_token.to(x.dtype).expand(x.shape[0], -1, -1), x], dim=1)
        x = x + self.pos_embed.to(x.dtype)
        for block in self.blocks:
            x = block(x)
        return self.norm(x)

    def forward(self, images: torch.Tensor) -> torch.Tensor:
        x = self.forward_features(images)
        pooled = x[:, 0] if self.cls_token is not None else x.mean(1)
        return self.head(pooled)


class _PostNormBlock(nn.Module):
    """norm(x + dense(mixer(x))); norm(x + ffn(x)) -- the BERT block."""

    def __init__(self, dim, heads, rank, hidden, eps):
        super().__init__()
        self.attention = MixerCall(dim, heads, rank)
        self.attention_out = nn.Linear(dim, dim)
        self.attention_norm = nn.LayerNorm(dim, eps=eps)
        self.ffn = _Mlp(dim, hidden)
        self.ffn_norm = nn.LayerNorm(dim, eps=eps)

    def forward(self, x, valid_mask=None, valid_counts=None):
        mixed = self.attention(x, valid_mask, valid_counts).to(x.dtype)
        x = self.attention_norm(x + self.attention_out(mixed))
        return self.ffn_norm(x + self.ffn(x))


class TextScaffold(nn.Module):
    """BERT-base-shaped masked-language model with the MemSolve layer in place of self-attention."""

    def __init__(self, *, vocab_size: int = 30522, dim: int = 768, depth: int = 12, heads: int = 12,
                 rank: int = 32, ffn: int = 3072, max_positions: int = 512, type_vocab: int = 2,
                 norm_eps: float = 1e-12):
        super().__init__()
        self.word = nn.Embedding(vocab_size, dim)
        self.position = nn.Embedding(max_positions, dim)
        self.token_type = nn.Embedding(type_vocab, dim)
        self.embed_norm = nn.LayerNorm(dim, eps=norm_eps)
        self.blocks = nn.ModuleList(_PostNormBlock(dim, heads, rank, ffn, norm_eps) for _ in range(depth))
        self.head_dense = nn.Linear(dim, dim)
        self.head_norm = nn.LayerNorm(dim, eps=norm_eps)
        self.decoder_bias = nn.Parameter(torch.zeros(vocab_size))

    def encode(self, input_ids: torch.Tensor, attention_mask: torch.Tensor | None = None,
               token_type_ids: torch.Tensor | None = None) -> torch.Tensor:
        if attention_mask is not None and attention_mask.ndim != 2:
            raise ValueError("the text scaffold accepts a 2D padding mask, not pairwise masks")
        batch, length = input_ids.shape
        if length > self.position.num_embeddings:
            raise ValueError("sequence longer than the position table")
        positions = torch.arange(length, device=input_ids.device)[None]
        types = torch.zeros_like(input_ids) if token_type_ids is None else token_type_ids
        x = self.embed_norm(self.word(input_ids) + self.position(positions) + self.token_type(types))
        valid_mask = None if attention_mask is None else attention_mask.to(device=x.device, dtype=torch.bool)
        valid_counts = _counts(valid_mask)
        for block in self.blocks:
            x = block(x, valid_mask, valid_counts)
        return x

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, labels=None):
        """Returns the logits, or the masked-language-model loss when `labels` (-100 = ignored) are given.

        With labels only the target positions go through the vocabulary projection."""
        x = self.encode(input_ids, attention_mask, token_type_ids)
        if labels is None:
            hidden = self.head_norm(F.gelu(self.head_dense(x)))
            return F.linear(hidden, self.word.weight, self.decoder_bias)
        positions = (labels.reshape(-1) != -100).nonzero().squeeze(1)
        return self._loss_at(x, positions, labels.reshape(-1)[positions])

    def _loss_at(self, x, positions, targets):
        hidden = self.head_norm(F.gelu(self.head_dense(x.reshape(-1, x.shape[-1])[positions])))
        logits = F.linear(hidden, self.word.weight, self.decoder_bias)
        return F.cross_entropy(logits.float(), targets)

    def masked_lm_loss(self, input_ids, positions, targets, attention_mask=None, token_type_ids=None):
        """The same loss with the target positions given as flat indices into `[batch * length]` (a tensor
        of fixed size: no host synchronisation, so the step can be captured in a CUDA graph)."""
        return self._loss_at(self.encode(input_ids, attention_mask, token_type_ids), positions, targets)
