"""A minimal ViT (timm ``vit_base_patch16_224`` layout: patch embedding, class token, learned
position embedding, pre-norm blocks with fused-qkv attention and a GELU MLP, final norm, linear
head) whose block linears are plain ``nn.Linear`` modules, so that ``replace_layers`` /
``apply_hot`` can swap them for ``HQ_Linear``.  The reference takes this model from timm
(ViT_main.py:250-251); timm is not a dependency here, and the benchmark needs the architecture
with random weights only.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .quant_matmul import HQ_Linear, ddp_ignore_hot_buffers, replace_layers


class Attention(nn.Module):
    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.heads = heads
        self.qkv = nn.Linear(dim, dim * 3)
        self.proj = nn.Linear(dim, dim)

    def forward(self, x):
        B, N, C = x.shape
        qkv = self.qkv(x).reshape(B, N, 3, self.heads, C // self.heads).permute(2, 0, 3, 1, 4)
        out = F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2])
        return self.proj(out.transpose(1, 2).reshape(B, N, C))


class Mlp(nn.Module):
    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.fc1 = nn.Linear(dim, hidden)
        self.act = nn.GELU()
        self.fc2 = nn.Linear(hidden, dim)

    def forward(self, x):
        return self.fc2(self.act(self.fc1(x)))


class Block(nn.Module):
    def __init__(self, dim: int, heads: int, mlp_ratio: float):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim, eps=1e-6)
        self.attn = Attention(dim, heads)
        self.norm2 = nn.LayerNorm(dim, eps=1e-6)
        self.mlp = Mlp(dim, int(dim * mlp_ratio))

    def forward(self, x):
        x = x + self.attn(self.norm1(x))
        return x + self.mlp(self.norm2(x))


class VisionTransformer(nn.Module):
    def __init__(self, img_size=224, patch=16, dim=768, depth=12, heads=12, mlp_ratio=4.0, num_classes=100):
        super().__init__()
        self.patch_embed = nn.Conv2d(3, dim, kernel_size=patch, stride=patch)
        n = (img_size // patch) ** 2
        self.cls_token = nn.Parameter(torch.zeros(1, 1, dim))
        self.pos_embed = nn.Parameter(torch.randn(1, n + 1, dim) * 0.02)
        self.blocks = nn.ModuleList(Block(dim, heads, mlp_ratio) for _ in range(depth))
        self.norm = nn.LayerNorm(dim, eps=1e-6)
        self.head = nn.Linear(dim, num_classes)

    def forward(self, x):
        x = self.patch_embed(x).flatten(2).transpose(1, 2)
        x = torch.cat([self.cls_token.expand(x.shape[0], -1, -1), x], dim=1) + self.pos_embed
        for blk in self.blocks:
            x = blk(x)
        return self.head(self.norm(x)[:, 0])


def vit_base_patch16_224(num_classes: int = 100) -> VisionTransformer:
    return VisionTransformer(num_classes=num_classes)


def apply_hot(model: VisionTransformer) -> int:
    """Swap the block linears (qkv, proj, fc1, fc2 of every block) for ``HQ_Linear`` and give each
    its module path as ``layer_name`` (what ViT_main.py:272-277 does for the whole model); the
    patch embedding and the classification head stay in full precision.  Returns the count."""
    replace_layers(model.blocks, nn.Linear, HQ_Linear)
    count = 0
    for name, layer in model.named_modules():
        if isinstance(layer, HQ_Linear):
            layer.layer_name = name
            count += 1
    ddp_ignore_hot_buffers(model)   # the model may be wrapped in DistributedDataParallel next
    return count
