"""Vision Transformers as flat, cut-able ``nn.Sequential``s (MoCo-v3 and soft-target KD).

Child granularity follows the reference conversion (`benchmarks/moco-v3/vit_convert.py:36-57`):
patch embedding, class-token concat, position embedding (+ dropout), one child per transformer block,
final norm, class-token selection ("pre-logits"), then the head layers one by one (MoCo: the 3-layer
projector; the online net appends the 2-layer predictor).  MoCo specifics
(`benchmarks/moco-v3/vits.py:39-100`): fixed 2-D sin-cos position embedding, qkv initialised as three
separate xavier-uniform matrices, class token ~ N(0, 1e-6), patch projection xavier-uniform, optional
``stop_grad_conv1``; heads from `benchmarks/moco-v3/moco/builder.py:36-52,124-134` (bias-free Linear + BN
(+ ReLU), last BN without affine).

The reference takes its blocks from ``timm``; these are written here on top of the fused ops of
:mod:`tspipe_b200.ops` (LayerNorm and bias+GELU kernels; attention through
:func:`tspipe_b200.ops.attention.attention`).
"""
from __future__ import annotations

import copy
import math
from collections import OrderedDict
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import fused
from ..ops.attention import attention, packed_attention, project_qkv, qkv_mode
from ..ops.linear import linear


@dataclass
class ViTConfig:
    img_size: int = 224
    patch_size: int = 16
    embed_dim: int = 768
    depth: int = 12
    num_heads: int = 12
    mlp_ratio: float = 4.0
    eps: float = 1e-6
    drop: float = 0.0
    conv_stem: bool = False      # patch embedding by a 4-layer 3x3/2 convolution stem instead of one 16x16/16 conv


CONFIGS = {
    "vit_small": ViTConfig(embed_dim=384, depth=12, num_heads=12),
    "vit_base": ViTConfig(embed_dim=768, depth=12, num_heads=12),
    "vit_large": ViTConfig(embed_dim=1024, depth=24, num_heads=16),
    "vit_huge": ViTConfig(embed_dim=1280, depth=32, num_heads=16, patch_size=14),
    # convolution-stem variants, one transformer block fewer (`benchmarks/moco-v3/vits.py:210-225`)
    "vit_conv_small": ViTConfig(embed_dim=384, depth=11, num_heads=12, conv_stem=True),
    "vit_conv_base": ViTConfig(embed_dim=768, depth=11, num_heads=12, conv_stem=True),
    "vit_tiny_test": ViTConfig(img_size=32, patch_size=8, embed_dim=64, depth=2, num_heads=4),
    "vit_conv_tiny_test": ViTConfig(img_size=32, patch_size=16, embed_dim=64, depth=2, num_heads=4, conv_stem=True),
}


class LayerNorm(nn.LayerNorm):
    def forward(self, x: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        return fused.layer_norm(x, self.weight, self.bias, self.eps)


class PatchEmbed(nn.Module):
    def __init__(self, cfg: ViTConfig, in_chans: int = 3):
        super().__init__()
        self.grid = cfg.img_size // cfg.patch_size
        self.proj = nn.Conv2d(in_chans, cfg.embed_dim, cfg.patch_size, stride=cfg.patch_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        # A p x p / p convolution is a GEMM over non-overlapping patches.  The library's convolution kernels for 3
        # input channels run at a few percent of the machine (2.6 ms for 512 images); one gather of the patches
        # (k order = (kh, kw, c), which is a plain reshape of channels-last images) and a GEMM take a tenth of that.
        if x.is_cuda and x.dim() == 4 and x.shape[2] % self.proj.kernel_size[0] == 0 \
                and x.shape[3] % self.proj.kernel_size[1] == 0:
            b, c, h, w = x.shape
            ph, pw = self.proj.kernel_size
            gh, gw = h // ph, w // pw
            patches = x.permute(0, 2, 3, 1).reshape(b, gh, ph, gw, pw, c).permute(0, 1, 3, 2, 4, 5)
            patches = patches.reshape(b * gh * gw, ph * pw * c)
            wmat = self.proj.weight.permute(0, 2, 3, 1).reshape(self.proj.out_channels, ph * pw * c)
            return F.linear(patches, wmat, self.proj.bias).view(b, gh * gw, self.proj.out_channels)
        return self.proj(x).flatten(2).transpose(1, 2)


class ConvStem(nn.Module):
    """Patch embedding as four ``Conv 3x3 / 2 -> BatchNorm -> ReLU`` layers (widths ``dim/8 .. dim``) and a 1x1
    projection: total stride 16 (`benchmarks/moco-v3/vits.py:91-126`)."""

    def __init__(self, cfg: ViTConfig, in_chans: int = 3):
        super().__init__()
        assert cfg.patch_size == 16 and cfg.embed_dim % 8 == 0, "the convolution stem has stride 16"
        self.grid = cfg.img_size // cfg.patch_size
        layers, cin, cout = [], in_chans, cfg.embed_dim // 8
        for _ in range(4):
            layers += [nn.Conv2d(cin, cout, 3, stride=2, padding=1, bias=False), nn.BatchNorm2d(cout), nn.ReLU()]
            cin, cout = cout, cout * 2
        layers.append(nn.Conv2d(cin, cfg.embed_dim, 1))
        self.proj = nn.Sequential(*layers)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj(x).flatten(2).transpose(1, 2)


class ClsToken(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.cls_token = nn.Parameter(torch.zeros(1, 1, dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.cat((self.cls_token.to(x.dtype).expand(x.shape[0], -1, -1), x), dim=1)


class PosEmbed(nn.Module):
    def __init__(self, n_tokens: int, dim: int, drop: float = 0.0, learnable: bool = True):
        super().__init__()
        self.pos_embed = nn.Parameter(torch.zeros(1, n_tokens, dim), requires_grad=learnable)
        self.pos_drop = nn.Dropout(drop)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.pos_drop(x + self.pos_embed.to(x.dtype))


class Attention(nn.Module):
    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.heads = heads
        self.qkv = nn.Linear(dim, dim * 3)
        self.proj = nn.Linear(dim, dim)

    def forward(self, x: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        b, n, c = x.shape
        if mask is None and x.is_cuda and qkv_mode() == "split":
            q, k, v = project_qkv(x, self.qkv.weight, self.qkv.bias, self.heads)
            o = attention(q, k, v).transpose(1, 2)
            return linear(o.reshape(b, n, c), self.proj.weight, self.proj.bias)
        qkv = linear(x, self.qkv.weight, self.qkv.bias).reshape(b, n, 3, self.heads, c // self.heads)
        o = packed_attention(qkv) if mask is None else None
        if o is None:
            q, k, v = qkv.permute(2, 0, 3, 1, 4)
            o = attention(q, k, v, mask).transpose(1, 2)
        return linear(o.reshape(b, n, c), self.proj.weight, self.proj.bias)


class Mlp(nn.Module):
    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.fc1 = nn.Linear(dim, hidden)
        self.fc2 = nn.Linear(hidden, dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = linear(x, self.fc1.weight, None)
        h = fused.gelu(h, self.fc1.bias)            # bias add fused into the activation kernel
        return linear(h, self.fc2.weight, self.fc2.bias)


class Block(nn.Module):
    def __init__(self, cfg: ViTConfig):
        super().__init__()
        self.norm1 = LayerNorm(cfg.embed_dim, eps=cfg.eps)
        self.attn = Attention(cfg.embed_dim, cfg.num_heads)
        self.norm2 = LayerNorm(cfg.embed_dim, eps=cfg.eps)
        self.mlp = Mlp(cfg.embed_dim, int(cfg.embed_dim * cfg.mlp_ratio))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = x + self.attn(self.norm1(x))
        return x + self.mlp(self.norm2(x))


class PreLogits(nn.Module):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x[:, 0]


def sincos_2d(grid: int, dim: int, temperature: float = 10000.0) -> torch.Tensor:
    assert dim % 4 == 0, "embed dimension must be divisible by 4 for the 2-D sin-cos position embedding"
    gw, gh = torch.meshgrid(torch.arange(grid, dtype=torch.float32), torch.arange(grid, dtype=torch.float32),
                            indexing="ij")
    omega = 1.0 / (temperature ** (torch.arange(dim // 4, dtype=torch.float32) / (dim // 4)))
    ow = gw.flatten()[:, None] * omega[None]
    oh = gh.flatten()[:, None] * omega[None]
    pe = torch.cat([ow.sin(), ow.cos(), oh.sin(), oh.cos()], dim=1)[None]
    return torch.cat([torch.zeros(1, 1, dim), pe], dim=1)


def vit_trunk_children(cfg: ViTConfig, moco_init: bool = True, stop_grad_conv1: bool = False
                       ) -> "OrderedDict[str, nn.Module]":
    ch: "OrderedDict[str, nn.Module]" = OrderedDict()
    pe = ConvStem(cfg) if cfg.conv_stem else PatchEmbed(cfg)
    n_tok = pe.grid * pe.grid + 1
    ch["patch_embed"] = pe
    ch["cls_token"] = ClsToken(cfg.embed_dim)
    ch["pos_embed"] = PosEmbed(n_tok, cfg.embed_dim, cfg.drop, learnable=not moco_init)
    for i in range(cfg.depth):
        ch[f"block{i}"] = Block(cfg)
    ch["norm"] = LayerNorm(cfg.embed_dim, eps=cfg.eps)
    ch["pre_logits"] = PreLogits()
    for name, m in [(n, m) for c in ch.values() for n, m in c.named_modules()]:
        if isinstance(m, nn.Linear):
            if name.endswith("qkv") and moco_init:
                val = math.sqrt(6.0 / float(m.weight.shape[0] // 3 + m.weight.shape[1]))
                nn.init.uniform_(m.weight, -val, val)
            else:
                nn.init.xavier_uniform_(m.weight)
            nn.init.zeros_(m.bias)
    if moco_init:
        nn.init.normal_(ch["cls_token"].cls_token, std=1e-6)
        with torch.no_grad():
            ch["pos_embed"].pos_embed.copy_(sincos_2d(pe.grid, cfg.embed_dim))
        if isinstance(pe, PatchEmbed):       # the convolution stem keeps its default initialisation
            val = math.sqrt(6.0 / float(3 * cfg.patch_size * cfg.patch_size + cfg.embed_dim))
            nn.init.uniform_(pe.proj.weight, -val, val)
            nn.init.zeros_(pe.proj.bias)
            if stop_grad_conv1:
                pe.proj.weight.requires_grad = False
                pe.proj.bias.requires_grad = False
    else:
        nn.init.trunc_normal_(ch["pos_embed"].pos_embed, std=0.02)
        nn.init.trunc_normal_(ch["cls_token"].cls_token, std=0.02)
    return ch


def moco_mlp_children(num_layers: int, input_dim: int, mlp_dim: int, output_dim: int, last_bn: bool = True,
                      prefix: str = "proj") -> "OrderedDict[str, nn.Module]":
    ch: "OrderedDict[str, nn.Module]" = OrderedDict()
    for l in range(num_layers):
        d1 = input_dim if l == 0 else mlp_dim
        d2 = output_dim if l == num_layers - 1 else mlp_dim
        ch[f"{prefix}_fc{l}"] = nn.Linear(d1, d2, bias=False)
        if l < num_layers - 1:
            ch[f"{prefix}_bn{l}"] = nn.BatchNorm1d(d2)
            ch[f"{prefix}_relu{l}"] = nn.ReLU()
        elif last_bn:
            ch[f"{prefix}_bn{l}"] = nn.BatchNorm1d(d2, affine=False)
    return ch


def moco_vit_networks(arch: str = "vit_base", dim: int = 256, mlp_dim: int = 4096, stop_grad_conv1: bool = False
                      ) -> Tuple[nn.Sequential, nn.Sequential, nn.Sequential]:
    """``(base, momentum, predictor)``: ViT + 3-layer projector each, 2-layer predictor for the base
    encoder; the momentum encoder starts as a copy (`benchmarks/moco-v3/moco/builder.py:32-34`)."""
    cfg = CONFIGS[arch]
    ch = vit_trunk_children(cfg, moco_init=True, stop_grad_conv1=stop_grad_conv1)
    ch.update(moco_mlp_children(3, cfg.embed_dim, mlp_dim, dim, True, "proj"))
    base = nn.Sequential(ch)
    momentum = copy.deepcopy(base)
    predictor = nn.Sequential(moco_mlp_children(2, dim, mlp_dim, dim, True, "pred"))
    return base, momentum, predictor


def vit_classifier(arch: str = "vit_base", num_classes: int = 1000) -> nn.Sequential:
    """Supervised ViT (soft-target KD teacher / student, `benchmarks/soft_target/models/vits.py`)."""
    cfg = CONFIGS[arch]
    ch = vit_trunk_children(cfg, moco_init=False)
    ch["head"] = nn.Linear(cfg.embed_dim, num_classes)
    nn.init.zeros_(ch["head"].weight)
    nn.init.zeros_(ch["head"].bias)
    return nn.Sequential(ch)
