"""ResNet trunks as flat, cut-able ``nn.Sequential``s, plus the BYOL MLP heads.

Child granularity follows the reference's ``to_sequential`` for BYOL
(`benchmarks/byol/models/resnet_base_network.py:60-77`, head `benchmarks/byol/models/mlp_head.py:4-26`):
stem conv / bn / relu / maxpool, one child per residual block (a block is never cut, so its skip
connection stays inside one stage), global pool, reshape, then the four head layers -
26 children for the ResNet-50 target network and 30 for online + predictor.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Optional

import torch
from torch import nn

from ..ops.conv import conv_bn_act
from ..ops.pool import GlobalAvgPool, MaxPool3x3s2


def _downsample(down: nn.Module, x: torch.Tensor) -> torch.Tensor:
    """The projection shortcut (1x1 convolution + BatchNorm) through the fused convolution path."""
    if isinstance(down, nn.Sequential) and len(down) == 2 and isinstance(down[0], nn.Conv2d):
        return conv_bn_act(down[0], down[1], x)
    return down(x)


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, inplanes: int, planes: int, stride: int = 1, downsample: Optional[nn.Module] = None):
        super().__init__()
        self.conv1 = nn.Conv2d(inplanes, planes, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(planes)
        self.conv2 = nn.Conv2d(planes, planes, 3, stride=stride, padding=1, bias=False)
        self.bn2 = nn.BatchNorm2d(planes)
        self.conv3 = nn.Conv2d(planes, planes * self.expansion, 1, bias=False)
        self.bn3 = nn.BatchNorm2d(planes * self.expansion)
        self.relu = nn.ReLU()
        self.downsample = downsample

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        identity = x if self.downsample is None else _downsample(self.downsample, x)
        out = conv_bn_act(self.conv1, self.bn1, x, relu=True)
        out = conv_bn_act(self.conv2, self.bn2, out, relu=True)
        return conv_bn_act(self.conv3, self.bn3, out, residual=identity, relu=True)


class BasicBlock(nn.Module):
    expansion = 1

    def __init__(self, inplanes: int, planes: int, stride: int = 1, downsample: Optional[nn.Module] = None):
        super().__init__()
        self.conv1 = nn.Conv2d(inplanes, planes, 3, stride=stride, padding=1, bias=False)
        self.bn1 = nn.BatchNorm2d(planes)
        self.conv2 = nn.Conv2d(planes, planes, 3, padding=1, bias=False)
        self.bn2 = nn.BatchNorm2d(planes)
        self.relu = nn.ReLU()
        self.downsample = downsample

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        identity = x if self.downsample is None else _downsample(self.downsample, x)
        out = conv_bn_act(self.conv1, self.bn1, x, relu=True)
        return conv_bn_act(self.conv2, self.bn2, out, residual=identity, relu=True)


class Reshape2d(nn.Module):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x.reshape(x.shape[0], x.shape[1])


_CFG = {"resnet18": (BasicBlock, [2, 2, 2, 2]), "resnet34": (BasicBlock, [3, 4, 6, 3]),
        "resnet50": (Bottleneck, [3, 4, 6, 3]), "resnet101": (Bottleneck, [3, 4, 23, 3]),
        "resnet152": (Bottleneck, [3, 8, 36, 3])}


def resnet_trunk_children(name: str = "resnet50") -> "OrderedDict[str, nn.Module]":
    block, layers = _CFG[name]
    ch: "OrderedDict[str, nn.Module]" = OrderedDict()
    ch["conv1"] = nn.Conv2d(3, 64, 7, stride=2, padding=3, bias=False)
    ch["bn1"] = nn.BatchNorm2d(64)
    ch["relu"] = nn.ReLU()
    ch["maxpool"] = MaxPool3x3s2()
    inplanes = 64
    for li, (planes, n) in enumerate(zip([64, 128, 256, 512], layers)):
        for bi in range(n):
            stride = 2 if (bi == 0 and li > 0) else 1
            down = None
            if stride != 1 or inplanes != planes * block.expansion:
                down = nn.Sequential(nn.Conv2d(inplanes, planes * block.expansion, 1, stride=stride, bias=False),
                                     nn.BatchNorm2d(planes * block.expansion))
            ch[f"layer{li + 1}_{bi}"] = block(inplanes, planes, stride, down)
            inplanes = planes * block.expansion
    ch["avgpool"] = GlobalAvgPool()
    ch["reshape"] = Reshape2d()
    for m in ch.values():
        for mod in m.modules():
            if isinstance(mod, nn.Conv2d):
                nn.init.kaiming_normal_(mod.weight, mode="fan_out", nonlinearity="relu")
    return ch


def trunk_width(name: str) -> int:
    block, _ = _CFG[name]
    return 512 * block.expansion


def mlp_head_children(in_channels: int, hidden: int, out: int, prefix: str = "proj") -> "OrderedDict[str, nn.Module]":
    return OrderedDict([(f"{prefix}_fc1", nn.Linear(in_channels, hidden)), (f"{prefix}_bn", nn.BatchNorm1d(hidden)),
                        (f"{prefix}_relu", nn.ReLU()), (f"{prefix}_fc2", nn.Linear(hidden, out))])


def byol_networks(name: str = "resnet50", hidden: int = 4096, proj: int = 256):
    """``(online, target, predictor)`` as Sequentials; the target starts as a copy of the online net
    (`benchmarks/byol/main.py:62-92`)."""
    import copy
    ch = resnet_trunk_children(name)
    ch.update(mlp_head_children(trunk_width(name), hidden, proj, "proj"))
    online = nn.Sequential(ch)
    target = copy.deepcopy(online)
    predictor = nn.Sequential(mlp_head_children(proj, hidden, proj, "pred"))
    return online, target, predictor
