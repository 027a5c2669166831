"""ResNet-50 (bottleneck blocks [3, 4, 6, 3], BatchNorm) for the data-parallel fp16 configuration.

The reference has the building blocks (Conv2d, BatchNorm2d, MaxPool2d, AdaptiveAvgPool2d,
Linear: rumus/src/nn/) but no ResNet definition; BatchNorm + ReLU (+ residual add) are fused
into one kernel on CUDA.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..nn import AdaptiveAvgPool2d, BatchNorm2d, Conv2d, Flatten, Linear, MaxPool2d, Module


class Bottleneck(Module):
    expansion = 4

    def __init__(self, in_ch: int, width: int, stride: int = 1, device=None, dtype=None):
        super().__init__()
        out_ch = width * self.expansion
        self.conv1 = Conv2d(in_ch, width, 1, 1, 0, bias=False, device=device, dtype=dtype)
        self.bn1 = BatchNorm2d(width, device=device, dtype=dtype)
        self.conv2 = Conv2d(width, width, 3, stride, 1, bias=False, device=device, dtype=dtype)
        self.bn2 = BatchNorm2d(width, device=device, dtype=dtype)
        self.conv3 = Conv2d(width, out_ch, 1, 1, 0, bias=False, device=device, dtype=dtype)
        self.bn3 = BatchNorm2d(out_ch, device=device, dtype=dtype)
        self.downsample = None
        if stride != 1 or in_ch != out_ch:
            self.downsample = nn.ModuleDict({
                "conv": Conv2d(in_ch, out_ch, 1, stride, 0, bias=False, device=device, dtype=dtype),
                "bn": BatchNorm2d(out_ch, device=device, dtype=dtype)})

    def forward(self, x):
        idt = x
        if self.downsample is not None:
            idt = self.downsample["bn"](self.downsample["conv"](x))
        y = self.bn1(self.conv1(x), relu=True)
        y = self.bn2(self.conv2(y), relu=True)
        return self.bn3(self.conv3(y), relu=True, residual=idt)


class ResNet50(Module):
    def __init__(self, num_classes: int = 1000, layers=(3, 4, 6, 3), width: int = 64, device=None,
                 dtype=None):
        super().__init__()
        self.conv1 = Conv2d(3, width, 7, 2, 3, bias=False, device=device, dtype=dtype)
        self.bn1 = BatchNorm2d(width, device=device, dtype=dtype)
        self.maxpool = MaxPool2d(3, 2, 1)
        blocks = []
        in_ch = width
        for i, n in enumerate(layers):
            w = width * (2 ** i)
            for j in range(n):
                blocks.append(Bottleneck(in_ch, w, stride=(2 if (j == 0 and i > 0) else 1),
                                         device=device, dtype=dtype))
                in_ch = w * Bottleneck.expansion
        self.blocks = nn.ModuleList(blocks)
        self.avgpool = AdaptiveAvgPool2d(1)
        self.flatten = Flatten()
        self.fc = Linear(in_ch, num_classes, True, device, dtype)

    def forward(self, x):
        x = self.maxpool(self.bn1(self.conv1(x), relu=True))
        for b in self.blocks:
            x = b(x)
        return self.fc(self.flatten(self.avgpool(x)))
