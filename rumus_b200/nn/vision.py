"""Vision layers (reference: rumus/src/nn/{conv,conv_transpose,pool,batch_norm}.rs and
rumus-vision/src/ops.rs).  Checkpoint layouts follow the reference: ``Conv2d.weight`` is 2-D
``[C_out, C_in*K*K]``, ``ConvTranspose2d.weight`` is ``[C_in, C_out*K*K]``, BatchNorm carries
``weight, bias, running_mean, running_var``."""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from ..ops import vision as V
from .modules import Module, _conv_rng, _embed_rng, _uniform


class Conv2d(Module):
    """rumus/src/nn/conv.rs:45-170 (square kernel, stride, padding) + dilation as in the
    vision crate's direct convolution (rumus-vision/src/ops.rs:333-365)."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int, stride: int = 1,
                 padding: int = 0, bias: bool = True, dilation: int = 1, device=None, dtype=None):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding, self.dilation = kernel_size, stride, padding, dilation
        fan_in = in_channels * kernel_size * kernel_size
        bound = math.sqrt(1.0 / fan_in)
        self.weight = nn.Parameter(_uniform((out_channels, fan_in), bound, _conv_rng, device, dtype))
        self.bias = nn.Parameter(_uniform((out_channels,), bound, _conv_rng, device, dtype)) if bias else None

    def weight4d(self):
        k = self.kernel_size
        return self.weight.view(self.out_channels, self.in_channels, k, k)

    def forward(self, x):
        return V.conv2d(x, self.weight4d(), self.bias, self.stride, self.padding, self.dilation)


class ConvTranspose2d(Module):
    """rumus/src/nn/conv_transpose.rs:42-155 — weight ``[C_in, C_out*K*K]``.  (The reference
    breaks the gradient chain here; this implementation is differentiable.)"""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int, stride: int = 1,
                 padding: int = 0, bias: bool = True, device=None, dtype=None):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding = kernel_size, stride, padding
        fan_in = in_channels * kernel_size * kernel_size
        bound = math.sqrt(1.0 / fan_in)
        self.weight = nn.Parameter(_uniform((in_channels, out_channels * kernel_size * kernel_size),
                                            bound, _embed_rng, device, dtype))
        self.bias = nn.Parameter(_uniform((out_channels,), bound, _embed_rng, device, dtype)) if bias else None

    def forward(self, x):
        k = self.kernel_size
        w = self.weight.view(self.in_channels, self.out_channels, k, k)
        return V.conv_transpose2d(x, w, self.bias, self.stride, self.padding)


class MaxPool2d(Module):
    """rumus/src/nn/pool.rs:16-34; overlapping windows and padding are supported
    (the reference requires stride >= kernel)."""

    def __init__(self, kernel_size: int, stride: Optional[int] = None, padding: int = 0):
        super().__init__()
        self.kernel_size, self.stride, self.padding = kernel_size, stride or kernel_size, padding

    def forward(self, x):
        squeeze = x.dim() == 3
        if squeeze:
            x = x.unsqueeze(0)
        y = V.max_pool2d(x, self.kernel_size, self.stride, self.padding)
        return y.squeeze(0) if squeeze else y


class AdaptiveAvgPool2d(Module):
    def __init__(self, output_size):
        super().__init__()
        self.output_size = (output_size, output_size) if isinstance(output_size, int) else tuple(output_size)

    def forward(self, x):
        return V.adaptive_avg_pool2d(x, self.output_size)


class BatchNorm2d(Module):
    """rumus/src/nn/batch_norm.rs:20-124: eps 1e-5, momentum 0.1, running variance is the
    *biased* batch variance (backend/cpu.rs:320-324), running stats stay on the device."""

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1, device=None,
                 dtype=None):
        super().__init__()
        self.num_features, self.eps, self.momentum = num_features, eps, momentum
        self.weight = nn.Parameter(torch.ones(num_features, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(num_features, device=device, dtype=dtype))
        self.register_buffer("running_mean", torch.zeros(num_features, device=device))
        self.register_buffer("running_var", torch.ones(num_features, device=device))

    def forward(self, x, relu: bool = False, residual=None):
        return V.batch_norm2d(x, self.weight, self.bias, self.running_mean, self.running_var,
                              self.training, self.momentum, self.eps, relu=relu, residual=residual)
