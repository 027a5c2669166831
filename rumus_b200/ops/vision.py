"""Vision ops: conv2d / conv_transpose2d / max_pool2d / adaptive_avg_pool2d / batch_norm2d.

CPU tensors use PyTorch math (the fp32 reference); CUDA tensors run the kernels in
``csrc/kernels/vision.cu`` (channels-last im2col / col2im around the tcgen05 GEMM with split-K
weight gradients, batch norm, pooling; reference-layout weights).

Reference: rumus-vision/src/ops.rs:56-410 (direct conv fwd / bwd-data / bwd-weight / bias,
max-pool with local argmax), rumus/src/tensor/ops.rs:1010-1233 (im2col conv, pools),
rumus/src/tensor/ops.rs:1840 (batch_norm_2d), :2019 (adaptive_avg_pool2d).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as TF


def _out_size(n, k, s, p, d=1):
    return (n + 2 * p - d * (k - 1) - 1) // s + 1


def conv2d(x, weight, bias=None, stride: int = 1, padding: int = 0, dilation: int = 1):
    """x [B,C,H,W], weight [Cout,Cin,Kh,Kw] (reference public API: rumus-vision/src/ops.rs:333)."""
    if not x.is_cuda:
        return TF.conv2d(x, weight, bias, stride, padding, dilation)
    from .vision_cuda import Conv2dFn
    return Conv2dFn.apply(x, weight, bias, stride, padding, dilation)


def conv_transpose2d(x, weight, bias=None, stride: int = 1, padding: int = 0):
    """x [B,Cin,H,W], weight [Cin,Cout,Kh,Kw]."""
    if not x.is_cuda:
        return TF.conv_transpose2d(x, weight, bias, stride, padding)
    from .vision_cuda import conv_transpose2d_cuda
    return conv_transpose2d_cuda(x, weight, bias, stride, padding)


def max_pool2d(x, kernel_size: int, stride: Optional[int] = None, padding: int = 0):
    stride = stride or kernel_size
    if not x.is_cuda:
        return TF.max_pool2d(x, kernel_size, stride, padding)
    from .vision_cuda import MaxPool2dFn
    return MaxPool2dFn.apply(x, kernel_size, stride, padding)


def adaptive_avg_pool2d(x, output_size: Tuple[int, int]):
    if not x.is_cuda:
        return TF.adaptive_avg_pool2d(x, output_size)
    from .vision_cuda import AdaptiveAvgPool2dFn
    return AdaptiveAvgPool2dFn.apply(x, tuple(output_size))


def batch_norm2d(x, weight, bias, running_mean, running_var, training: bool, momentum: float = 0.1,
                 eps: float = 1e-5, relu: bool = False, residual=None):
    """Batch norm over (B,H,W) per channel, optional fused residual-add and ReLU
    (``y = relu(bn(x) + residual)``).  Running variance uses the biased batch variance like the
    reference (rumus/src/backend/cpu.rs:320-324)."""
    if not x.is_cuda:
        acc = torch.float64 if x.dtype == torch.float64 else torch.float32   # fp64 stays fp64 for finite-difference checks
        xf = x.to(acc)
        if training:
            mean = xf.mean(dim=(0, 2, 3))
            var = xf.var(dim=(0, 2, 3), unbiased=False)
            with torch.no_grad():
                running_mean.mul_(1 - momentum).add_(mean.detach(), alpha=momentum)
                running_var.mul_(1 - momentum).add_(var.detach(), alpha=momentum)
        else:
            mean, var = running_mean, running_var
        y = (xf - mean[None, :, None, None]) * torch.rsqrt(var[None, :, None, None] + eps)
        y = y * weight.to(acc)[None, :, None, None] + bias.to(acc)[None, :, None, None]
        if residual is not None:
            y = y + residual.to(acc)
        if relu:
            y = torch.relu(y)
        return y.to(x.dtype)
    from .vision_cuda import BatchNorm2dFn
    return BatchNorm2dFn.apply(x, weight, bias, running_mean, running_var, training, momentum, eps,
                               relu, residual)
